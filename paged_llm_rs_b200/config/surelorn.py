"""Typed configuration of the Surelorn decoder.

Its config.json is nested: ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and a
list ``layers`` whose entries give the mixer's kind (``type``), the mixer's sizes
(``mixer``), the feed-forward (``mlp``: dense, a mixture of experts, or null) and,
for a layer that borrows another layer's tensors, ``weights_of``.  Every size and
every constant that can differ between two models of the design is read here;
nothing about a particular model stands in code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError, UnsupportedModelError
from .schema import _take


def _obj(d: Mapping[str, Any], key: str, optional: bool = False) -> Optional[Mapping[str, Any]]:
    v = d.get(key)
    if v is None:
        if optional:
            return None
        raise ConfigError(f"missing object `{key}`")
    if not isinstance(v, Mapping):
        raise ConfigError(f"`{key}` must be an object")
    return v


def _positive(d, key: str) -> int:
    v = _take(d, key, int)
    if v < 1:
        raise ConfigError(f"`{key}` must be at least 1")
    return v


@dataclass(frozen=True)
class LatentAttentionConfig:
    """Attention whose keys and values are made per head from one cached latent row a token."""

    heads: int
    dim: int          # query / key dimensions a head
    vdim: int         # value dimensions a head
    kv_rank: int      # width of the cached latent
    q_rank: int       # width of the queries' latent
    scale: float      # multiplies q . k

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LatentAttentionConfig":
        return cls(heads=_positive(d, "heads"), dim=_positive(d, "dim"), vdim=_positive(d, "vdim"),
                   kv_rank=_positive(d, "kv_rank"), q_rank=_positive(d, "q_rank"), scale=_take(d, "scale", float))


@dataclass(frozen=True)
class RoutedConfig:
    """A mixture of gated feed-forward experts with a softmax router."""

    experts: int              # experts with tensors
    identity: int             # further router outputs whose expert is the identity
    top: int                  # experts a token uses
    group_count: int          # equal groups of neighbouring router outputs
    group_keep: int           # groups a token may choose from
    expert_ff: int
    shared_ff: Optional[int]  # inner width of the expert every token uses, None: there is none

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RoutedConfig":
        r = _obj(d, "router")
        experts, identity, top = _positive(r, "experts"), _take(r, "identity", int, 0), _positive(r, "top")
        g = _obj(r, "groups", optional=True)
        count, keep = (_positive(g, "count"), _positive(g, "keep")) if g is not None else (1, 1)
        total = experts + identity
        if total % count:
            raise ConfigError(f"{total} router outputs do not form {count} equal groups")
        if keep > count:
            raise ConfigError(f"groups.keep {keep} exceeds groups.count {count}")
        if top > keep * (total // count):
            raise ConfigError(f"top {top} experts cannot come from {keep} groups of {total // count}")
        shared = _obj(d, "shared", optional=True)
        return cls(experts=experts, identity=identity, top=top, group_count=count, group_keep=keep,
                   expert_ff=_positive(_obj(d, "expert"), "ff"),
                   shared_ff=_positive(shared, "ff") if shared is not None else None)


@dataclass(frozen=True)
class SurelornLayer:
    mixer_kind: str
    mixer: LatentAttentionConfig
    mlp_kind: Optional[str]           # "dense", "moe" or None: the layer has no feed-forward
    dense_ff: Optional[int] = None
    routed: Optional[RoutedConfig] = None
    weights_of: Optional[int] = None  # the layer whose tensors this one uses


_MIXERS = {"latent_attention": LatentAttentionConfig}


@dataclass(frozen=True)
class SurelornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[SurelornLayer, ...]
    architecture: str = "Surelorn"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SurelornConfig":
        entries = d.get("layers")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("`layers` must list at least one layer")
        layers = []
        for i, e in enumerate(entries):
            if not isinstance(e, Mapping):
                raise ConfigError(f"layers[{i}] must be an object")
            kind = _take(e, "type", str)
            if kind not in _MIXERS:
                raise UnsupportedModelError(f"layers[{i}]: mixer type {kind!r} is not implemented; known: {sorted(_MIXERS)}")
            mixer = _MIXERS[kind].from_dict(_obj(e, "mixer"))
            mlp = _obj(e, "mlp", optional=True)
            mlp_kind = dense_ff = routed = None
            if mlp is not None:
                mlp_kind = _take(mlp, "kind", str)
                if mlp_kind == "dense":
                    dense_ff = _positive(mlp, "ff")
                elif mlp_kind == "moe":
                    routed = RoutedConfig.from_dict(mlp)
                else:
                    raise UnsupportedModelError(f"layers[{i}]: feed-forward kind {mlp_kind!r} is not implemented")
            src = e.get("weights_of")
            if src is not None:
                src = _take(e, "weights_of", int)
                if src >= i or layers[src].weights_of is not None:
                    raise ConfigError(f"layers[{i}].weights_of must name an earlier layer with tensors of its own")
            layers.append(SurelornLayer(kind, mixer, mlp_kind, dense_ff, routed, src))
        eps = _take(_obj(d, "norm"), "eps", float)
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        width = _positive(d, "width")
        if width % 2:
            raise ConfigError(f"width {width} must be even: the position vector pairs a sine with a cosine")
        emb = _obj(d, "embedding", optional=True) or {}
        return cls(vocab=_positive(d, "vocab"), width=width, embedding_scale=_take(emb, "scale", float, 1.0),
                   norm_eps=eps, layers=tuple(layers), architecture=_take(d, "architecture", str, "Surelorn"))
