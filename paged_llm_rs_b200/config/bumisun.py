"""Typed configuration of the Bumisun decoder.

Its config.json is nested: ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``logit_scale`` and a list
``layers`` whose entries give the mixer's kind (``type``: ``attention`` or ``mamba2``), the mixer's sizes and
constants (``mixer``) and the feed-forward (``mlp``: dense, a mixture of experts, or null).  Every size and every
constant that can differ between two models of the design is read here; nothing about a particular model stands
in code.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError, UnsupportedModelError
from .schema import _take
from .surelorn import _obj, _positive


@dataclass(frozen=True)
class SinkAttentionConfig:
    """Grouped-query attention with a capped score, a window that keeps the first tokens and a sink a head."""

    heads: int
    kv_heads: int
    dim: int                   # query / key entries a head
    vdim: int                  # value entries a head
    scale: float               # multiplies q . k
    softcap: float             # score <- softcap * tanh(score / softcap); 0: none
    window: int                # position i sees j when i - j < window ...
    keep_first: int            # ... or j < keep_first (and j <= i)
    rot_dims: int              # leading entries of each head that are rotated; 0: none
    rot_base: float
    v_mix: bool                # values are mixed with those of the first layer that says so

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SinkAttentionConfig":
        heads, kv = _positive(d, "heads"), _positive(d, "kv_heads")
        if heads % kv:
            raise ConfigError(f"{heads} heads do not group over {kv} kv_heads")
        dim = _positive(d, "dim")
        mask = _obj(d, "mask")
        rot = _obj(d, "rot", optional=True)
        rot_dims, rot_base = (_take(rot, "dims", int), _take(rot, "base", float)) if rot is not None else (0, 10000.0)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"rot.dims {rot_dims} must be even and at most dim {dim}")
        if rot_dims and rot_base <= 0:
            raise ConfigError("rot.base must be positive")
        cap = _take(d, "softcap", float, 0.0)
        if cap < 0:
            raise ConfigError("softcap must not be negative")
        return cls(heads=heads, kv_heads=kv, dim=dim, vdim=_positive(d, "vdim"), scale=_take(d, "scale", float), softcap=cap,
                   window=_positive(mask, "size"), keep_first=_take(mask, "keep_first", int, 0), rot_dims=rot_dims,
                   rot_base=rot_base, v_mix=_take(d, "v_mix", bool, False))


@dataclass(frozen=True)
class Mamba2Config:
    """A selective state space with one decay a head (state space duality)."""

    heads: int
    vdim: int           # entries of x a head
    state: int          # rows of a head's state matrix
    groups: int         # groups of heads that share B and C
    conv: int           # taps of the causal convolution
    norm_groups: int    # equal parts the gated output is normed in

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Mamba2Config":
        heads, groups, ng = _positive(d, "heads"), _take(d, "groups", int, 1), _take(d, "norm_groups", int, 1)
        vdim = _positive(d, "vdim")
        if groups < 1 or heads % groups:
            raise ConfigError(f"{heads} heads do not form {groups} groups")
        if ng < 1 or (heads * vdim) % ng:
            raise ConfigError(f"{heads * vdim} inner entries do not form {ng} norm_groups")
        return cls(heads=heads, vdim=vdim, state=_positive(d, "state"), groups=groups, conv=_positive(d, "conv"), norm_groups=ng)


@dataclass(frozen=True)
class ClampedMoeConfig:
    """Experts with the clamped gated activation behind a router that takes the largest logits."""

    experts: int
    top: int
    expert_ff: int
    expert_limit: float
    shared_ff: Optional[int]          # None: no shared expert
    shared_limit: float

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ClampedMoeConfig":
        r, e = _obj(d, "router"), _obj(d, "expert")
        experts, top = _positive(r, "experts"), _positive(r, "top")
        if top > experts:
            raise ConfigError(f"top {top} of {experts} experts")
        shared = _obj(d, "shared", optional=True)
        return cls(experts=experts, top=top, expert_ff=_positive(e, "ff"), expert_limit=_take(e, "limit", float),
                   shared_ff=_positive(shared, "ff") if shared is not None else None,
                   shared_limit=_take(shared, "limit", float) if shared is not None else 0.0)


@dataclass(frozen=True)
class BumisunLayer:
    mixer_kind: str                       # "attention" or "mamba2"
    mixer: object                         # SinkAttentionConfig or Mamba2Config
    mlp_kind: Optional[str]               # "dense", "moe" or None: the layer has no feed-forward
    dense_ff: Optional[int] = None
    moe: Optional[ClampedMoeConfig] = None


_MIXERS = {"attention": SinkAttentionConfig, "mamba2": Mamba2Config}


@dataclass(frozen=True)
class BumisunConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    logit_scale: float
    layers: Tuple[BumisunLayer, ...]
    architecture: str = "Bumisun"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "BumisunConfig":
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
            try:
                mixer = _MIXERS[kind].from_dict(_obj(e, "mixer"))
                mlp = _obj(e, "mlp", optional=True)
                mlp_kind = dense_ff = moe = None
                if mlp is not None:
                    mlp_kind = _take(mlp, "kind", str)
                    if mlp_kind == "dense":
                        dense_ff = _positive(mlp, "ff")
                    elif mlp_kind == "moe":
                        moe = ClampedMoeConfig.from_dict(mlp)
                    else:
                        raise UnsupportedModelError(f"feed-forward kind {mlp_kind!r} is not implemented")
            except ConfigError as err:
                raise ConfigError(f"layers[{i}]: {err}") from None
            layers.append(BumisunLayer(kind, mixer, mlp_kind, dense_ff, moe))
        mixing = [L.mixer for L in layers if L.mixer_kind == "attention" and L.mixer.v_mix]
        if len({(m.kv_heads, m.vdim) for m in mixing}) > 1:
            raise ConfigError("layers that mix values must have the same kv_heads and vdim")
        eps = _take(_obj(d, "norm"), "eps", float)
        if eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {eps}")
        return cls(vocab=_positive(d, "vocab"), width=_positive(d, "width"), norm_eps=eps,
                   residual_mult=_take(d, "residual_mult", float, 1.0), logit_scale=_take(d, "logit_scale", float, 1.0),
                   layers=tuple(layers), architecture=_take(d, "architecture", str, "Bumisun"))
