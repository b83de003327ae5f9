"""Surelorn, described as parts.

A decoder whose layers are listed in its configuration: each names its mixer (latent
attention), its feed-forward (a dense gated one, a mixture of experts, or none) and, when it
borrows them, the layer whose tensors it uses: such a layer is another RUN of that layer in
the schedule, with a cache of its own.  The residual stream is float32; each sublayer reads
the stream itself and its output is RMS-normed before it is added (``outnorm_residual``).
The embedding is scaled and a sinusoidal position vector is added behind it; mixers have no
position encoding of their own, so nothing bounds a request's length but the float32
positions (exact up to 2^24).

Tensors: ``embed``, ``head``, ``final.norm``, and per layer i with tensors of its own
``l<i>.norm1|norm2`` and ``l<i>.mix.*`` / ``l<i>.mlp.*`` (see the parts for the leaves).
"""

from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.surelorn import SurelornConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24      # positions enter the position vector as float32


def describe_surelorn(cfg: SurelornConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda name: PartSpec("rmsnorm_stream32", dict(width=W, eps=cfg.norm_eps, leaf=""), name)
    layers, index_of = [], {}
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        p = f"l{i}"
        m = L.mixer
        mixer = PartSpec(L.mixer_kind, dict(hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, q_rank=m.q_rank,
                                            kv_rank=m.kv_rank, scale=m.scale, eps=cfg.norm_eps), f"{p}.mix")
        norms = {"mixer": norm(f"{p}.norm1")}
        ff = None
        if L.mlp_kind == "dense":
            ff = PartSpec("swiglu_mlp", dict(hidden_size=W, intermediate_size=L.dense_ff,
                                             names=dict(gate="gate", up="up", down="down")), f"{p}.mlp")
        elif L.mlp_kind == "moe":
            r = L.routed
            ff = PartSpec("routed_experts", dict(hidden_size=W, expert_size=r.expert_ff, experts=r.experts, identity=r.identity,
                                                 top=r.top, groups=r.group_count, keep=r.group_keep, shared_size=r.shared_ff),
                          f"{p}.mlp")
        if ff is not None:
            norms["feed_forward"] = norm(f"{p}.norm2")
        index_of[i] = len(layers)
        layers.append(LayerSpec(block="outnorm_residual", mixer=mixer, feed_forward=ff, norms=norms, prefix=p))
    schedule = [ScheduleEntry(index_of[i if L.weights_of is None else L.weights_of]) for i, L in enumerate(cfg.layers)]
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=W, scale=cfg.embedding_scale,
                                                   stream="float32", leaf=""), "embed"),
        layers=layers,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, hidden_size=W, leaf=""), "head"),
        position_encodings={"sinusoidal": PartSpec("sinusoidal", dict(width=W, base=10000.0))},
    )


SURELORN = Architecture(name="Surelorn", parse=SurelornConfig.from_dict, describe=describe_surelorn, aliases=("surelorn",))
register_architecture(SURELORN)
