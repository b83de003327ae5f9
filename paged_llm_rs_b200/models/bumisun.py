"""Bumisun, described as parts.

A decoder whose layers are listed in its configuration: each names its mixer (attention with a capped score, a window
that keeps the first tokens, a sink and mixed values; or a Mamba-2 state space) and its feed-forward (a dense gated one
with relu, a mixture of clamped experts behind a router that takes the largest logits, with a gated shared expert, or
none).  The embedding is normed; the residual stream is float32 and every sublayer's output is multiplied by one constant
as it is added (``prenorm_stream32``); the logits are multiplied by another.  Attention layers rotate part of each head;
nothing bounds a request's length but float32 positions (exact up to 2^24).

Tensors: ``embed``, ``embed.norm``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.*`` and
``l<i>.mlp.*`` (see the parts for the leaves).
"""

from __future__ import annotations

from ..config.bumisun import BumisunConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 24      # positions enter the rotation as float32


def describe_bumisun(cfg: BumisunConfig) -> ModelSpec:
    W = cfg.width
    norm = lambda name: PartSpec("rmsnorm_scaled_stream32", dict(width=W, eps=cfg.norm_eps, mult=cfg.residual_mult, leaf=""), name)
    layers, mixing_seen = [], False
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        if L.mixer_kind == "attention":
            mix = None
            if m.v_mix:
                mix, mixing_seen = ("mixed" if mixing_seen else "source"), True
            mixer = PartSpec("sink_window_attention",
                             dict(hidden_size=W, num_heads=m.heads, num_kv_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                                  scale=m.scale, softcap=m.softcap, window=m.window, keep_first=m.keep_first, rot_dims=m.rot_dims,
                                  rot_base=m.rot_base, sink=True, value_mix=mix), f"{p}.mix")
        else:
            mixer = PartSpec("mamba2", dict(hidden_size=W, heads=m.heads, vdim=m.vdim, state=m.state, groups=m.groups, conv=m.conv,
                                            norm_groups=m.norm_groups, eps=cfg.norm_eps), f"{p}.mix")
        norms = {"mixer": norm(f"{p}.norm1")}
        ff = None
        if L.mlp_kind == "dense":
            ff = PartSpec("swiglu_mlp", dict(hidden_size=W, intermediate_size=L.dense_ff, activation="relu",
                                             names=dict(gate="gate", up="up", down="down")), f"{p}.mlp")
        elif L.mlp_kind == "moe":
            e = L.moe
            ff = PartSpec("routed_experts", dict(hidden_size=W, expert_size=e.expert_ff, experts=e.experts, top=e.top,
                                                 correction=False, router_bias=True, activation="clamped", limit=e.expert_limit,
                                                 shared_size=e.shared_ff, shared_activation="clamped", shared_limit=e.shared_limit,
                                                 shared_gate=e.shared_ff is not None), f"{p}.mlp")
        if ff is not None:
            norms["feed_forward"] = norm(f"{p}.norm2")
        layers.append(LayerSpec(block="prenorm_stream32", mixer=mixer, feed_forward=ff, norms=norms, prefix=p))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=W,
        vocab_size=cfg.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("normed_token_embedding", dict(vocab_size=cfg.vocab, hidden_size=W, eps=cfg.norm_eps, leaf="",
                                                          norm="embed.norm"), "embed"),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, hidden_size=W, leaf="", scale=cfg.logit_scale), "head"),
    )


BUMISUN = Architecture(name="Bumisun", parse=BumisunConfig.from_dict, describe=describe_bumisun, aliases=("bumisun",))
register_architecture(BUMISUN)
