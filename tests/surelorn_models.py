"""Small Surelorn configurations for the tests, and random weights for them.

Every size differs between the configurations and between the layers of one: heads that do not
divide a kernel's tile, latent widths that are no multiple of a 16-byte vector, query / key and
value sizes that differ, one expert a token and several, groups and none, identity experts and
none, a shared expert and none, a layer without a feed-forward, layers that run another layer's
tensors.  Weights are drawn wide enough that attention and routing decide something: matrices
N(0, 1 / fan_in), gains near one, so activations stay near unit size at every depth.
"""

import json
import os

import torch


def mixer(heads, dim, vdim, kv_rank, q_rank, scale=None):
    return dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank,
                scale=scale if scale is not None else 1.5 / dim ** 0.5)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, identity=0, groups=None, shared=None):
    r = dict(experts=experts, top=top, identity=identity)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    m = dict(kind="moe", router=r, expert=dict(ff=ff))
    if shared:
        m["shared"] = dict(ff=shared)
    return m


def layer(mix, mlp, weights_of=None):
    d = dict(type="latent_attention", mixer=mix, mlp=mlp)
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


_MA, _MB = mixer(3, 16, 24, 40, 24), mixer(4, 8, 8, 24, 16, scale=0.5)
_EA = moe(6, 2, 48, groups=(3, 2), shared=32)
# S: two widths of latent (two cache groups), a layer with no feed-forward, two layers that run earlier layers' tensors
SMALL = dict(architecture="Surelorn", vocab=200, width=64, embedding=dict(scale=4.0), norm=dict(eps=1e-6), layers=[
    layer(_MA, dense(96)), layer(_MB, _EA), layer(_MA, None), layer(_MB, _EA, weights_of=1), layer(_MA, dense(96), weights_of=0)])

# T: five heads, widths that are no multiple of eight, one expert a token with identity experts and no groups, no shared expert
ODD = dict(architecture="Surelorn", vocab=333, width=90, embedding=dict(scale=2.5), norm=dict(eps=1e-5), layers=[
    layer(mixer(5, 12, 6, 36, 20), moe(5, 1, 30, identity=3)),
    layer(mixer(5, 12, 6, 36, 20), dense(50)),
    layer(mixer(2, 10, 14, 36, 12), dense(50))])         # the same latent width under another number of heads

# U: more heads than one CTA's rows, four experts a token out of two kept groups of four, a shared expert of another width
WIDE = dict(architecture="Surelorn", vocab=512, width=128, embedding=dict(scale=8.0), norm=dict(eps=1e-6), layers=[
    layer(mixer(20, 32, 16, 72, 48), moe(14, 4, 64, identity=2, groups=(4, 2), shared=96)),
    layer(mixer(20, 32, 16, 72, 48), moe(14, 4, 64, identity=2, groups=(4, 2), shared=96), weights_of=0)])

# V: sizes the tensor-core kernels take (latent of 128, sixteen heads, widths that are multiples of 128)
TENSOR = dict(architecture="Surelorn", vocab=1024, width=256, embedding=dict(scale=1.0), norm=dict(eps=1e-6), layers=[
    layer(mixer(16, 64, 64, 128, 128), dense(512)),
    layer(mixer(16, 64, 64, 128, 128), moe(8, 2, 128, groups=(2, 1), shared=128))])

CONFIGS = dict(small=SMALL, odd=ODD, wide=WIDE, tensor=TENSOR)


def tensor_shapes(cfg):
    """name -> (shape, kind) with kind "matrix", "gain", "offset" or "table"."""
    D = cfg["width"]
    out = {"embed": ((cfg["vocab"], D), "table"), "head": ((cfg["vocab"], D), "matrix"), "final.norm": ((D,), "gain")}
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        m, p = L["mixer"], f"l{i}"
        A, d, e, r, u = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        out.update({f"{p}.norm1": ((D,), "gain"), f"{p}.mix.dq": ((u, D), "matrix"), f"{p}.mix.dq.norm": ((u,), "gain"),
                    f"{p}.mix.uq": ((A * d, u), "matrix"), f"{p}.mix.dkv": ((r, D), "matrix"), f"{p}.mix.dkv.norm": ((r,), "gain"),
                    f"{p}.mix.uk": ((A * d, r), "matrix"), f"{p}.mix.uv": ((A * e, r), "matrix"), f"{p}.mix.o": ((D, A * e), "matrix")})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        out[f"{p}.norm2"] = ((D,), "gain")

        def ffn(q, ff):
            out.update({f"{q}.gate": ((ff, D), "matrix"), f"{q}.up": ((ff, D), "matrix"), f"{q}.down": ((D, ff), "matrix")})
        if mlp["kind"] == "dense":
            ffn(f"{p}.mlp", mlp["ff"])
        else:
            r_ = mlp["router"]
            total = r_["experts"] + r_.get("identity", 0)
            out[f"{p}.mlp.router"] = ((total, D), "router")
            out[f"{p}.mlp.correction"] = ((total,), "offset")
            for k in range(r_["experts"]):
                ffn(f"{p}.mlp.e{k}", mlp["expert"]["ff"])
            if mlp.get("shared"):
                ffn(f"{p}.mlp.shared", mlp["shared"]["ff"])
    return out


def random_weights(cfg, seed):
    """bfloat16 tensors (what a model file holds), drawn so that nothing is near zero or near a tie."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if kind == "gain":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif kind == "offset":
            t = 0.3 * torch.randn(shape, generator=g)            # as large as the scores it is added to, both signs
        elif kind == "table":
            t = torch.randn(shape, generator=g) / cfg.get("embedding", {}).get("scale", 1.0)
        elif kind == "router":
            t = 2.0 * torch.randn(shape, generator=g) / shape[-1] ** 0.5
        else:
            t = torch.randn(shape, generator=g) / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(folder, name, seed=0, cfg=None):
    """A model folder for configuration ``name``; returns (folder, config dict, float64 weights for the plain implementation)."""
    from paged_llm_rs_b200.weights.safetensors_io import write_safetensors

    cfg = cfg or CONFIGS[name]
    w = random_weights(cfg, seed)
    d = os.path.join(str(folder), f"surelorn_{name}_{seed}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    return d, cfg, {k: v.double() for k, v in w.items()}
