"""Small Bumisun configurations for the tests, and random weights for them.

Sizes differ between the configurations and between the layers of one: head counts that do not divide a kernel's
tile, key and value sizes that differ and that are no multiple of a 16-byte vector, windows shorter than a page and
longer than the prompt, no kept tokens and several pages of them, rotation of a whole head and of none, several
convolution widths, state groups and norm groups, one expert a token and several, a shared expert and none, a layer
without a feed-forward, models of one mixer kind only.  Weights are drawn so that attention, the recurrence and the
routing all decide something: matrices N(0, 1 / fan_in), gains near one, sinks and biases of the size of the scores.
With ``calm_router`` the router's matrix is drawn small and its bias holds well separated values: every token then takes
the same experts by a wide margin.  Whole models in bfloat16 are compared with those weights, because rounding turns a
router's close call about once in a hundred tokens (the plain implementation is float64), which moves that token's
logits, and through caches and states those behind it, by far more than rounding does; the float32 comparisons and the
router's own test use routers that decide token by token.
"""

import json
import os

import torch


def attention(heads, kv_heads, dim, vdim, size, keep_first, rot=None, base=10000.0, scale=None, softcap=20.0, v_mix=False):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=size, keep_first=keep_first),
             scale=scale if scale is not None else 1.5 / dim ** 0.5, softcap=softcap, v_mix=v_mix)
    if rot:
        m["rot"] = dict(dims=rot, base=base)
    return dict(type="attention", mixer=m)


def mamba2(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit=1.25, shared=None, shared_limit=2.0):
    m = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit))
    if shared:
        m["shared"] = dict(ff=shared, limit=shared_limit)
    return m


def layer(mix, mlp):
    return dict(mix, mlp=mlp)


def model(vocab, width, layers, eps=1e-6, mult=0.8, logit_scale=0.25):
    return dict(architecture="Bumisun", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, logit_scale=logit_scale,
                layers=layers)


# S: both mixers, three value-mixing attention layers of one shape and one of another that does not mix, a window shorter
# than two pages, a layer with no feed-forward
SMALL = model(200, 64, [
    layer(attention(6, 2, 16, 8, 20, 3, rot=8, v_mix=True), moe(6, 2, 48, shared=32)),
    layer(mamba2(4, 8, 16, conv=4), dense(96)),
    layer(attention(6, 2, 16, 8, 20, 3, rot=8, v_mix=True), None),
    layer(attention(4, 4, 24, 16, 33, 0, rot=24, softcap=0.0), moe(5, 1, 40)),
    layer(attention(6, 2, 16, 8, 20, 3, rot=8, v_mix=True), dense(72))])

# O: sizes that are no multiple of eight, five heads over one kv head, no rotation, many kept tokens, two state groups,
# three norm groups, a convolution of two taps and one of five
ODD = model(333, 90, [
    layer(mamba2(6, 12, 10, groups=2, conv=2, norm_groups=3), moe(7, 3, 30, limit=0.7, shared=50, shared_limit=1.0)),
    layer(attention(5, 1, 12, 20, 9, 21), dense(50)),
    layer(mamba2(3, 20, 7, conv=5), None),
    layer(attention(5, 5, 12, 6, 64, 1, rot=4, base=50.0, v_mix=True), moe(4, 4, 20))], eps=1e-5, mult=1.0, logit_scale=1.0)

# W: more heads than one CTA's rows, vector-sized heads, a window longer than the prompts, a wide state
WIDE = model(512, 128, [
    layer(attention(20, 1, 32, 32, 500, 4, rot=16, v_mix=True), moe(10, 4, 72, shared=88)),
    layer(mamba2(8, 32, 64, groups=4, norm_groups=2), moe(10, 4, 72, shared=88)),
    layer(attention(20, 1, 32, 32, 500, 4, rot=16, v_mix=True), dense(256))], mult=0.5)

# only state-space layers, and only attention layers
STATE_ONLY = model(128, 48, [layer(mamba2(2, 24, 12, conv=3), dense(64)), layer(mamba2(6, 8, 32, groups=3, norm_groups=6), None)])
ATTENTION_ONLY = model(128, 48, [layer(attention(3, 3, 16, 16, 7, 2, rot=16), dense(64)),
                                 layer(attention(8, 2, 8, 24, 100, 0, rot=2, v_mix=True), moe(3, 2, 16, shared=16))])

CONFIGS = dict(small=SMALL, odd=ODD, wide=WIDE, state_only=STATE_ONLY, attention_only=ATTENTION_ONLY)


def tensor_shapes(cfg):
    """name -> (shape, kind)."""
    D = cfg["width"]
    out = {"embed": ((cfg["vocab"], D), "table"), "embed.norm": ((D,), "gain"), "head": ((cfg["vocab"], D), "matrix"),
           "final.norm": ((D,), "gain")}

    def ffn(q, ff):
        out.update({f"{q}.gate": ((ff, D), "matrix"), f"{q}.up": ((ff, D), "matrix"), f"{q}.down": ((D, ff), "matrix")})
    for i, L in enumerate(cfg["layers"]):
        m, p = L["mixer"], f"l{i}"
        out[f"{p}.norm1"] = ((D,), "gain")
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({f"{p}.mix.q": ((H * d, D), "matrix"), f"{p}.mix.k": ((G * d, D), "matrix"), f"{p}.mix.v": ((G * e, D), "matrix"),
                        f"{p}.mix.o": ((D, H * e), "matrix"), f"{p}.mix.sink": ((H,), "sink")})
            if m.get("v_mix"):
                out[f"{p}.mix.vmix"] = ((), "lambda")
        else:
            Hn, e, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = Hn * e, Hn * e + 2 * G * N
            out.update({f"{p}.mix.in": ((inner + ch + Hn, D), "matrix"), f"{p}.mix.conv": ((ch, taps), "conv"),
                        f"{p}.mix.conv.b": ((ch,), "bias"), f"{p}.mix.dt_bias": ((Hn,), "bias"), f"{p}.mix.A_log": ((Hn,), "a_log"),
                        f"{p}.mix.D": ((Hn,), "gain"), f"{p}.mix.norm": ((inner,), "gain"), f"{p}.mix.o": ((D, inner), "matrix")})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        out[f"{p}.norm2"] = ((D,), "gain")
        if mlp["kind"] == "dense":
            ffn(f"{p}.mlp", mlp["ff"])
        else:
            E = mlp["router"]["experts"]
            out[f"{p}.mlp.router"] = ((E, D), "router")
            out[f"{p}.mlp.router.b"] = ((E,), "router_bias")
            for k in range(E):
                ffn(f"{p}.mlp.e{k}", mlp["expert"]["ff"])
            if mlp.get("shared"):
                ffn(f"{p}.mlp.shared", mlp["shared"]["ff"])
                out[f"{p}.mlp.shared.sg"] = ((1, D), "router")
    return out


def random_weights(cfg, seed, calm_router=False):
    """bfloat16 tensors (what a model file holds)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        r = lambda: torch.randn(shape, generator=g)
        if kind == "gain":
            t = 1.0 + 0.2 * r()
        elif kind == "bias":
            t = 0.5 * r()
        elif kind == "router_bias":
            t = 0.8 * torch.randperm(shape[0], generator=g).float() if calm_router else 0.5 * r()
        elif kind == "sink":
            t = 1.0 + r()
        elif kind == "lambda":
            t = 0.2 + 0.6 * torch.rand(shape, generator=g)
        elif kind == "a_log":
            t = -1.0 + r()                        # decays from nearly one down to a fraction a token
        elif kind == "conv":
            t = 0.6 * r()
        elif kind == "router":
            t = (0.05 if calm_router and name.endswith(".router") else 2.0) * r() / shape[-1] ** 0.5
        elif kind == "table":
            t = r()
        else:
            t = 1.3 * r() / shape[-1] ** 0.5
        w[name] = t.to(torch.bfloat16)
    return w


def write_model(folder, name, seed=0, cfg=None, calm_router=False):
    """A model folder for configuration ``name``; returns (folder, config dict, float64 weights for the plain implementation)."""
    from paged_llm_rs_b200.weights.safetensors_io import write_safetensors

    cfg = cfg or CONFIGS[name]
    w = random_weights(cfg, seed, calm_router)
    d = os.path.join(str(folder), f"bumisun_{name}_{seed}{'_calm' if calm_router else ''}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), w)
    return d, cfg, {k: v.double() for k, v in w.items()}
