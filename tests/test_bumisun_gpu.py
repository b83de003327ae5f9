"""Bumisun on the GPU against the plain implementation (tests/plain_bumisun.py): each mechanism alone, then whole
models through the engine's step function, cache manager, state slots and scheduler."""

import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_bumisun as P
from bumisun_models import CONFIGS, attention, dense, layer, mamba2, model, moe, write_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


def ops_():
    from paged_llm_rs_b200.kernels import ops
    return ops


def close(got, want, dtype, what="", f32=2e-5, bf16=2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max()) / max(1e-9, float(want.abs().max()))
    assert err < (f32 if dtype == torch.float32 else bf16), f"{what}: relative error {err}"


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def gen(seed):
    return torch.Generator().manual_seed(seed)


# ------------------------------------------------------------------------ each mechanism alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 64), (5, 90), (300, 1024), (3, 4100), (2, 9000)])
def test_normed_embedding_and_the_scaled_add_before_a_norm(dtype, rows, width):
    ops = ops_()
    g = gen(0)
    table = torch.randn(50, width, generator=g).to(dtype)
    gain = 1 + 0.1 * torch.randn(width, generator=g)
    toks = torch.randint(0, 50, (rows,), generator=g)
    x = torch.empty(rows, width, dtype=torch.float32, device=DEV)
    ops.embed_norm32(toks.int().to(DEV), table.to(DEV), gain.to(DEV), 1e-5, x, status())
    x0 = P.rms_norm(table.double()[toks], gain.double(), 1e-5)
    close(x, x0, torch.float32, "normed embedding")
    d = (torch.randn(rows, width, generator=g) * 0.5).to(dtype)
    # some rows only: the sum is formed for them and not stored
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    y = torch.empty(2, width, dtype=dtype, device=DEV)
    before = x.clone()
    ops.add_scaled_norm32(x, d.to(DEV), 0.6, gain.to(DEV), 1e-5, y, rows=idx)
    assert torch.equal(x, before)
    want = P.rms_norm(before.double().cpu() + 0.6 * d.double(), gain.double(), 1e-5)
    close(y, want[[rows - 1, 0]], dtype, "norm of gathered rows", bf16=8e-3)
    # every row: the stream takes the sum
    y = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.add_scaled_norm32(x, d.to(DEV), 0.6, gain.to(DEV), 1e-5, y)
    close(x, before.double().cpu() + 0.6 * d.double(), torch.float32, "stream")
    close(y, want, dtype, "norm", bf16=8e-3)
    # nothing pending
    ops.add_scaled_norm32(x, None, 0.6, gain.to(DEV), 1e-5, y)
    close(y, want, dtype, "norm alone", bf16=8e-3)
    z = x.clone()
    ops.add_scaled32(z, d.to(DEV), -0.6)
    close(z, before, torch.float32, "scaled add", f32=1e-5)
    ops.scale32(z, 0.25)
    close(z, before * 0.25, torch.float32, "scale", f32=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act,limit", [("silu", 0.0), ("relu", 0.0), ("clamped", 1.25), ("clamped", 0.3)])
@pytest.mark.parametrize("rows,inter,width", [(3, 64, 256), (70, 128, 128), (5, 37, 50), (300, 256, 192)])
def test_gated_activations_in_every_form(dtype, act, limit, rows, inter, width):
    """The activation kernel alone, and the gate/up product that carries it (the few-rows kernel, the tcgen05
    product's epilogue, or a product and the kernel, whichever the shapes select)."""
    ops = ops_()
    g = gen(1)
    x = torch.randn(rows, width, generator=g).to(dtype)
    w = (torch.randn(2 * inter, width, generator=g) * 2 / width ** 0.5).to(dtype)
    gu = x.double() @ w.double().T

    def ref(gu):
        a, b = gu[:, :inter], gu[:, inter:]
        if act == "silu":
            return P.silu(a) * b
        if act == "relu":
            return torch.relu(a) * b
        a, b = torch.clamp(a, max=limit), torch.clamp(b, -limit, limit)
        return a * torch.sigmoid(1.702 * a) * (b + 1)
    out = torch.empty(rows, inter, dtype=dtype, device=DEV)
    ops.swiglu(gu.to(dtype).to(DEV), out, act, limit)
    close(out, ref(gu.to(dtype).double()), dtype, "activation kernel", bf16=1e-2)
    y = ops.linear_glu(x.to(DEV), w.to(DEV), act=act, limit=limit)
    close(y, ref(gu), dtype, "gate/up product", bf16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,W,E,top,extra", [(5, 64, 6, 2, 1), (300, 90, 7, 3, 0), (17, 128, 12, 4, 1), (3, 50, 1, 1, 1), (9, 192, 33, 1, 0)])
def test_router_takes_the_largest_logits(dtype, T, W, E, top, extra):
    ops = ops_()
    g = gen(2)
    h = torch.randn(T, W, generator=g).to(dtype)
    wr = (torch.randn(E + extra, W, generator=g) * 3 / W ** 0.5).to(torch.bfloat16).float()
    b = torch.randn(E, generator=g)
    res = ops.moe_route(h.to(DEV), wr.to(DEV), None, top, 1, 1, bias=b.to(DEV), extra=extra)
    ids, wt = P.route(h.double(), wr[:E].double(), b.double(), top)
    z = h.double() @ wr[:E].double().T + b.double()
    srt = torch.sort(z, -1, descending=True).values
    clear = (srt[:, top - 1] - srt[:, top]) > 1e-3 if top < E else torch.ones(T, dtype=torch.bool)
    assert torch.equal(res[0].cpu().long()[clear], ids[clear])
    close(res[1][clear.to(DEV)], wt[clear], torch.float32, "weights", f32=1e-4)
    if extra:
        close(res[2], h.double() @ wr[E:].double().T, torch.float32, "the extra row", f32=1e-4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("form", ["few", "auto"])
@pytest.mark.parametrize("T,W,ff,E,top,shared_ff", [(4, 64, 48, 6, 2, 32), (130, 128, 64, 5, 3, 128), (9, 90, 30, 7, 1, None), (64, 256, 128, 8, 2, 64)])
def test_clamped_experts_and_the_gated_shared_expert(dtype, form, T, W, ff, E, top, shared_ff):
    ops = ops_()
    g = gen(3)
    r = lambda *s: torch.randn(*s, generator=g)
    h = r(T, W).to(dtype)
    w = {}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"], w[f"m.e{e}.down"] = (2 * r(ff, W) / W ** 0.5).to(dtype), (2 * r(ff, W) / W ** 0.5).to(dtype), (r(W, ff) / ff ** 0.5).to(dtype)
    w["m.router"], w["m.router.b"] = (3 * r(E, W) / W ** 0.5).to(torch.bfloat16), r(E).to(torch.bfloat16)
    mlp = dict(router=dict(experts=E, top=top), expert=dict(ff=ff, limit=0.9))
    if shared_ff:
        w["m.shared.gate"], w["m.shared.up"], w["m.shared.down"] = (2 * r(shared_ff, W) / W ** 0.5).to(dtype), (2 * r(shared_ff, W) / W ** 0.5).to(dtype), (r(W, shared_ff) / shared_ff ** 0.5).to(dtype)
        w["m.shared.sg"] = (3 * r(1, W) / W ** 0.5).to(torch.bfloat16)
        mlp["shared"] = dict(ff=shared_ff, limit=1.4)
    wd = {k: v.double() for k, v in w.items()}
    ids, wt = P.route(h.double(), wd["m.router"], wd["m.router.b"], top)
    want = P.moe_ff(h.double(), wd, "m", mlp)
    w_gu = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]], 0) for e in range(E)]).to(DEV)
    w_d = torch.stack([w[f"m.e{e}.down"] for e in range(E)]).to(DEV)
    shared = gate = None
    if shared_ff:
        act = ops.linear_glu(h.to(DEV), torch.cat([w["m.shared.gate"], w["m.shared.up"]], 0).to(DEV), act="clamped", limit=1.4)
        shared = ops.linear(act, w["m.shared.down"].to(DEV))
        gate = (h.double() @ wd["m.shared.sg"].T).float().view(-1).to(DEV)
    fn = ops.moe_experts_few if form == "few" else ops.moe_experts
    kw = dict(act="clamped", limit=0.9, shared_gate=gate)
    got = fn(h.to(DEV), ids.int().to(DEV), wt.float().to(DEV), w_gu, w_d, shared, **kw) if form == "few" else \
        fn(h.to(DEV), ids.int().to(DEV), wt.float().to(DEV), w_gu, w_d, shared, None, **kw)
    close(got, want, dtype, "experts", bf16=3e-2)


def run_rope_write(dtype, T, nh, nkv, dk, dv, rot, page, mix):
    ops = ops_()
    g = gen(4)
    qkv = torch.randn(T, nh * dk + nkv * (dk + dv), generator=g).to(dtype)
    pos = torch.randint(0, 5000, (T,), generator=g).int()
    n_pages = T // page + 2
    slots = torch.randperm(n_pages * page, generator=g)[:T].int()
    slots[0] = -1                                                     # (a padded row writes nothing)
    pool = torch.full((n_pages, nkv, page, dk + dv), 7.0, dtype=dtype, device=DEV)
    inv = torch.tensor([77.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32) if rot else None
    vf_all = torch.randn(T, 3 + nkv * dv, generator=g).to(dtype).to(DEV)
    vf = vf_all[:, 3:] if mix else None                               # (a strided view, as the source layer's values are)
    lam = torch.tensor([0.3], device=DEV) if mix else None
    q = torch.empty(T, nh * dk, dtype=dtype, device=DEV)
    st = status()
    ops.rope_mix_kv_write(qkv.to(DEV), q, inv.to(DEV) if rot else None, rot, pos.to(DEV), slots.to(DEV), pool, vf, lam, nh, nkv, dk, dv, st)
    assert st.item() == 0
    qd = qkv.double()
    qq, kk, vv = qd[:, :nh * dk].view(T, nh, dk), qd[:, nh * dk:nh * dk + nkv * dk].view(T, nkv, dk), qd[:, nh * dk + nkv * dk:].view(T, nkv, dv)
    if rot:
        qq, kk = P.rotate(qq, pos.tolist(), rot, 77.0), P.rotate(kk, pos.tolist(), rot, 77.0)
    if mix:
        vv = 0.7 * vv + 0.3 * vf.double().cpu().view(T, nkv, dv)
    # the angle is a float32 product: at position p its error is about p * 6e-8
    close(q.view(T, nh, dk), qq, dtype, "q", f32=2e-3, bf16=2e-2)
    rows = pool.double().cpu().permute(0, 2, 1, 3).reshape(n_pages * page, nkv, dk + dv)
    for t in range(1, T):
        close(rows[slots[t], :, :dk], kk[t], dtype, "cached key", f32=2e-3, bf16=2e-2)
        close(rows[slots[t], :, dk:], vv[t], dtype, "cached value", f32=1e-5, bf16=1e-2)
    untouched = torch.ones(n_pages * page, dtype=torch.bool)
    untouched[slots[1:].long()] = False
    assert bool((rows[untouched] == 7.0).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,nh,nkv,dk,dv,rot,page,mix", [(9, 6, 2, 16, 8, 8, 16, True), (40, 5, 1, 12, 20, 0, 8, False),
                                                          (3, 8, 4, 128, 64, 48, 16, True), (17, 4, 4, 24, 16, 24, 4, False)])
def test_rotation_value_mixing_and_the_cache_write(dtype, T, nh, nkv, dk, dv, rot, page, mix):
    run_rope_write(dtype, T, nh, nkv, dk, dv, rot, page, mix)


def run_attention(dtype, reqs, nh, nkv, dk, dv, page, window, keep, cap, scale=None, craft=None, target_ctas=296, sink=None):
    """reqs: (cached tokens before, new tokens).  Random keys and values in shuffled pages; returns per request
    (got [n, nh, dv], want) and the number of reductions."""
    from paged_llm_rs_b200.kernels import attention_plan
    from paged_llm_rs_b200.parts.base import AttentionWork
    ops = ops_()
    g = gen(5)
    scale = scale if scale is not None else 1.0 / dk ** 0.5
    group = nh // nkv
    tile, ctas = ops.attention_sink_tile_tokens(nh, nkv, dtype, dk, dv), ops.attention_sink_ctas_per_item(nh, nkv, dtype, dk, dv)
    total_pages = sum(-(-(c + n) // page) for c, n in reqs) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    pool = torch.zeros(total_pages, nkv, page, dk + dv)
    width = max(-(-(c + n) // page) for c, n in reqs)
    tables = torch.full((len(reqs), width), -1, dtype=torch.int32)
    segs, qs, ks, vs, at = [], [], [], [], 0
    sinks = sink if sink is not None else torch.randn(nh, generator=g)
    for r, (c, n) in enumerate(reqs):
        L = c + n
        k, v, q = torch.randn(L, nkv, dk, generator=g), torch.randn(L, nkv, dv, generator=g), torch.randn(n, nh, dk, generator=g)
        if craft:
            craft(r, q, k, v)
        k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
        for b in range(-(-L // page)):
            pg = order.pop()
            tables[r, b] = pg
            m = min(page, L - b * page)
            pool[pg, :, :m, :dk] = k[b * page:b * page + m].float().transpose(0, 1)
            pool[pg, :, :m, dk:] = v[b * page:b * page + m].float().transpose(0, 1)
        # pages that a window has passed are given back (but those of the kept tokens)
        if window:
            for b in range(max(0, c - window + 1) // page):
                if b >= -(-keep // page):
                    tables[r, b] = -1
        segs.append((at, n, c)); qs.append(q); ks.append(k); vs.append(v); at += n
    work, red, parts = attention_plan.plan_attention(segs, tile, window or None, ctas, target_ctas)
    dev = lambda t: t.to(DEV)
    workd = dev(torch.from_numpy(np.ascontiguousarray(work)).reshape(-1, 8)) if len(work) else torch.zeros(1, 8, dtype=torch.int32, device=DEV)
    workd = torch.cat([workd, torch.zeros(3, 8, dtype=torch.int32, device=DEV)])            # (idle items of a captured step)
    redd = dev(torch.from_numpy(np.ascontiguousarray(red)).reshape(-1, 4)) if len(red) else torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    w = AttentionWork(workd, dev(torch.tensor([len(work)], dtype=torch.int32)), len(work) + 3, redd,
                      dev(torch.tensor([len(red)], dtype=torch.int32)), len(red),
                      torch.zeros(max(parts, 1), nh, dv, device=DEV), torch.zeros(max(parts, 1), nh, 2, device=DEV), kinds=3,
                      many_splits=attention_plan.many_splits(len(reqs), ctas, target_ctas))
    qd = dev(torch.cat(qs).contiguous())
    out = torch.zeros(at, nh, dv, dtype=dtype, device=DEV)
    st = status()
    ops.attention_sink(qd, dev(pool.to(dtype)), dev(tables), w, out, dev(sinks.float()), nh, nkv, dk, dv, window, keep, scale, cap, st)
    assert st.item() == 0
    res = []
    for (a, n, c), q, k, v in zip(segs, qs, ks, vs):
        want = P.sink_window_attention(q.double(), k.double(), v.double(), list(range(c, c + n)), scale, cap,
                                       window if window else 1 << 30, keep, sinks.double())
        res.append((out[a:a + n].double().cpu(), want))
    return res, len(red)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,dk,dv,page,window,keep,cap", [
    (6, 2, 16, 8, 16, 20, 3, 20.0), (5, 1, 12, 20, 8, 9, 21, 0.0), (8, 4, 128, 64, 16, 48, 5, 25.0), (20, 1, 32, 32, 16, 500, 4, 5.0),
    (4, 4, 24, 16, 4, 33, 0, 2.0), (3, 3, 16, 16, 16, 7, 2, 50.0), (8, 2, 64, 64, 32, 128, 16, 30.0), (2, 1, 256, 256, 16, 0, 0, 0.0),
    (64, 8, 64, 64, 16, 128, 0, 0.0), (10, 2, 32, 128, 8, 70, 9, 10.0), (80, 1, 64, 32, 16, 30, 2, 0.0), (3, 3, 128, 128, 16, 100, 65, 30.0)])
def test_attention_mixed_batch(dtype, nh, nkv, dk, dv, page, window, keep, cap):
    reqs = [(0, 1), (0, 37), (130, 1), (63, 2), (64, 5), (200, 1), (15, 17), (0, 2), (300, 40)]
    res, _ = run_attention(dtype, reqs, nh, nkv, dk, dv, page, window, keep, cap)
    for i, (got, want) in enumerate(res):
        close(got, want, dtype, f"request {i}", f32=3e-5, bf16=2.5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,dk,dv,window,keep", [(6, 2, 16, 8, 20, 3), (8, 4, 128, 64, 48, 5), (4, 1, 32, 24, 64, 17), (5, 5, 12, 6, 16, 16)])
def test_one_key_decides_at_every_edge(dtype, nh, nkv, dk, dv, window, keep):
    """One cached key pulls the last query of every head: just inside the window it takes (nearly) all the weight, just
    outside it none; likewise the last kept token and the first token that is not kept; in a decoded token and at the
    end of a prompt portion, at page borders and among hundreds of keys."""
    page, ctx = 16, 420
    p_last = ctx                                                # position of the last query
    edges = [(p_last - window + 1, True), (p_last - window, p_last - window < keep), (keep - 1, keep > 0), (keep, p_last - keep < window),
             (0, keep > 0), (p_last, True), (p_last - 1, True), (15, 15 < keep), (16, 16 < keep), (255, False), (256, False)]
    for at, seen in edges:
        if at < 0:
            continue

        def craft(r, q, k, v, at=at):
            if at >= k.shape[0]:
                return
            k[at] = 0.0; k[at, :, : dk // 2] = 2.0
            v[at] = 0.0; v[at, :, : dv // 2] = 3.0
            q[-1] = 0.0; q[-1, :, : dk // 2] = 5.0
        for reqs in ([(ctx, 1)], [(ctx - 20, 21)], [(5, 1), (ctx, 1), (ctx - 2, 3)]):
            res, _ = run_attention(dtype, reqs, nh, nkv, dk, dv, page, window, keep, 0.0, scale=1.0, craft=craft,
                                   sink=torch.zeros(nh))
            for got, want in res:
                close(got, want, dtype, f"key {at} in {reqs}", f32=3e-5, bf16=2.5e-2)
            last = res[0][0][-1] if len(reqs) == 1 else res[1][0][-1]
            pulled = float((last[:, : dv // 2] - 3.0).abs().max()) < 0.05 and float(last[:, dv // 2:].abs().max()) < 0.05
            assert pulled == seen, (at, seen, reqs)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_weight_and_gives_nothing(dtype):
    big = torch.tensor([30.0, -30.0, 0.0, 30.0])
    res, _ = run_attention(dtype, [(50, 1), (0, 9)], 4, 2, 16, 8, 16, 0, 0, 0.0, sink=big)
    for got, want in res:
        close(got, want, dtype, "sinks", f32=3e-5, bf16=2.5e-2)
        assert float(got[:, 0].abs().max()) < 1e-6 and float(got[:, 3].abs().max()) < 1e-6 and float(got[:, 1].abs().max()) > 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
def test_split_ranges_count_the_sink_and_the_kept_tokens_once(dtype):
    """Few requests with long windows: the key ranges are cut into splits; the first split alone takes the sink and
    the kept first tokens."""
    def craft(r, q, k, v):
        k[2] = 0.0; k[2, :, :8] = 2.0; v[2] = 0.0; v[2, :, :4] = 3.0; q[-1] = 0.0; q[-1, :, :8] = 5.0
    res, red = run_attention(dtype, [(3000, 1), (1500, 1)], 6, 2, 16, 8, 16, 1024, 5, 0.0, scale=1.0, craft=craft, target_ctas=64,
                             sink=torch.full((6,), 2.0))
    assert red > 0
    for got, want in res:
        close(got, want, dtype, "split", f32=3e-5, bf16=2.5e-2)
    assert float((res[0][0][-1][:, :4] - 3.0).abs().max()) < 0.05


def run_mamba(dtype, cuts_by_request, heads, groups, P_, N, taps, norm_groups, seed=6):
    """Every request's tokens in the given portions, the requests of a step side by side; returns per request (got, want)
    of the mixer between its projections."""
    ops = ops_()
    g = gen(seed)
    inner, ch = heads * P_, heads * P_ + 2 * groups * N
    lengths = [sum(c) for c in cuts_by_request]
    us = [torch.randn(L, inner + ch + heads, generator=g).to(dtype) for L in lengths]
    conv_w, conv_b = (0.6 * torch.randn(ch, taps, generator=g)).to(dtype), (0.3 * torch.randn(ch, generator=g)).to(dtype)
    dt_bias, a_log, d = 0.5 * torch.randn(heads, generator=g), -1 + torch.randn(heads, generator=g), 1 + 0.2 * torch.randn(heads, generator=g)
    gain = 1 + 0.1 * torch.randn(inner, generator=g)
    floats = ops.mamba2_state_floats(heads, groups, P_, N, taps)
    state = torch.full((len(lengths) + 2, floats + 5), 9.0, device=DEV)          # (a slot that was used before: the first step must not read it)
    slots = list(range(len(lengths), 0, -1))
    at = [0] * len(lengths)
    got = [[] for _ in lengths]
    steps = max(len(c) for c in cuts_by_request)
    for s in range(steps):
        segs, rows, t0 = [], [], 0
        for r, cuts in enumerate(cuts_by_request):
            if s < len(cuts):
                n = cuts[s]
                segs.append((t0, n, at[r], slots[r])); rows.append(us[r][at[r]:at[r] + n]); t0 += n
        segs += [(0, 0, 0, 0)] * 2                                               # (a captured step's empty segments)
        u = torch.cat(rows).contiguous().to(DEV)
        out = torch.empty(t0, inner, dtype=dtype, device=DEV)
        ops.mamba2_mix(u, conv_w.to(DEV), conv_b.to(DEV), dt_bias.to(DEV), a_log.to(DEV), d.to(DEV), gain.to(DEV),
                       torch.tensor(segs, dtype=torch.int32, device=DEV), t0, state, out, heads, groups, P_, N, taps, norm_groups, 1e-5)
        i = 0
        for r, cuts in enumerate(cuts_by_request):
            if s < len(cuts):
                t, n = segs[i][0], cuts[s]
                got[r].append(out[t:t + n].double().cpu()); at[r] += n; i += 1
    res = []
    for r, L in enumerate(lengths):
        ud = us[r].double()
        z, xbc, dt = ud[:, :inner], ud[:, inner:inner + ch], ud[:, inner + ch:]
        c = P.causal_conv_silu(xbc, conv_w.double(), conv_b.double())
        y = P.selective_scan(c[:, :inner].reshape(L, heads, P_), c[:, inner:inner + groups * N].reshape(L, groups, N),
                             c[:, inner + groups * N:].reshape(L, groups, N), P.softplus(dt + dt_bias.double()), a_log.double(), d.double(),
                             heads // groups).reshape(L, inner)
        res.append((torch.cat(got[r]), P.gated_group_norm(y, z, gain.double(), norm_groups, 1e-5)))
    return res


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,groups,P_,N,taps,norm_groups", [(4, 1, 8, 16, 4, 1), (6, 2, 12, 10, 2, 3), (3, 1, 20, 7, 5, 1), (8, 4, 32, 64, 4, 2),
                                                                 (2, 1, 64, 128, 4, 1), (6, 3, 8, 32, 1, 6), (1, 1, 128, 256, 3, 1), (2, 1, 64, 512, 4, 1)])
def test_mamba2_whole_in_portions_and_token_by_token(dtype, heads, groups, P_, N, taps, norm_groups):
    L = 75
    cuts = [[L], [2] * 5 + [1, 1, 3, 17, 16, 20, 1, 1, 1, 1, 1, 1], [1] * L, [40, 35]]
    for got, want in run_mamba(dtype, cuts, heads, groups, P_, N, taps, norm_groups):
        close(got, want, dtype, "mixer", f32=1e-4, bf16=3e-2)


# ------------------------------------------------------------------------ whole models through the engine

class Served:
    """A model on the engine's runner with its cache manager: steps of (request, tokens, wanted places)."""

    def __init__(self, folder, dtype, page=16, pages=64, max_requests=4):
        from paged_llm_rs_b200.engine.runner import ModelRunner
        self.runner = ModelRunner(folder, dtype=NAMES[dtype], page_size=page, num_pages=pages, max_requests=max_requests,
                                  prefix_cache=False, use_graphs=False)

    def step(self, entries, trace=None):
        from paged_llm_rs_b200.engine.step import StepEntry
        cache = self.runner.cache
        es = []
        for rid, toks, want in entries:
            if not cache.has(rid):
                cache.open(rid)
            assert cache.reserve(rid, len(toks)), "no pages left"
            es.append(StepEntry(rid, list(toks), list(want)))
        out = self.runner.step(es, trace=trace).double().cpu()
        for rid, toks, _ in entries:
            cache.commit(rid, len(toks), None)
        return out

    def end(self, rid):
        self.runner.cache.close(rid)


def errors(got, want):
    """Per position: difference of logits with its mean taken off, root mean square over the vocabulary, over the logits' own."""
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def agrees(got, want, dtype):
    """float32: every position within rounding.  bfloat16 (models whose routers do not decide by close calls, see
    bumisun_models.py): most positions well within, a few may be out, none far."""
    e = errors(got, want)
    if dtype == torch.float32:
        return float(e.max()) < TOL[dtype]
    return float(e.median()) < 0.5 * TOL[dtype] and float((e > TOL[dtype]).double().mean()) <= 0.1 and float(e.max()) < 0.3


def stream_agrees(got, want, dtype, what):
    if dtype == torch.float32:
        return close(got, want, dtype, what, f32=5e-5)
    got, want = got.double().cpu(), want.double().cpu()
    per_token = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt()
    assert float(per_token.median()) < 2e-2 and float(per_token.max()) < 0.5, f"{what}: {per_token}"


_models = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("bumisun")

    def get(name, dtype):
        calm = dtype == torch.bfloat16
        if (name, calm) not in _models:
            _models[(name, calm)] = write_model(root, name, seed=len(_models), calm_router=calm)
        return _models[(name, calm)]
    return get


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_layer(models, dtype, name):
    folder, cfg, w = models(name, dtype)
    toks = tokens_for(cfg, 45, 1)
    want, streams = P.forward(cfg, w, toks, want_layers=True)
    s = Served(folder, dtype)
    trace = {}
    got = s.step([("a", toks, list(range(len(toks))))], trace=trace)
    assert agrees(got, want, dtype)
    for i in range(len(cfg["layers"])):
        stream_agrees(trace[f"l{i}.out"], streams[i], dtype, f"stream after layer {i}")
    # the first tokens of a sequence, alone
    s2 = Served(folder, dtype)
    first = torch.cat([s2.step([("b", toks[:1], [0])]), s2.step([("b", toks[1:2], [0])]), s2.step([("b", toks[2:4], [0, 1])])])
    assert agrees(first, want[:4], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("small", 16), ("odd", 8), ("wide", 32), ("state_only", 16), ("attention_only", 4)])
def test_prefill_against_token_by_token_decoding(models, dtype, name, page):
    folder, cfg, w = models(name, dtype)
    toks = tokens_for(cfg, 70, 2)
    want = P.forward(cfg, w, toks)
    s = Served(folder, dtype, page=page, pages=40)
    whole = s.step([("w", toks, list(range(70)))])
    one = torch.cat([s.step([("d", toks[i:i + 1], [0])]) for i in range(70)])
    assert agrees(whole, want, dtype) and agrees(one, want, dtype)
    if dtype == torch.float32:
        assert float(errors(one, whole).max()) < 3e-5          # cutting changes nothing beyond rounding


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "odd", "wide"])
def test_portions_of_every_size(models, dtype, name):
    folder, cfg, w = models(name, dtype)
    toks = tokens_for(cfg, 150, 3)
    want = P.forward(cfg, w, toks)
    for cuts in ([2] * 10 + [3, 5, 16, 17, 31, 33, 25], [64, 64, 22], [1, 2, 13, 48, 1, 1, 84], [149, 1]):
        assert sum(cuts) == 150
        s = Served(folder, dtype, page=16, pages=12)
        at, outs = 0, []
        for c in cuts:
            outs.append(s.step([("p", toks[at:at + c], list(range(c)))]))
            at += c
        assert agrees(torch.cat(outs), want, dtype), cuts


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "odd", "wide"])
def test_batches_of_unequal_requests_pages_and_slots_used_again(models, dtype, name):
    """Four live requests, portions beside single tokens, in a pool and with state slots that only hold them if those
    of finished requests are used again; every row against the plain implementation of its request alone."""
    folder, cfg, w = models(name, dtype)
    lengths = dict(a=90, b=33, c=7, d=64, e=50, f=21)
    toks = {k: tokens_for(cfg, n, 10 + i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: P.forward(cfg, w, t) for k, t in toks.items()}
    s = Served(folder, dtype, page=16, pages=14, max_requests=4)
    at = {k: 0 for k in toks}
    got = {k: [] for k in toks}
    plan = [[("a", 40), ("b", 2), ("c", 1)], [("a", 1), ("b", 30), ("c", 3), ("d", 17)], [("a", 1), ("c", 3), ("d", 47), ("b", 1)],
            [("a", 48), ("e", 2)], [("e", 47), ("f", 1)], [("e", 1), ("f", 20)]]
    for step in plan:
        out = s.step([(k, toks[k][at[k]:at[k] + n], list(range(n))) for k, n in step])
        row = 0
        for k, n in step:
            got[k].append(out[row:row + n]); row += n; at[k] += n
            if at[k] == lengths[k]:
                s.end(k)
    for k in toks:
        assert at[k] == lengths[k]
        assert agrees(torch.cat(got[k]), want[k], dtype), k
    s.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("small", 8), ("odd", 4)])
def test_long_decoding_while_windows_pass_and_pages_go_back(models, dtype, name, page):
    folder, cfg, w = models(name, dtype)
    toks = tokens_for(cfg, 330, 5)
    want = P.forward(cfg, w, toks)
    s = Served(folder, dtype, page=page, pages=30)        # fewer pages than 330 tokens need: the windows' pages are used again
    s.step([("x", toks[:10], [])])
    outs = torch.cat([s.step([("x", toks[i:i + 1], [0])]) for i in range(10, 330)])
    assert agrees(outs, want[10:], dtype)
    assert any(b < 0 for t in s.runner.cache.get("x").tables for b in t.blocks)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_request_left_out_of_steps_goes_on_later(models, dtype):
    folder, cfg, w = models("small", dtype)
    ta, tb = tokens_for(cfg, 60, 8), tokens_for(cfg, 40, 9)
    wa, wb = P.forward(cfg, w, ta), P.forward(cfg, w, tb)
    s = Served(folder, dtype)
    a1 = s.step([("a", ta[:25], list(range(25)))])
    b1 = s.step([("b", tb[:39], list(range(39)))])
    both = s.step([("a", ta[25:], list(range(35))), ("b", tb[39:], [0])])
    assert agrees(torch.cat([a1, both[:35]]), wa, dtype) and agrees(torch.cat([b1, both[35:]]), wb, dtype)


# ------------------------------------------------------------------------ generation, replay, command line

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "wide"])
def test_greedy_generation_through_the_scheduler(models, dtype, name):
    """Engine.generate: chunked prompts, captured decode steps, several requests at once; every produced token
    against the plain implementation on the same history."""
    from paged_llm_rs_b200 import Engine
    folder, cfg, w = models(name, dtype)
    prompts = [tokens_for(cfg, n, 20 + n) for n in (3, 41, 18, 70, 1)]
    eng = Engine(folder, dtype=NAMES[dtype], block_size=16, blocks=64, max_batch=4, chunk=32, prefix_cache=False)
    outs = eng.generate(prompts, max_tokens=12)
    decided = total = out_of_noise = 0
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        seq = list(p)
        for tok in o:
            logits = P.forward(cfg, w, seq)[-1]
            best = P.greedy(logits)
            top2 = torch.topk(logits, 2).values
            noise = (1e-4 if dtype == torch.float32 else 0.05) * max(1.0, float(logits.abs().max()))
            out_of_noise += float(logits[best] - logits[tok]) >= noise
            decided += float(top2[0] - top2[1]) >= noise
            total += 1
            seq.append(tok)
    assert out_of_noise <= (0 if dtype == torch.float32 else 0.05 * total), (out_of_noise, total)
    assert decided >= 0.5 * total


def test_trace_replay_and_command_line(models, tmp_path):
    folder, cfg, w = models("small", torch.float32)
    from trace_tools import TraceBuilder, replay
    toks = tokens_for(cfg, 60, 7)
    tb = TraceBuilder()
    tb.step([("r", toks[:33], [0, 32])])
    tb.step([("r", toks[33:59], [25]), ("q", toks[:5], [4])], end=["q"])
    tb.step([("r", toks[59:], [0])], end=["r"])
    got = tb.collect(replay(folder, "float32", tb.steps, 128, cfg["vocab"]))
    want = P.forward(cfg, w, toks)
    for pos, row in got["r"].items():
        assert float(errors(torch.from_numpy(row).double()[None], want[pos:pos + 1]).max()) < 2e-4
    # the captured and replayed steps of generation give the same logits
    got2 = tb.collect(replay(folder, "float32", tb.steps, 128, cfg["vocab"], graphs=True, step_tokens=48))
    for pos, row in got2["r"].items():
        assert float(errors(torch.from_numpy(row).double()[None], want[pos:pos + 1]).max()) < 2e-4
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "paged_llm_rs_b200", "generate", "--model", folder, "--dtype", "f32",
                        "--prompt-ids", ",".join(map(str, toks[:9])), "--max-tokens", "4", "--blocks", "32"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    out = [int(t) for t in r.stdout.strip().splitlines()[-1].split(",")]
    seq = toks[:9]
    for tok in out:
        assert tok == P.greedy(P.forward(cfg, w, seq)[-1])
        seq = seq + [tok]


# ------------------------------------------------------------------------ configurations drawn at random

def random_configuration(seed):
    """Sizes, counts, layer order and constants drawn from a seed."""
    rnd = random.Random(seed)
    width = rnd.choice([48, 64, 96, 128, 192])
    shared_shape = (rnd.choice([1, 2, 4]), rnd.choice([8, 16, 24, 64]))        # kv heads and value size of the value-mixing layers

    def an_attention():
        mixes = rnd.random() < 0.6
        kv, vdim = shared_shape if mixes else (rnd.choice([1, 2, 3]), rnd.choice([8, 12, 32, 64]))
        heads = kv * rnd.choice([1, 2, 4, 5])
        dim = rnd.choice([8, 16, 24, 32, 64, 128])
        rot = rnd.choice([0, 2, dim // 2, dim])
        return attention(heads, kv, dim, vdim, rnd.choice([1, 5, 16, 31, 64, 200]), rnd.choice([0, 0, 1, 4, 17, 40]),
                         rot=rot - rot % 2, base=rnd.choice([100.0, 10000.0, 5e5]), scale=rnd.choice([0.1, 0.3, 1.0]) / dim ** 0.5 * 4,
                         softcap=rnd.choice([0.0, 3.0, 25.0]), v_mix=mixes)

    def a_mamba():
        groups = rnd.choice([1, 1, 2])
        heads = groups * rnd.choice([1, 2, 3])
        vdim = rnd.choice([8, 16, 24, 32])
        ng = rnd.choice([g for g in (1, 2, heads) if (heads * vdim) % g == 0])
        return mamba2(heads, vdim, rnd.choice([4, 16, 24, 64]), groups=groups, conv=rnd.choice([2, 3, 4]), norm_groups=ng)

    def a_mlp():
        kind = rnd.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            return dense(rnd.choice([32, 72, 128, 192]))
        if kind is None:
            return None
        experts = rnd.choice([1, 2, 5, 8, 12])
        return moe(experts, rnd.randint(1, min(experts, 4)), rnd.choice([24, 64, 128]), limit=rnd.choice([0.5, 1.25, 7.0]),
                   shared=rnd.choice([None, 32, 64, 128]), shared_limit=rnd.choice([0.5, 1.25, 7.0]))
    layers = [layer(an_attention() if rnd.random() < 0.55 else a_mamba(), a_mlp()) for _ in range(rnd.randint(2, 6))]
    return model(rnd.choice([97, 256, 640]), width, layers, eps=rnd.choice([1e-5, 1e-6]), mult=rnd.choice([0.5, 0.8, 1.0]),
                 logit_scale=rnd.choice([0.25, 0.5, 1.0]))


@pytest.mark.parametrize("seed", list(range(1, 15)))
def test_configurations_drawn_at_random(tmp_path, seed):
    cfg = random_configuration(seed)
    toks = tokens_for(cfg, 130, seed)
    for dtype in DTYPES:
        folder, cfg, w = write_model(tmp_path, f"random{seed}", seed=seed, cfg=cfg, calm_router=dtype == torch.bfloat16)
        want = P.forward(cfg, w, toks)
        s = Served(folder, dtype, page=16, pages=24)
        whole = s.step([("w", toks, list(range(130)))])
        s.end("w")
        outs, at = [], 0
        for c in [50, 2, 47, 1, 1, 19, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1]:
            outs.append(s.step([("c", toks[at:at + c], list(range(c)))]))
            at += c
        assert at == 130
        assert agrees(whole, want, dtype), (seed, dtype, cfg)
        assert agrees(torch.cat(outs), want, dtype), (seed, dtype, cfg)
