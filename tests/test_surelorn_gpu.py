"""Surelorn on the GPU against the plain implementation (tests/plain_surelorn.py): each mechanism
alone, then whole models through the engine's step function, cache manager and scheduler."""

import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_surelorn as P
from surelorn_models import CONFIGS, SMALL, write_model

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


# ------------------------------------------------------------------------ each mechanism alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,vocab,scale", [(64, 50, 4.0), (90, 33, 0.5), (1024, 200, 16.0)])
def test_scaled_embedding_and_position_vectors(dtype, width, vocab, scale):
    ops = ops_()
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, width, generator=g).to(dtype)
    toks = torch.randint(0, vocab, (9,), generator=g)
    pos = [0, 1, 2, 63, 64, 1000, 4097, 20000, 65537]
    x = torch.empty(9, width, dtype=torch.float32, device=DEV)
    ops.embed_scaled32(toks.int().to(DEV), table.to(DEV), scale, x, status())
    inv = torch.from_numpy(np.power(10000.0, -2.0 * np.arange(width // 2) / width).astype(np.float32)).to(DEV)
    ops.sinusoid_add(x, torch.tensor(pos, dtype=torch.int32, device=DEV), inv)
    want = table.double()[toks] * scale + P.position_vectors(pos, width)
    # the angle is a float32 product: at position p its error is about p * 6e-8
    assert float((x.double().cpu() - want).abs().max()) < 1e-5 + 65537 * 1.3e-7


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width", [(1, 64), (5, 90), (300, 1024), (3, 4100)])
def test_output_norm_adds_into_a_float32_stream(dtype, rows, width):
    ops = ops_()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(rows, width, generator=g) * 3
    a = (torch.randn(rows, width, generator=g) * 0.3).to(dtype)
    gain = 1 + 0.1 * torch.randn(width, generator=g)
    xd, h = x.to(DEV), (torch.empty(rows, width, dtype=dtype, device=DEV) if dtype != torch.float32 else None)
    ops.outnorm_add(xd, a.to(DEV), gain.to(DEV), 1e-5, h)
    want = x.double() + P.unit_rms(a.double(), 1e-5) * gain.double()
    close(xd, want, torch.float32, "stream")                 # the sum is float32 whatever the dtype
    if h is not None:
        assert torch.equal(h.cpu(), xd.cpu().to(dtype))      # the stream's rounding, bit for bit
    rows_idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    y = torch.empty(2, width, dtype=dtype, device=DEV)
    ops.rmsnorm_from32(xd, gain.to(DEV), 1e-5, y, rows=rows_idx)
    close(y, (P.unit_rms(xd.double().cpu(), 1e-5) * gain.double())[[rows - 1, 0]], dtype, "norm of gathered rows", bf16=8e-3)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("u,r", [(24, 40), (20, 36), (128, 512), (7, 3)])
def test_latent_norms_and_the_cache_write(dtype, u, r):
    ops = ops_()
    g = torch.Generator().manual_seed(2)
    T, page, pages = 6, 4, 5
    qa = torch.randn(T, u + r, generator=g).to(dtype)
    gq, gk = 1 + 0.1 * torch.randn(u, generator=g), 1 + 0.1 * torch.randn(r, generator=g)
    pool = torch.full((pages, page, r), 7.0, dtype=dtype, device=DEV)
    slots = torch.tensor([13, 2, -1, 19, 0, 7], dtype=torch.int32, device=DEV)
    cq = torch.empty(T, u, dtype=dtype, device=DEV)
    st = status()
    ops.latent_norm_write(qa.to(DEV), gq.to(DEV), gk.to(DEV), 1e-6, cq, pool, slots, u, r, st)
    assert st.item() == 0
    close(cq, P.unit_rms(qa.double()[:, :u], 1e-6) * gq.double(), dtype, "q latent", bf16=8e-3)
    c = P.unit_rms(qa.double()[:, u:], 1e-6) * gk.double()
    flat = pool.view(-1, r)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            close(flat[s], c[t], dtype, f"row {s}", bf16=8e-3)
    untouched = [s for s in range(pages * page) if s not in slots.tolist()]
    assert bool((flat[untouched] == 7.0).all())              # a negative slot writes nothing, nor does anything else
    ops.latent_norm_write(qa.to(DEV), gq.to(DEV), gk.to(DEV), 1e-6, cq, pool, torch.tensor([99] * T, dtype=torch.int32, device=DEV), u, r, st)
    assert st.item() == 2                                    # a slot outside the pool is refused, not written


def plain_route(z_w, corr, x, top, groups, keep):
    w = {"m.router": z_w.double()}
    if corr is not None:
        w["m.correction"] = corr.double()
    total = z_w.shape[0]
    return P.route(w, "m", dict(experts=total, identity=0, top=top, groups=dict(count=groups, keep=keep)), x.double())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("outputs,top,groups,keep,corr", [
    (8, 2, 1, 1, 0.0), (10, 3, 2, 1, 0.3), (6, 2, 3, 2, 0.3), (16, 4, 4, 2, 1.0), (8, 1, 1, 1, 0.3), (64, 6, 8, 3, 0.2),
    (12, 4, 3, 1, 5.0), (5, 5, 1, 1, None)])
def test_router(dtype, outputs, top, groups, keep, corr):
    """Chosen outputs and weights.  Corrections as large as -5 make whole groups negative: a group that is not
    kept must count as minus infinity, not as zero."""
    ops = ops_()
    g = torch.Generator().manual_seed(outputs * 7 + top)
    T, width = 40, 72
    x = torch.randn(T, width, generator=g).to(dtype)
    zw = (3 * torch.randn(outputs, width, generator=g) / width ** 0.5).to(torch.bfloat16).float()
    c = None if corr is None else (corr * torch.randn(outputs, generator=g) - (corr if corr >= 1 else 0)).to(torch.bfloat16).float()
    ids, wts = ops.moe_route(x.to(DEV), zw.to(DEV), None if c is None else c.to(DEV), top, groups, keep)
    picks, weights = plain_route(zw, c, x.float(), top, groups, keep)
    ids, wts = ids.cpu().tolist(), wts.cpu().double()
    for t in range(T):
        assert sorted(ids[t]) == sorted(picks[t]), (t, ids[t], picks[t])
        want = dict(zip(picks[t], weights[t]))
        for j, wj in zip(ids[t], wts[t].tolist()):
            assert abs(wj - want[j]) < 1e-5
        assert abs(sum(wts[t].tolist()) - 1) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,width,ff,experts,identity,top,shared", [
    (5, 64, 48, 6, 0, 2, True), (3, 90, 30, 5, 3, 1, False), (70, 128, 64, 14, 2, 4, True), (1, 256, 128, 8, 0, 2, False),
    (300, 256, 128, 8, 2, 3, True), (1000, 128, 192, 5, 0, 1, False), (64, 256, 64, 40, 0, 6, False)])
def test_routed_experts_with_identity_and_shared(dtype, T, width, ff, experts, identity, top, shared):
    ops = ops_()
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, width, generator=g).to(dtype)
    w = {}
    for e in range(experts):
        w[f"m.e{e}.gate"] = (torch.randn(ff, width, generator=g) / width ** 0.5).to(dtype)
        w[f"m.e{e}.up"] = (torch.randn(ff, width, generator=g) / width ** 0.5).to(dtype)
        w[f"m.e{e}.down"] = (torch.randn(width, ff, generator=g) / ff ** 0.5).to(dtype)
    total = experts + identity
    ids = torch.stack([torch.randperm(total, generator=g)[:top] for _ in range(T)]).int()
    if identity:
        ids[0, 0] = total - 1                                  # an identity expert is used for certain
    wt = torch.rand(T, top, generator=g) + 0.1
    wt = wt / wt.sum(-1, keepdim=True)
    sh = torch.randn(T, width, generator=g).to(dtype) if shared else None
    w_gu = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(experts)]).to(DEV)
    w_d = torch.stack([w[f"m.e{e}.down"] for e in range(experts)]).to(DEV)
    for form in ("few", "auto"):
        fn = ops.moe_experts_few if form == "few" else ops.moe_experts
        got = fn(x.to(DEV), ids.to(DEV), wt.to(DEV), w_gu, w_d, None if sh is None else sh.to(DEV))
        wd = {k: v.double() for k, v in w.items()}
        want = torch.zeros(T, width, dtype=torch.float64)
        for t in range(T):
            for j, a in zip(ids[t].tolist(), wt[t].tolist()):
                want[t] += a * (x[t].double() if j >= experts else P.gated(wd, f"m.e{j}", x[t:t + 1].double())[0])
        if sh is not None:
            want += sh.double()
        close(got, want, dtype, f"experts ({form})", f32=2e-5, bf16=2.5e-2)


def run_latent_attention(dtype, reqs, heads, R, page, target_ctas=296, craft=None, seed=0, scale=None, idle=0):
    """reqs: (tokens in the cache before the step, query tokens).  Pages are dealt out of order.  Returns per
    request (got [n, heads, R], want [n, heads, R]), and how many reductions the plan had."""
    from paged_llm_rs_b200.kernels import attention_plan
    from paged_llm_rs_b200.parts.base import AttentionWork
    ops = ops_()
    g = torch.Generator().manual_seed(seed)
    scale = scale if scale is not None else R ** -0.5
    n_pages = sum(-(-(c + n) // page) for c, n in reqs) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    pool = torch.zeros(n_pages, page, R, dtype=dtype)
    width = max(-(-(c + n) // page) for c, n in reqs)
    tables = torch.full((len(reqs), width), -1, dtype=torch.int32)
    qs, cs, segs, t0 = [], [], [], 0
    for r, (c, n) in enumerate(reqs):
        rows = torch.randn(c + n, R, generator=g)
        q = torch.randn(n, heads, R, generator=g)
        if craft:
            craft(r, q, rows)
        rows, q = rows.to(dtype), q.to(dtype)
        for b in range(-(-(c + n) // page)):
            pg = perm.pop()
            tables[r, b] = pg
            m = min(page, c + n - b * page)
            pool[pg, :m] = rows[b * page:b * page + m]
        qs.append(q); cs.append(rows); segs.append((t0, n, c))
        t0 += n
    tile = ops.latent_attention_tile_tokens(heads, R, dtype)
    ctas = ops.latent_attention_ctas_per_item(heads, R, dtype)
    work, red, parts = attention_plan.plan_attention(segs, tile, None, ctas, target_ctas, min_split_keys=64, multi_min_split_keys=64)
    dev = lambda t: t.to(DEV)
    workd = dev(torch.from_numpy(np.ascontiguousarray(work)).reshape(-1, 8)) if len(work) else torch.zeros(1, 8, dtype=torch.int32, device=DEV)
    if idle:
        workd = torch.cat([workd, torch.zeros(idle, 8, dtype=torch.int32, device=DEV)])
    redd = dev(torch.from_numpy(np.ascontiguousarray(red)).reshape(-1, 4)) if len(red) else torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    kinds = (1 if any(n == 1 for _, n in reqs) else 0) | (2 if any(n > 1 for _, n in reqs) else 0)
    w = AttentionWork(workd, dev(torch.tensor([len(work)], dtype=torch.int32)), len(work) + idle, redd,
                      dev(torch.tensor([len(red)], dtype=torch.int32)), len(red),
                      torch.zeros(max(parts, 1), heads, R, device=DEV), torch.zeros(max(parts, 1), heads, 2, device=DEV), kinds=kinds,
                      many_splits=attention_plan.many_splits(len(reqs), ctas, target_ctas))
    qd = dev(torch.cat(qs).contiguous())
    out = torch.zeros_like(qd)
    st = status()
    ops.latent_attention(qd, dev(pool), dev(tables), w, out, scale, st)
    assert st.item() == 0
    res = []
    for (a, n, c), q, rows in zip(segs, qs, cs):
        qf, rf = q.double(), rows.double()
        want = torch.zeros(n, heads, R, dtype=torch.float64)
        for i in range(n):
            p = torch.softmax((qf[i] @ rf[: c + i + 1].T) * scale, -1)        # [heads, keys]
            want[i] = p @ rf[: c + i + 1]
        res.append((out[a:a + n].double().cpu(), want))
    return res, len(red)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,R,page", [(3, 40, 16), (5, 36, 8), (20, 72, 16), (16, 128, 16), (6, 96, 64), (1, 8, 4), (2, 520, 16),
                                          (16, 512, 16), (8, 64, 32), (16, 256, 16), (40, 128, 8), (12, 256, 32), (5, 64, 16)])
def test_latent_attention_mixed_batch(dtype, heads, R, page):
    reqs = [(0, 1), (0, 37), (130, 1), (63, 2), (64, 5), (200, 1), (15, 17), (0, 2)]
    res, _ = run_latent_attention(dtype, reqs, heads, R, page)
    for i, (got, want) in enumerate(res):
        close(got, want, dtype, f"request {i}", f32=3e-5, bf16=2.5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,R", [(3, 40), (16, 128), (20, 72), (16, 256)])
def test_a_far_row_among_hundreds_decides(dtype, heads, R):
    """One cached row far back, at a page's border, pulls every head's query; without it the output is another."""
    page, ctx = 16, 700
    for far in (0, 15, 16, 17, 255, 256, 511, 640, ctx - 1, ctx):
        def craft(r, q, rows, far=far):
            if far >= rows.shape[0]:
                return
            rows[far] = 0.0
            rows[far, : R // 2] = 3.0
            q[-1] = 0.0
            q[-1, :, : R // 2] = 6.0
        for reqs in ([(ctx, 1)], [(ctx - 20, 21)], [(5, 1), (ctx, 1), (ctx - 3, 4)]):
            res, red = run_latent_attention(dtype, reqs, heads, R, page, craft=craft, scale=1.0)
            for got, want in res:
                close(got, want, dtype, f"far row {far} in {reqs}", f32=3e-5, bf16=2.5e-2)
            got_last = res[-1][0][-1] if len(reqs) == 1 else res[1][0][-1]
            # the last query sees (nearly) that row alone: half threes, half zeros
            assert float((got_last[:, : R // 2] - 3.0).abs().max()) < 0.05 and float(got_last[:, R // 2:].abs().max()) < 0.05


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_ranges_are_split_and_combined(dtype):
    res, red = run_latent_attention(dtype, [(3000, 1), (1500, 1)], 6, 96, 16, target_ctas=64, idle=5)
    assert red > 0
    for got, want in res:
        close(got, want, dtype, "split", f32=3e-5, bf16=2.5e-2)
    def craft(r, q, rows):
        rows[1] = 0.0; rows[1, :8] = 4.0; q[-1] = 0.0; q[-1, :, :8] = 8.0
    res, red = run_latent_attention(dtype, [(2999, 1)], 6, 96, 16, target_ctas=64, craft=craft, scale=1.0)
    assert red > 0 and float((res[0][0][-1][:, :8] - 4.0).abs().max()) < 0.05


# ------------------------------------------------------------------------ whole models through the engine

class Served:
    """A model on the engine's runner with its cache manager: steps of (request, tokens, wanted places)."""

    def __init__(self, folder, dtype, page=16, pages=64, max_requests=4):
        from paged_llm_rs_b200.engine.runner import ModelRunner
        self.runner = ModelRunner(folder, dtype=NAMES[dtype], page_size=page, num_pages=pages, max_requests=max_requests,
                                  prefix_cache=False, use_graphs=False)

    def step(self, entries):
        from paged_llm_rs_b200.engine.step import StepEntry
        cache = self.runner.cache
        es = []
        for rid, toks, want in entries:
            if not cache.has(rid):
                cache.open(rid)
            assert cache.reserve(rid, len(toks)), "no pages left"
            es.append(StepEntry(rid, list(toks), list(want)))
        out = self.runner.step(es).double().cpu()
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


def rel(got, want):
    return float(errors(got, want).max())


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def agrees(got, want, dtype):
    """float32: every position within rounding.  bfloat16: rounding may turn a router's close call, which moves that
    token's logits by much more than rounding does (and its successors' by a little), so a few positions may be out
    as long as most are well within."""
    e = errors(got, want)
    if dtype == torch.float32:
        return float(e.max()) < TOL[dtype]
    return float(e.median()) < 0.5 * TOL[dtype] and float((e > TOL[dtype]).double().mean()) <= 0.1
_models = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("surelorn")

    def get(name):
        if name not in _models:
            _models[name] = write_model(root, name, seed=len(_models))
        return _models[name]
    return get


def tokens_for(cfg, n, seed):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "odd", "wide", "tensor"])
def test_whole_prompt_and_every_layer(models, dtype, name):
    folder, cfg, w = models(name)
    toks = tokens_for(cfg, 45, 1)
    streams = []
    want = P.forward(cfg, w, toks, streams)
    s = Served(folder, dtype)
    trace = {}
    from paged_llm_rs_b200.engine.step import StepEntry
    s.runner.cache.open("a"); s.runner.cache.reserve("a", len(toks))
    got = s.runner.step([StepEntry("a", toks, list(range(len(toks))))], trace=trace).double().cpu()
    assert agrees(got, want, dtype)
    # the stream after the LAST run of each layer with tensors of its own is recorded under the layer's name
    last_run = {}
    for i, L in enumerate(cfg["layers"]):
        last_run[L.get("weights_of", i) if L.get("weights_of") is not None else i] = i
    for src, run in last_run.items():
        close(trace[f"l{src}.out"], streams[run], dtype, f"stream after run {run}", f32=5e-5, bf16=3e-2)
    # the first tokens of a sequence, alone
    s2 = Served(folder, dtype)
    first = torch.cat([s2.step([("b", toks[:1], [0])]), s2.step([("b", toks[1:2], [0])]), s2.step([("b", toks[2:4], [0, 1])])])
    assert agrees(first, want[:4], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,page", [("small", 16), ("odd", 8), ("wide", 32)])
def test_prefill_against_token_by_token_decoding(models, dtype, name, page):
    folder, cfg, w = models(name)
    toks = tokens_for(cfg, 70, 2)
    want = P.forward(cfg, w, toks)
    s = Served(folder, dtype, page=page, pages=40)
    whole = s.step([("w", toks, list(range(70)))])
    one = torch.cat([s.step([("d", toks[i:i + 1], [0])]) for i in range(70)])
    assert agrees(whole, want, dtype) and agrees(one, want, dtype)
    if dtype == torch.float32:
        assert rel(one, whole) < 3e-5          # cutting changes nothing beyond rounding


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "odd", "tensor"])
def test_portions_of_every_size(models, dtype, name):
    folder, cfg, w = models(name)
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
@pytest.mark.parametrize("name", ["small", "wide"])
def test_batches_of_unequal_requests_and_pages_used_again(models, dtype, name):
    """Four live requests, portions beside single tokens, in a pool that only holds them if pages of finished
    requests are used again; every row against the plain implementation of its request alone."""
    folder, cfg, w = models(name)
    lengths = dict(a=90, b=33, c=7, d=64, e=50, f=21)
    toks = {k: tokens_for(cfg, n, 10 + i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: P.forward(cfg, w, t) for k, t in toks.items()}
    s = Served(folder, dtype, page=16, pages=14, max_requests=4)
    at = {k: 0 for k in toks}
    got = {k: [] for k in toks}
    plan = [[("a", 40), ("b", 2), ("c", 1)], [("a", 1), ("b", 30), ("c", 3), ("d", 17)], [("a", 1), ("c", 3), ("d", 47), ("b", 1)],
            [("a", 48), ("e", 2)], [("e", 47), ("f", 1)], [("e", 1), ("f", 20)]]
    for step in plan:
        entries = []
        for k, n in step:
            entries.append((k, toks[k][at[k]:at[k] + n], list(range(n))))
        out = s.step(entries)
        row = 0
        for k, n in step:
            got[k].append(out[row:row + n]); row += n; at[k] += n
            if at[k] == lengths[k]:
                s.end(k)
    for k in toks:
        assert at[k] == lengths[k]
        assert agrees(torch.cat(got[k]), want[k], dtype), k
    for grp in s.runner.cache.groups:
        grp.allocator.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_across_many_pages(models, dtype):
    folder, cfg, w = models("small")
    toks = tokens_for(cfg, 330, 5)
    want = P.forward(cfg, w, toks)
    s = Served(folder, dtype, page=8, pages=50)
    s.step([("x", toks[:10], [])])
    outs = torch.cat([s.step([("x", toks[i:i + 1], [0])]) for i in range(10, 330)])
    assert agrees(outs, want[10:], dtype)


# ------------------------------------------------------------------------ generation, replay, command line

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["small", "tensor"])
def test_greedy_generation_through_the_scheduler(models, dtype, name):
    """Engine.generate: chunked prompts, captured decode steps, several requests at once; every produced token
    against the plain implementation on the same history."""
    from paged_llm_rs_b200 import Engine
    folder, cfg, w = models(name)
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
    # (in bfloat16 a router's close call may fall the other way, which moves a token's logits by more than rounding does)
    assert out_of_noise <= (0 if dtype == torch.float32 else 0.05 * total), (out_of_noise, total)
    assert decided >= 0.5 * total


def test_trace_replay_and_command_line(models, tmp_path):
    folder, cfg, w = models("small")
    from trace_tools import TraceBuilder, replay
    toks = tokens_for(cfg, 60, 7)
    tb = TraceBuilder()
    tb.step([("r", toks[:33], [0, 32])])
    tb.step([("r", toks[33:59], [25]), ("q", toks[:5], [4])], end=["q"])
    tb.step([("r", toks[59:], [0])], end=["r"])
    got = tb.collect(replay(folder, "float32", tb.steps, 128, cfg["vocab"]))
    want = P.forward(cfg, w, toks)
    for pos, row in got["r"].items():
        assert rel(torch.from_numpy(row).double()[None], want[pos:pos + 1]) < 2e-4
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
    """Sizes, counts, layer order and constants drawn from a seed: heads from 1 to 24, latent widths with and without the
    tensor-core kernels' sizes, routers with and without groups, identity experts, shared experts, layers without a
    feed-forward and layers that run earlier layers' tensors."""
    import random
    from surelorn_models import dense, layer, mixer, moe
    rnd = random.Random(seed)
    width = rnd.choice([48, 64, 96, 128, 256])

    def a_mixer():
        return mixer(rnd.choice([1, 2, 3, 4, 6, 8, 12, 16, 24]), rnd.choice([8, 16, 24, 32, 64]), rnd.choice([8, 16, 40, 64]),
                     rnd.choice([16, 24, 40, 64, 96, 128, 256]), rnd.choice([8, 24, 32, 80]), scale=rnd.choice([0.1, 0.25, 0.5]))

    def a_mlp():
        kind = rnd.choice(["dense", "moe", "moe", None])
        if kind == "dense":
            return dense(rnd.choice([32, 72, 128, 192]))
        if kind is None:
            return None
        count = rnd.choice([1, 2, 4])
        per = rnd.choice([1, 2, 3])
        total = count * per
        identity = rnd.choice([0, 0, 1, min(2, total - 1)])
        keep = rnd.randint(1, count)
        top = rnd.randint(1, min(keep * per, 4))
        return moe(total - identity, top, rnd.choice([24, 64, 128]), identity=identity,
                   groups=(count, keep) if rnd.random() < 0.8 else None, shared=rnd.choice([None, 32, 64, 128]))
    layers = []
    for i in range(rnd.randint(2, 5)):
        lenders = [j for j, L in enumerate(layers) if L.get("weights_of") is None]
        if lenders and rnd.random() < 0.3:
            j = rnd.choice(lenders)
            layers.append(layer(layers[j]["mixer"], layers[j]["mlp"], weights_of=j))
        else:
            layers.append(layer(a_mixer(), a_mlp()))
    for L in layers:      # a router without groups has no `groups` key; `top` must fit what can be chosen
        m = L["mlp"]
        if m and m["kind"] == "moe" and "groups" not in m["router"]:
            m["router"]["top"] = min(m["router"]["top"], m["router"]["experts"] + m["router"]["identity"])
    return dict(architecture="Surelorn", vocab=rnd.choice([97, 256, 640]), width=width,
                embedding=dict(scale=rnd.choice([1.0, 4.0, 16.0])), norm=dict(eps=rnd.choice([1e-5, 1e-6])), layers=layers)


@pytest.mark.parametrize("seed", list(range(1, 13)))
def test_configurations_drawn_at_random(tmp_path, seed):
    cfg = random_configuration(seed)
    folder, cfg, w = write_model(tmp_path, f"random{seed}", seed=seed, cfg=cfg)
    toks = tokens_for(cfg, 130, seed)
    want = P.forward(cfg, w, toks)
    for dtype in DTYPES:
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
