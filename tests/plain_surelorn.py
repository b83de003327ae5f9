"""A plain, slow Surelorn in float64 on the CPU: one function per mechanism, written from the
design's equations, sharing no code with the engine.  It runs a whole sequence at once with
explicit loops where a loop says it best; the tests compare the engine's kernels, cache and
scheduler against it.

Notation: n tokens, D the stream's width, A heads, each with d query/key and e value entries,
r the cached latent's width, u the queries' latent's width.  A weight dict maps tensor names
to float64 tensors; linear weights are [out, in].
"""

import math

import torch

F = torch.float64


# ---- pieces ------------------------------------------------------------------------------------

def unit_rms(x, eps):
    """x scaled to root mean square one (eps inside the root)."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def position_vectors(positions, D, base=10000.0):
    """Row p: (sin(p f_0), cos(p f_0), sin(p f_1), cos(p f_1), ...), f_i = base^(-2i / D)."""
    out = torch.zeros(len(positions), D, dtype=F)
    for row, p in enumerate(positions):
        for i in range(D // 2):
            angle = p * base ** (-2.0 * i / D)
            out[row, 2 * i] = math.sin(angle)
            out[row, 2 * i + 1] = math.cos(angle)
    return out


def embed(w, tokens, scale, first_position=0):
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * scale
    return x + position_vectors(range(first_position, first_position + len(tokens)), x.shape[1])


def gated(w, prefix, x):
    """down(silu(gate x) * (up x))."""
    g = x @ w[f"{prefix}.gate"].T
    return (g * torch.sigmoid(g) * (x @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def latent_attention(w, prefix, m, eps, x):
    """Keys and values per head made from the normed latent; causal softmax; token by token."""
    A, d, e = m["heads"], m["dim"], m["vdim"]
    n = x.shape[0]
    cq = unit_rms(x @ w[f"{prefix}.dq"].T, eps) * w[f"{prefix}.dq.norm"]
    q = (cq @ w[f"{prefix}.uq"].T).reshape(n, A, d)
    c = unit_rms(x @ w[f"{prefix}.dkv"].T, eps) * w[f"{prefix}.dkv.norm"]
    k = (c @ w[f"{prefix}.uk"].T).reshape(n, A, d)
    v = (c @ w[f"{prefix}.uv"].T).reshape(n, A, e)
    heads_out = torch.zeros(n, A, e, dtype=F)
    for i in range(n):
        for a in range(A):
            scores = (k[: i + 1, a] @ q[i, a]) * m["scale"]
            p = torch.softmax(scores, 0)
            heads_out[i, a] = p @ v[: i + 1, a]
    return heads_out.reshape(n, A * e) @ w[f"{prefix}.o"].T


def route(w, prefix, r, x):
    """Per token: (chosen router outputs, their weights).  Lists of lists."""
    total = r["experts"] + r.get("identity", 0)
    z = x @ w[f"{prefix}.router"].T
    s = torch.softmax(z, -1)
    correction = w.get(f"{prefix}.correction")
    picks, weights = [], []
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = total // groups["count"]
    for t in range(x.shape[0]):
        choice = [float(s[t, j]) + (float(correction[j]) if correction is not None else 0.0) for j in range(total)]
        group_best = [max(choice[g * per:(g + 1) * per]) for g in range(groups["count"])]
        kept = sorted(range(groups["count"]), key=lambda g: (-group_best[g], g))[: groups["keep"]]
        allowed = [j for j in range(total) if j // per in kept]
        chosen = sorted(allowed, key=lambda j: (-choice[j], j))[: r["top"]]
        norm = sum(float(s[t, j]) for j in chosen) + 1e-20
        picks.append(chosen)
        weights.append([float(s[t, j]) / norm for j in chosen])
    return picks, weights


def routed(w, prefix, mlp, x):
    r = mlp["router"]
    picks, weights = route(w, prefix, r, x)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        row = x[t:t + 1]
        for j, g in zip(picks[t], weights[t]):
            out[t] += g * (row[0] if j >= r["experts"] else gated(w, f"{prefix}.e{j}", row)[0])
    if mlp.get("shared"):
        out = out + gated(w, f"{prefix}.shared", x)
    return out


# ---- the model ------------------------------------------------------------------------------------

def forward(cfg, w, tokens, streams=None):
    """float64 logits [n, vocab] of the whole sequence; ``streams`` (a list) receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = embed(w, tokens, cfg.get("embedding", {}).get("scale", 1.0))
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of")
        p = f"l{i if src is None else src}"
        x = x + unit_rms(latent_attention(w, f"{p}.mix", layer["mixer"], eps, x), eps) * w[f"{p}.norm1"]
        mlp = layer.get("mlp")
        if mlp is not None:
            f = gated(w, f"{p}.mlp", x) if mlp["kind"] == "dense" else routed(w, f"{p}.mlp", mlp, x)
            x = x + unit_rms(f, eps) * w[f"{p}.norm2"]
        if streams is not None:
            streams.append(x.clone())
    return (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T


def greedy(logits):
    return int(torch.argmax(logits))
