"""Bumisun in plain PyTorch on the CPU, float64, one function per mechanism, one token sequence at a
time and nothing kept between calls: what the engine's kernels, caches and state slots are compared with.

Notation: x is the residual stream [T, width]; positions count from 0; weights are stored [out, in].
"""

import torch

F64 = torch.float64


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return unit_rms(x, eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


# ------------------------------------------------------------------------------------------ attention

def rotate(x, positions, dims, base):
    """x [T, heads, dim]: the first ``dims`` entries of each head turn by position * base^(-2i/dims), entry i
    paired with entry i + dims/2; the rest pass."""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = torch.as_tensor(positions, dtype=F64)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def visible(i, j, size, keep_first):
    return j <= i and (i - j < size or j < keep_first)


def sink_window_attention(q, k, v, positions, scale, softcap, size, keep_first, sink):
    """q [T, H, d], k [S, G, d], v [S, G, e]: keys 0..S-1 stand at positions 0..S-1, the queries at ``positions``.
    One token and one head at a time; the sink adds exp(sink_h) to the softmax's denominator only."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for t in range(T):
        i = int(positions[t])
        js = [j for j in range(k.shape[0]) if visible(i, j, size, keep_first)]
        for h in range(H):
            g = h // (H // G)
            s = (k[js, g] @ q[t, h]) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[t, h] = (e[:, None] * v[js, g]).sum(0) / (e.sum() + torch.exp(sink[h] - m))
    return out


def attention_mixer(h, w, p, m, positions, v_first, lam):
    """Returns (output [T, width], this layer's own values [T, G, e] before any mixing).
    ``v_first``: the first value-mixing layer's values of the same tokens, or None when this layer does not mix."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[f"{p}.q"].T).view(T, H, d)
    k = (h @ w[f"{p}.k"].T).view(T, G, d)
    v = (h @ w[f"{p}.v"].T).view(T, G, e)
    own = v
    rot = m.get("rot")
    if rot:
        q, k = rotate(q, positions, rot["dims"], rot["base"]), rotate(k, positions, rot["dims"], rot["base"])
    if v_first is not None:
        v = (1 - lam) * v + lam * v_first
    o = sink_window_attention(q, k, v, positions, m["scale"], m.get("softcap"), m["mask"]["size"], m["mask"]["keep_first"],
                              w[f"{p}.sink"])
    return o.reshape(T, H * e) @ w[f"{p}.o"].T, own


# ------------------------------------------------------------------------------------------ mamba2

def causal_conv_silu(u, taps_w, bias):
    """u [T, C]; taps_w [C, taps], the last column the current token's; zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    out = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        acc = bias.clone()
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                acc = acc + taps_w[:, j] * u[s]
        out[t] = silu(acc)
    return out


def selective_scan(x, B, C, dt, a_log, D, heads_per_group):
    """x [T, heads, e], B and C [T, groups, N], dt [T, heads] (already positive).  Token by token:
    S <- exp(-exp(a_log) dt) S + dt B x^T;  y = S^T C + D x."""
    T, Hn, e = x.shape
    N = B.shape[-1]
    S = torch.zeros(Hn, N, e, dtype=F64)
    y = torch.zeros(T, Hn, e, dtype=F64)
    for t in range(T):
        for h in range(Hn):
            g = h // heads_per_group
            S[h] = torch.exp(-torch.exp(a_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S[h].T @ C[t, g] + D[h] * x[t, h]
    return y


def gated_group_norm(y, z, gain, groups, eps):
    """(y * silu(z)) normed in ``groups`` equal parts, each by its own root mean square, times the gain."""
    T, inner = y.shape
    g = (y * silu(z)).view(T, groups, inner // groups)
    return unit_rms(g, eps).reshape(T, inner) * gain


def mamba2_mixer(h, w, p, m, eps):
    T = h.shape[0]
    Hn, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hn * e
    u = h @ w[f"{p}.in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, w[f"{p}.conv"], w[f"{p}.conv.b"])
    x = xbc[:, :inner].view(T, Hn, e)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[f"{p}.dt_bias"])
    y = selective_scan(x, B, C, dt, w[f"{p}.A_log"], w[f"{p}.D"], Hn // G).reshape(T, inner)
    return gated_group_norm(y, z, w[f"{p}.norm"], m["norm_groups"], eps) @ w[f"{p}.o"].T


# ------------------------------------------------------------------------------------------ feed-forwards

def dense_ff(h, w, p):
    return (torch.relu(h @ w[f"{p}.gate"].T) * (h @ w[f"{p}.up"].T)) @ w[f"{p}.down"].T


def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[f"{p}.gate"].T, max=limit)
    u = torch.clamp(h @ w[f"{p}.up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[f"{p}.down"].T


def route(h, w_router, bias, top):
    """(ids [T, top], weights [T, top]): the largest logits, the softmax over them alone."""
    z = h @ w_router.T + bias
    val, ids = torch.sort(z, dim=-1, descending=True, stable=True)
    return ids[:, :top], torch.softmax(val[:, :top], -1)


def moe_ff(h, w, p, mlp):
    ids, wt = route(h, w[f"{p}.router"], w[f"{p}.router.b"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(ids.shape[1]):
            out[t] += wt[t, k] * clamped_expert(h[t:t + 1], w, f"{p}.e{int(ids[t, k])}", mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[f"{p}.shared.sg"].T)
        out = out + gate * clamped_expert(h, w, f"{p}.shared", mlp["shared"]["limit"])
    return out


# ------------------------------------------------------------------------------------------ the model

def forward(cfg, w, tokens, want_layers=False):
    """Logits [T, vocab] of one sequence run whole (and the stream after every layer)."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    T = len(tokens)
    positions = list(range(T))
    x = rms_norm(w["embed"][torch.as_tensor(tokens)], w["embed.norm"], eps)
    v_first, streams = None, []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}"
        h = rms_norm(x, w[f"{p}.norm1"], eps)
        if L["type"] == "attention":
            mixes = bool(L["mixer"].get("v_mix"))
            a, own = attention_mixer(h, w, f"{p}.mix", L["mixer"], positions, v_first if mixes else None,
                                     w[f"{p}.mix.vmix"] if mixes else None)
            if mixes and v_first is None:
                v_first = own
        elif L["type"] == "mamba2":
            a = mamba2_mixer(h, w, f"{p}.mix", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + mult * a
        mlp = L.get("mlp")
        if mlp is not None:
            h = rms_norm(x, w[f"{p}.norm2"], eps)
            x = x + mult * (dense_ff(h, w, f"{p}.mlp") if mlp["kind"] == "dense" else moe_ff(h, w, f"{p}.mlp", mlp))
        streams.append(x)
    logits = (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg["logit_scale"]
    return (logits, torch.stack(streams)) if want_layers else logits


def greedy(logits):
    """The lowest index among the largest logits."""
    return int(torch.nonzero(logits == logits.max())[0])
