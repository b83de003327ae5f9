"""Grouped-query attention with a capped score, a window that keeps a request's first tokens, a sink in the
softmax and, optionally, values mixed with an earlier layer's.

With h the mixer's input, per token at position p and query head a (kv head a // (heads / kv_heads)):

    q = rot_p(W_q h)_a     k = rot_p(W_k h)     v = W_v h
    score(p, j)  = cap * tanh(scale * q . k_j / cap)                       (cap 0: no cap)
    seen(p, j)   = j <= p and (p - j < window or j < keep_first)
    weight(p, j) = exp(score) / (exp(sink_a) + sum over seen j' of exp(score(p, j')))
    out = W_o [sum over seen j of weight(p, j) v_j]_a

rot_p turns the first ``rot_dims`` entries of a head, entry i with entry i + rot_dims / 2, by the angle
p * base^(-2i / rot_dims), a float32 product; the other entries pass.  The sink is a learned logit a head that takes
weight and gives nothing.  Query / key size and value size may differ; a token's key and value lie side by side in
one cache row (``JoinedKVNeed``), and only the window's pages and those of the first tokens stay with a request.

Value mixing: the first layer of a model that mixes (``value_mix="source"``) hands its values of the step's tokens to
the later ones (``"mixed"``), which cache and attend over (1 - lam) v + lam v_first, lam a learned number of the layer.

Head counts, sizes, scale, cap, window, kept tokens, rotation and tensor leaves are parameters.
"""

from __future__ import annotations

import numpy as np
import torch

from ..errors import KernelError
from ..kernels import ops
from .base import JoinedKVNeed, Mixer, PlanWish, register_mixer
from .spec import TensorSpec


class SinkWindowAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["key_dim"]), int(p["value_dim"])
        self.scale, self.cap = float(p["scale"]), float(p.get("softcap") or 0.0)
        self.window, self.keep_first = int(p.get("window") or 0), int(p.get("keep_first") or 0)
        self.rot, self.rot_base = int(p.get("rot_dims") or 0), float(p.get("rot_base", 10000.0))
        self.has_sink = bool(p.get("sink", True))
        self.value_mix = p.get("value_mix")                      # None, "source" or "mixed"
        self.carry_key = p.get("value_mix_key", "value_mix.first")
        if self.value_mix not in (None, "source", "mixed"):
            raise ValueError(f"value_mix {self.value_mix!r}: None, 'source' or 'mixed'")
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads do not group over {self.nkv} kv heads")
        if self.rot % 2 or self.rot > self.dk:
            raise ValueError(f"rot_dims {self.rot} must be even and at most key_dim {self.dk}")
        if max(self.dk, self.dv) > 256:
            raise KernelError(f"key_dim {self.dk} / value_dim {self.dv}: the attention kernel takes sizes up to 256")
        self.names = dict(q="q", k="k", v="v", o="o", sink="sink", lam="vmix")
        self.names.update(p.get("names", {}))
        self.w_qkv = self.w_o = self.sinks = self.lam = self.inv_freq = None
        self._need = None

    def tensors(self):
        n, H = self.names, self.hidden
        t = [TensorSpec(self._name(n["q"]), (self.nh * self.dk, H)), TensorSpec(self._name(n["k"]), (self.nkv * self.dk, H)),
             TensorSpec(self._name(n["v"]), (self.nkv * self.dv, H)), TensorSpec(self._name(n["o"]), (H, self.nh * self.dv))]
        if self.has_sink:
            t.append(TensorSpec(self._name(n["sink"]), (self.nh,), "offset"))
        if self.value_mix is not None:
            t.append(TensorSpec(self._name(n["lam"]), (), "offset"))      # (the source layer's is in the file and unused)
        return t

    def bind(self, tensors):
        n = self.names
        self.w_qkv = torch.cat([tensors[self._name(n[k])] for k in ("q", "k", "v")], 0).contiguous()
        self.w_o = tensors[self._name(n["o"])]
        self.sinks = tensors[self._name(n["sink"])] if self.has_sink else None
        if self.value_mix == "mixed":
            self.lam = tensors[self._name(n["lam"])].reshape(1).contiguous()
        if self.rot:
            f = np.power(np.float64(self.rot_base), -2.0 * np.arange(self.rot // 2, dtype=np.float64) / self.rot)
            self.inv_freq = torch.from_numpy(f.astype(np.float32)).to(self.w_o.device)

    def cache_need(self):
        if self._need is None:
            self._need = JoinedKVNeed("window" if self.window else "full", self.nkv, self.dk, self.dv, self.window or None,
                                      self.keep_first if self.window else 0, group_size=self.nh // self.nkv)
        return self._need

    def plan_wish(self, page_size: int):
        a = (self.nh, self.nkv, self.rt.dtype, self.dk, self.dv)
        return PlanWish(ops.attention_sink_tile_tokens(*a), ops.attention_sink_ctas_per_item(*a), self.nh, self.dv)

    def forward(self, x, step, cache, writes_cache=True):
        kv_pool, gi = cache
        g = step.groups[gi]
        T, st = x.shape[0], self.rt.status
        qkv = ops.linear(x, self.w_qkv, status=st)
        v_first = None
        if self.value_mix == "source":
            step.carry[self.carry_key] = qkv[:, self.nh * self.dk + self.nkv * self.dk:]
        elif self.value_mix == "mixed":
            v_first = step.carry.get(self.carry_key)
            if v_first is None:
                raise KernelError(f"{self.prefix}: mixes values, but no earlier layer of the step handed any on")
        q = torch.empty((T, self.nh * self.dk), dtype=x.dtype, device=x.device)
        ops.rope_mix_kv_write(qkv, q, self.inv_freq, self.rot, step.positions, g.slots, kv_pool if writes_cache else None,
                              v_first, self.lam if v_first is not None else None, self.nh, self.nkv, self.dk, self.dv, st)
        o = torch.empty((T, self.nh * self.dv), dtype=x.dtype, device=x.device)
        ops.attention_sink(q, kv_pool, g.block_tables, g.plan, o, self.sinks, self.nh, self.nkv, self.dk, self.dv, self.window,
                           self.keep_first, self.scale, self.cap, st)
        out = ops.linear(o, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("q.rotated", q), ("o.in", o), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


register_mixer("sink_window_attention", SinkWindowAttention)
