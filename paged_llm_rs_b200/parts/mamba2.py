"""The Mamba-2 mixer: a selective state space whose decay is one number a head and token.

With h the mixer's input, W_in h = [z: inner | x: inner | B: G N | C: G N | dt: heads] a token, inner = heads * P:

    (x, B, C) <- silu(conv(x | B | C) + b)      a causal convolution of ``conv`` taps a channel, zeros before the start
    dt <- softplus(dt + dt_bias)                per head
    S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T        (N x P a head; head a uses B, C of group a // (heads / G))
    y_t = S_t^T C_t + D x_t
    out = W_o [ norm_g(y * silu(z)) * gain ]    normed in ``norm_groups`` equal parts, each by its own root mean square

Between steps a request keeps, in a slot of fixed size (``StateNeed``, float32): every head's S and each channel's
last conv - 1 inputs.  The recurrence, dt, the decay and the norm are float32 whatever the compute dtype.  A step's
requests are found through its segment list on the device, so a captured step replays with any requests.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, StateNeed, register_mixer
from .spec import TensorSpec


class Mamba2Mixer(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads, self.vdim, self.state, self.groups = int(p["heads"]), int(p["vdim"]), int(p["state"]), int(p.get("groups", 1))
        self.taps, self.norm_groups, self.eps = int(p["conv"]), int(p.get("norm_groups", 1)), float(p["eps"])
        self.inner = self.heads * self.vdim
        self.channels = self.inner + 2 * self.groups * self.state
        if self.heads % self.groups or self.inner % self.norm_groups:
            raise ValueError("heads must divide into groups and the inner width into norm_groups")
        self.names = dict(w_in="in", conv="conv", conv_b="conv.b", dt_bias="dt_bias", a_log="A_log", d="D", norm="norm", o="o")
        self.names.update(p.get("names", {}))
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d = self.gain = None

    def tensors(self):
        n, W = self.names, self.hidden
        return [TensorSpec(self._name(n["w_in"]), (self.inner + self.channels + self.heads, W)),
                TensorSpec(self._name(n["conv"]), (self.channels, self.taps)), TensorSpec(self._name(n["conv_b"]), (self.channels,)),
                TensorSpec(self._name(n["dt_bias"]), (self.heads,), "offset"), TensorSpec(self._name(n["a_log"]), (self.heads,), "offset"),
                TensorSpec(self._name(n["d"]), (self.heads,), "offset"), TensorSpec(self._name(n["norm"]), (self.inner,), "gain"),
                TensorSpec(self._name(n["o"]), (W, self.inner))]

    def bind(self, tensors):
        t = lambda k: tensors[self._name(self.names[k])]
        self.w_in, self.w_o, self.conv_w, self.conv_b = t("w_in"), t("o"), t("conv"), t("conv_b")
        self.dt_bias, self.a_log, self.d, self.gain = t("dt_bias"), t("a_log"), t("d"), t("norm")

    def cache_need(self):
        return StateNeed((ops.mamba2_state_floats(self.heads, self.groups, self.vdim, self.state, self.taps),), torch.float32)

    def forward(self, x, step, cache, writes_cache=True):
        st = self.rt.status
        u = ops.linear(x, self.w_in, status=st)
        y = torch.empty((x.shape[0], self.inner), dtype=x.dtype, device=x.device)
        ops.mamba2_mix(u, self.conv_w, self.conv_b, self.dt_bias, self.a_log, self.d, self.gain, step.segments, step.max_segment_tokens or step.n_tokens,
                       cache, y, self.heads, self.groups, self.vdim, self.state, self.taps, self.norm_groups, self.eps)
        out = ops.linear(y, self.w_o, status=st)
        if self.rt.trace is not None:
            for leaf, t in (("in.out", u), ("o.in", y), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


register_mixer("mamba2", Mamba2Mixer)
