"""Token embedding (crates/pagedllm/src/model/mod.rs:323-327: a row gather, no
scale; with ``scale`` the rows are multiplied by it, and with ``stream="float32"`` they
leave as float32 whatever the table's dtype, for a decoder that keeps its residual sum
unrounded) and the output head (mod.rs:222-236, 350-351: ``lm_head.weight`` when the
file has it, else the embedding when the config ties them, else an error).
Logits leave the head in float32."""

from __future__ import annotations

import torch

from ..errors import WeightError
from ..kernels import ops
from .base import Part, register_embedding, register_head
from .spec import TensorSpec


class TokenEmbedding(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.stream32 = spec.params.get("stream") == "float32"
        self.leaf = spec.params.get("leaf", "weight")      # the table's name under the prefix ("" when the prefix is the name)
        if self.scale != 1.0 and not self.stream32:
            raise ValueError("a scaled embedding leaves as float32: give stream='float32'")
        self.table = None

    def _table_name(self):
        return self._name(self.leaf) if self.leaf else self.prefix

    def tensors(self):
        return [TensorSpec(self._table_name(), (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.table = tensors[self._table_name()]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.stream32:
            out = torch.empty((tokens.numel(), self.hidden), dtype=torch.float32, device=self.table.device)
            ops.embed_scaled32(tokens, self.table, self.scale, out, self.rt.status)
            self.rt.record(self._name("out"), out)
            return out
        out = torch.empty((tokens.numel(), self.hidden), dtype=self.table.dtype, device=self.table.device)
        ops.embed(tokens, self.table, out, self.rt.status)
        self.rt.record(self._name("out"), out)
        return out


class NormedTokenEmbedding(Part):
    """A row gather with an RMS norm right behind it, into a float32 residual stream: x = norm(table[token]) * gain.
    ``norm`` names the gain's tensor."""

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.vocab, self.hidden, self.eps = int(p["vocab_size"]), int(p["hidden_size"]), float(p["eps"])
        self.leaf, self.norm_name = p.get("leaf", "weight"), p["norm"]
        self.table = self.gain = None

    def _table_name(self):
        return self._name(self.leaf) if self.leaf else self.prefix

    def tensors(self):
        return [TensorSpec(self._table_name(), (self.vocab, self.hidden)), TensorSpec(self.norm_name, (self.hidden,), "gain")]

    def bind(self, tensors):
        self.table, self.gain = tensors[self._table_name()], tensors[self.norm_name]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        out = torch.empty((tokens.numel(), self.hidden), dtype=torch.float32, device=self.table.device)
        ops.embed_norm32(tokens, self.table, self.gain, self.eps, out, self.rt.status)
        self.rt.record(self._name("out"), out)
        return out


class LinearHead(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.vocab, self.hidden = int(p["vocab_size"]), int(p["hidden_size"])
        self.tied, self.tied_to = bool(p.get("tied", False)), p.get("tied_to")
        self.leaf = p.get("leaf", "weight")
        self.scale = float(p.get("scale", 1.0))             # logits = (W x) * scale
        self.weight = None

    def _name(self, leaf: str) -> str:
        if leaf == "weight":
            return super()._name(self.leaf) if self.leaf else self.prefix
        return super()._name(leaf)

    def tensors(self):
        t = [TensorSpec(self._name("weight"), (self.vocab, self.hidden), optional=self.tied)]
        if self.tied:
            t.append(TensorSpec(self.tied_to, (self.vocab, self.hidden)))
        return t

    def bind(self, tensors):
        own = tensors.get(self._name("weight"))
        if own is not None:
            self.weight = own
        elif self.tied:
            self.weight = tensors[self.tied_to]  # the same storage as the embedding, no copy
        else:
            raise WeightError(f"no {self._name('weight')}, and the config does not tie the embeddings")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        logits = ops.linear(x, self.weight, out_dtype=torch.float32)
        if self.scale != 1.0:
            ops.scale32(logits, self.scale)
        self.rt.record(self._name("out"), logits)
        return logits


register_embedding("token_embedding", TokenEmbedding)
register_embedding("normed_token_embedding", NormedTokenEmbedding)
register_head("linear_head", LinearHead)
