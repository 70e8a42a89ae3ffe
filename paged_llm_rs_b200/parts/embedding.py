"""Token embedding (crates/pagedllm/src/model/mod.rs:323-327: a row gather, no
scale) and the output head (mod.rs:222-236, 350-351: ``lm_head.weight`` when the
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
        self.table = None

    def tensors(self):
        return [TensorSpec(self._name("weight"), (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.table = tensors[self._name("weight")]

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        out = torch.empty((tokens.numel(), self.hidden), dtype=self.table.dtype, device=self.table.device)
        ops.embed(tokens, self.table, out, self.rt.status)
        self.rt.record(self._name("out"), out)
        return out


class LinearHead(Part):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.vocab, self.hidden = int(p["vocab_size"]), int(p["hidden_size"])
        self.tied, self.tied_to = bool(p.get("tied", False)), p.get("tied_to")
        self.weight = None

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
        self.rt.record(self._name("out"), logits)
        return logits


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)
