"""RMSNorm (crates/pagedllm/src/model/layers.rs:40-65): x / sqrt(mean(x^2) + eps)
times a gain, the statistic in float.  ``add_norm`` fuses the residual add that
precedes it (crates/pagedllm/src/model/mod.rs:131-132) into the same kernel."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, register_norm
from .spec import TensorSpec


class RMSNorm(Norm):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.gain = None

    def tensors(self):
        return [TensorSpec(self._name("weight"), (self.width,), "gain")]

    def bind(self, tensors):
        self.gain = tensors[self._name("weight")]

    def forward(self, x, rows=None):
        n = rows.numel() if rows is not None else x.shape[0]
        out = torch.empty((n, self.width), dtype=x.dtype, device=x.device)
        ops.rmsnorm(x, self.gain, self.eps, out, rows=rows)
        self.rt.record(self._name("out"), out)
        return out

    def add_norm(self, residual, delta, rows=None):
        n = rows.numel() if rows is not None else residual.shape[0]
        out = torch.empty((n, self.width), dtype=residual.dtype, device=residual.device)
        # With rows the sum is formed for those rows only and not stored.
        ops.rmsnorm(residual, self.gain, self.eps, out, delta=delta,
                    residual_out=residual if (delta is not None and rows is None) else None, rows=rows)
        self.rt.record(self._name("out"), out)
        return out


register_norm("rmsnorm", RMSNorm)
