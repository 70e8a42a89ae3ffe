"""The gated feed-forward, down(silu(gate(x)) * up(x))
(crates/pagedllm/src/model/layers.rs:67-106).  gate and up are one matrix
product over the stacked weights, with the activation in its epilogue for the
few rows of a decode step and as a kernel of its own otherwise."""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, register_feed_forward
from .spec import TensorSpec


class SwiGLUMLP(FeedForward):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up = self.w_down = None

    def tensors(self):
        return [TensorSpec(self._name("gate_proj.weight"), (self.inter, self.hidden)),
                TensorSpec(self._name("up_proj.weight"), (self.inter, self.hidden)),
                TensorSpec(self._name("down_proj.weight"), (self.hidden, self.inter))]

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors[self._name("gate_proj.weight")], tensors[self._name("up_proj.weight")]], 0)
        self.w_down = tensors[self._name("down_proj.weight")]

    def forward(self, x, step):
        act = ops.linear_glu(x, self.w_gate_up, status=self.rt.status)
        out = ops.linear(act, self.w_down, status=self.rt.status)
        if self.rt.trace is not None:
            self.rt.record(self._name("down_proj.in"), act)
            self.rt.record(self._name("down_proj.out"), out)
            self.rt.record(self._name("out"), out)
        return out


register_feed_forward("swiglu_mlp", SwiGLUMLP)
