"""Rotary position encoding (crates/pagedllm/src/model/rope.rs:32-63).

inv_freq[i] = 1 / theta^(2i / rotary_dim); the angle position * inv_freq[i] is
formed in float64 on the host and only float32 cos/sin tables reach the device.
The tables hold each angle once, [max_positions, rotary_dim/2]: dimension i
pairs with i + rotary_dim/2 (rope.rs:96-107), which the kernel that applies
them does.  rotary_dim may be smaller than the head (the rest is not rotated).
"""

from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, register_position_encoding


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.head_dim = int(p["head_dim"])
        self.rotary_dim = int(p.get("rotary_dim", self.head_dim))
        self.theta = float(p["theta"])
        self.max_positions = int(p["max_positions"])
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.cos = self.sin = None

    def _tables(self):
        rt = self.rt
        half = self.rotary_dim // 2
        inv_freq = 1.0 / np.power(np.float64(self.theta), 2.0 * np.arange(half, dtype=np.float64) / self.rotary_dim)
        angle = np.arange(self.max_positions, dtype=np.float64)[:, None] * inv_freq[None, :]
        self.cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(rt.device)
        self.sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(rt.device)

    def rotary(self):
        if self.cos is None:
            self._tables()
        return self.cos, self.sin, self.rotary_dim


class NoPositionEncoding(PositionEncoding):
    pass


register_position_encoding("rope", RotaryEncoding)
register_position_encoding("none", NoPositionEncoding)
