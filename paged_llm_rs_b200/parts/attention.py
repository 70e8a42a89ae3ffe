"""Grouped-query attention over the paged cache
(crates/pagedllm/src/model/attention.rs:123-216).

q, k and v come from one matrix product over the stacked projection weights;
one kernel then norms q and k per head, rotates them and writes k and v into
the cache pages; the attention kernel reads the pages through the block tables;
the output projection follows.  Head counts, head size, norm eps, scale, window
and the position encoding are parameters.
"""

from __future__ import annotations

import torch

from ..errors import KernelError
from ..kernels import ops
from .base import KVNeed, Mixer, PlanWish, register_mixer
from .spec import TensorSpec


class GQAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt, position_encodings=None):
        super().__init__(spec, rt)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.qk_norm_eps = p.get("qk_norm_eps")  # None: no per-head norm
        self.scale = float(p["scale"])
        self.window = p.get("window")
        name = p.get("position_encoding")
        self.position = (position_encodings or {}).get(name) if name else None
        if name and self.position is None:
            raise KeyError(f"position encoding {name!r} is not among the model's")
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads do not group over {self.nkv} kv heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            # said when the model is built, not by the first step's kernel
            raise KernelError(f"head_dim {self.hd}: the attention kernels take multiples of 16 from 16 to 256")
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None
        self._need = None

    def tensors(self):
        H, qw, kw = self.hidden, self.nh * self.hd, self.nkv * self.hd
        t = [TensorSpec(self._name("q_proj.weight"), (qw, H)), TensorSpec(self._name("k_proj.weight"), (kw, H)),
             TensorSpec(self._name("v_proj.weight"), (kw, H)), TensorSpec(self._name("o_proj.weight"), (H, qw))]
        if self.qk_norm_eps is not None:
            t += [TensorSpec(self._name("q_norm.weight"), (self.hd,), "gain"),
                  TensorSpec(self._name("k_norm.weight"), (self.hd,), "gain")]
        return t

    def bind(self, tensors):
        # one [q; k; v] matrix: a single product makes all three
        self.w_qkv = torch.cat([tensors[self._name(n)] for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")], 0)
        self.w_o = tensors[self._name("o_proj.weight")]
        if self.qk_norm_eps is not None:
            self.q_gain, self.k_gain = tensors[self._name("q_norm.weight")], tensors[self._name("k_norm.weight")]

    def cache_need(self):
        if self._need is None:
            swizzled = self.rt.device.type == "cuda" and ops.pool_is_swizzled(self.rt.dtype, self.nh, self.nkv, self.hd)
            self._need = KVNeed("window" if self.window else "full", self.nkv, self.hd, self.window, swizzled,
                                group_size=self.nh // self.nkv)
        return self._need

    def plan_wish(self, page_size: int):
        group = self.nh // self.nkv
        tile = ops.attention_tile_tokens(self.nh, self.nkv, self.rt.dtype, self.hd, page_size, self.window or 0)
        # CTAs an item: one for every kv head and every 16 query heads of its group
        return PlanWish(tile, self.nkv * -(-group // 16), self.nh, self.hd)

    def forward(self, x, step, cache, writes_cache=True):
        k_pool, v_pool, gi = cache
        g = step.groups[gi]
        w = g.plan
        T = x.shape[0]
        rot = self.position.rotary() if self.position is not None else None
        cos, sin, rdim = rot if rot is not None else (None, None, 0)
        swizzled = self.cache_need().swizzled
        qkv = ops.linear(x, self.w_qkv, status=self.rt.status)
        if writes_cache and w.kinds == 1 and ops.decode_attention_fuses(x.dtype, self.nh, self.nkv, self.hd, k_pool.shape[2],
                                                                          self.window or 0, rdim, swizzled):
            # a step of single decoded tokens: the attention kernel norms and rotates q and k and
            # writes the cache rows itself, straight from the projection's output
            o = torch.empty((T, self.nh * self.hd), dtype=x.dtype, device=x.device)
            ops.decode_attention_fused(qkv, self.q_gain, self.k_gain, self.qk_norm_eps or 0.0, cos, sin, k_pool, v_pool,
                                       g.block_tables, w, o, self.nh, self.nkv, self.hd, self.scale, self.rt.status)
            return ops.linear(o, self.w_o, status=self.rt.status)
        q = torch.empty((T, self.nh * self.hd), dtype=x.dtype, device=x.device)
        ops.qk_norm_rope_kv(qkv, q, self.q_gain, self.k_gain, self.qk_norm_eps or 0.0, cos, sin, rdim,
                            step.positions, g.slots, k_pool if writes_cache else None,
                            v_pool if writes_cache else None, self.nh, self.nkv, self.hd, self.rt.status,
                            swizzled=swizzled)
        o = torch.empty_like(q)
        ops.paged_attention(q, k_pool, v_pool, g.block_tables, w, o, self.nh, self.nkv, self.hd, self.window or 0,
                            self.scale, self.rt.status, swizzled=swizzled)
        out = ops.linear(o, self.w_o, status=self.rt.status)
        if self.rt.trace is not None:
            qw, kw = self.nh * self.hd, self.nkv * self.hd
            for leaf, t in (("q_proj.out", qkv[:, :qw]), ("k_proj.out", qkv[:, qw:qw + kw]), ("v_proj.out", qkv[:, qw + kw:]),
                            ("o_proj.in", o), ("o_proj.out", out), ("out", out)):
                self.rt.record(self._name(leaf), t)
        return out


register_mixer("gqa_attention", GQAttention)
