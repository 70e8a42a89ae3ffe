"""The pre-norm residual block: x + mixer(norm(x)), then x + ff(norm(x))
(crates/pagedllm/src/model/mod.rs:117-135).  Each residual add is done by the
norm kernel that follows it: the block hands on the residual stream and the
addition that is still pending."""

from __future__ import annotations

from .base import Block, register_block


class PreNormResidualBlock(Block):
    def pre_mixer(self, residual, delta):
        return self.norms["mixer"].add_norm(residual, delta)         # residual += delta, in place

    def post_mixer(self, residual, a, step):
        h = self.norms["feed_forward"].add_norm(residual, a)
        out = self.feed_forward.forward(h, step)
        rt = self.mixer.rt
        if rt.trace is not None and self.prefix:
            rt.record(f"{self.prefix}.out", residual + out)          # (otherwise formed by the next norm's kernel)
        return residual, out

    def forward(self, residual, delta, step, cache, writes_cache=True):
        h = self.pre_mixer(residual, delta)
        a = self.mixer.forward(h, step, cache, writes_cache)
        return self.post_mixer(residual, a, step)


register_block("prenorm_residual", PreNormResidualBlock)
