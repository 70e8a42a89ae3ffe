"""The pre-norm residual block: x + mixer(norm(x)), then x + ff(norm(x))
(crates/pagedllm/src/model/mod.rs:117-135).  Each residual add is done by the
norm kernel that follows it."""

from __future__ import annotations

from .base import Block, register_block


class PreNormResidualBlock(Block):
    def forward(self, residual, delta, step, cache, writes_cache=True):
        h = self.norms["mixer"].add_norm(residual, delta)
        a = self.mixer.forward(h, step, cache, writes_cache)
        h = self.norms["feed_forward"].add_norm(residual, a)
        return residual, self.feed_forward.forward(h, step)


register_block("prenorm_residual", PreNormResidualBlock)
