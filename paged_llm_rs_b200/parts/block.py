"""The pre-norm residual block: x + mixer(norm(x)), then x + ff(norm(x))
(crates/pagedllm/src/model/mod.rs:117-135).  Each residual add is done by the
norm kernel that follows it, or, where the norm can be deferred and the part
takes it so, by the part's first product."""

from __future__ import annotations

from .base import Block, register_block


class PreNormResidualBlock(Block):
    @staticmethod
    def _normed(norm, part, residual, delta):
        """(input for the part, the residual stream after the add or None if not yet known)."""
        h = norm.add_norm_deferred(residual, delta) if part.takes_normed_input else None
        if h is None:
            return norm.add_norm(residual, delta), residual   # added in place
        return h, None

    @staticmethod
    def _residual_after(h, residual):
        if residual is not None:
            return residual
        if not h.consumed:
            raise RuntimeError("a part that takes a deferred norm did not pass it to a product")
        return h.residual_out

    def forward(self, residual, delta, step, cache, writes_cache=True):
        h, r = self._normed(self.norms["mixer"], self.mixer, residual, delta)
        a = self.mixer.forward(h, step, cache, writes_cache)
        residual = self._residual_after(h, r)
        h, r = self._normed(self.norms["feed_forward"], self.feed_forward, residual, a)
        out = self.feed_forward.forward(h, step)
        residual = self._residual_after(h, r)
        rt = self.mixer.rt
        if rt.trace is not None and self.prefix:
            rt.record(f"{self.prefix}.out", residual + out)      # (otherwise formed by the next norm's kernel)
        return residual, out


register_block("prenorm_residual", PreNormResidualBlock)
