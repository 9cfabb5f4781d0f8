"""Arrangement of the parts in a block.  "prenorm": h += mixer(norm1(h)); h += ffn(norm2(h)),
the residual stream h staying FP32 (reference: crates/engine/src/flint.rs:815-1075, :617)."""
from __future__ import annotations

from .. import ops
from .base import Block, PostNormed, WeightedRows, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, h, ctx, cache, state, pending=None):
        if pending is not None and not (isinstance(pending, WeightedRows) and self.norm1.fuses_weighted_rows):
            pending.apply(h)
            pending = None
        ops.current_tag = "norm.mixer"
        xn = self.norm1.forward(h, add=pending)         # the add the block before left is made here
        delta = self.mixer.forward(xn, ctx, cache, state, h)
        ops.current_tag = "norm.ffn"
        xn = self.norm2.forward(h, add=delta)           # h += delta inside the norm when the mixer returned its result
        if self.ffn.defers_add:
            return self.ffn.forward(xn, ctx, h, defer=True)
        self.ffn.forward(xn, ctx, h)
        return None


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm on both sides of each sublayer: h += norm1b(mixer(norm1(h))); h += norm2b(ffn(norm2(h))); a block without
    a feed-forward has the first half only.  The closing add of a sublayer is left to the norm that opens the next one
    (this block's, or the next block's first), which makes both in one pass over the row."""
    takes_extra = True

    def forward(self, h, ctx, cache, state, pending=None, extra=None):
        ops.current_tag = "norm.mixer"
        xn = self.norm1.forward(h, add=pending, extra=extra)
        y = self.mixer.forward(xn, ctx, cache, state, None)
        if y is None:
            raise TypeError(f"{type(self.mixer).__name__} adds into the stream itself; this arrangement needs its result")
        if self.ffn is None:
            return PostNormed(y, self.norm1b)
        ops.current_tag = "norm.ffn"
        xn = self.norm2.forward(h, add=PostNormed(y, self.norm1b))
        return PostNormed(self.ffn.compute(xn, ctx), self.norm2b)
