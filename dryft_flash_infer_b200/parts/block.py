"""Arrangements of a layer's parts around the residual stream."""

from __future__ import annotations

from ..ops import kernels
from .base import Block, register_part


class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))``.

    The adds are not done here: each delta is handed to the next norm, which adds and
    normalises in one pass, as the reference's chain does (engine/engine.py:918-961).
    When decoding (few bfloat16 rows) and the parts on both sides of a norm can, even that
    pass disappears: the product before the norm adds its result to the residual and leaves
    the rows scaled by the norm's weight, and the product after it applies 1/rms.  Over a prompt's
    many bfloat16 rows the product takes the residual as its addend, so that the delta is never
    written, and the norm reads the sum alone.
    """

    kind = "pre_norm"
    norm_names = ("mixer_norm", "ffn_norm")
    fuses_next_norm = True

    def __init__(self, mixer, feed_forward, norms):
        super().__init__(mixer, feed_forward, norms)
        self.mixer_norm, self.ffn_norm = self.norms["mixer_norm"], self.norms["ffn_norm"]

    @property
    def first_norm(self):
        return self.mixer_norm

    @property
    def takes_scaled_pending(self) -> bool:
        return self.mixer.accepts_scaled_rows and self.mixer_norm.scale_fusion() is not None

    def forward(self, residual, pending, ctx, cache, state, next_norm=None):
        after = ctx.upcoming                     # what follows this block; the mixer is followed by the feed-forward
        ctx.upcoming = self.feed_forward.first_weights()
        try:
            return self._forward(residual, pending, ctx, cache, state, next_norm, after)
        finally:
            ctx.upcoming = after

    def _forward(self, residual, pending, ctx, cache, state, next_norm, after):
        fusable = kernels.add_norm_fusable(residual)
        if isinstance(pending, kernels.ScaledRows):
            normed = pending                     # the block before added its result and prepared this norm
        elif pending is None:
            normed = self.mixer_norm.forward(residual)
        else:
            normed = self.mixer_norm.add_forward(residual, pending)
        fusion = self.ffn_norm.scale_fusion() if fusable and self.mixer.fuses_add_norm \
            and self.feed_forward.accepts_scaled_rows else None
        if fusion is not None:
            normed = self.mixer.forward(normed, ctx, cache, state, add_norm=(residual, *fusion))
        else:
            mixed = self.mixer.forward(normed, ctx, cache, state)
            normed = self.ffn_norm.add_forward(residual, mixed)
        ctx.upcoming = after
        fusion = next_norm.scale_fusion() if next_norm is not None and fusable and self.feed_forward.fuses_add_norm else None
        if fusion is not None:
            return residual, self.feed_forward.forward(normed, ctx, add_norm=(residual, *fusion))
        return residual, self.feed_forward.forward(normed, ctx)


register_part("block", PreNormBlock.kind, PreNormBlock)
