"""Arrangements of a layer's parts around the residual stream."""

from __future__ import annotations

from .base import Block, register_part


class PreNormBlock(Block):
    """``x += mixer(norm(x)); x += feed_forward(norm(x))``.

    The adds are not done here: each delta is handed to the next norm, which adds and
    normalises in one pass, as the reference's chain does (engine/engine.py:918-961).
    """

    kind = "pre_norm"

    def forward(self, residual, pending, ctx, cache, state):
        normed = self.mixer_norm.forward(residual) if pending is None else self.mixer_norm.add_forward(residual, pending)
        mixed = self.mixer.forward(normed, ctx, cache, state)
        normed = self.ffn_norm.add_forward(residual, mixed)
        return residual, self.feed_forward.forward(normed, ctx)


register_part("block", PreNormBlock.kind, PreNormBlock)
