"""Block arrangements."""
from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    """x += mixer(norm(x)); x += feed_forward(norm(x))   (reference: python/model.py:48-51).
    Each add is folded into the norm that follows it, so a layer's feed-forward output
    is handed on as pending and added by the next layer's first norm (or the final norm)."""

    def forward(self, ctx, x, pending, cache, state):
        h = self.norm_mixer.forward(ctx, x, pending)
        d = self.mixer.forward(ctx, h, cache, state)
        h = self.norm_feed_forward.forward(ctx, x, d)
        return self.feed_forward.forward(ctx, h)


register_block("pre_norm", PreNormBlock)
