"""Arrangements of norms, a mixer and a feed-forward in one layer."""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    """x + mixer(norm1(x)), then y + feed_forward(norm2(y)); no post-norms
    (src/models/gpt2/model.rs:218-270 of the reference)."""

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, feed_forward: FeedForward):
        self.norm1, self.mixer, self.norm2, self.feed_forward = norm1, mixer, norm2, feed_forward

    def parts(self):
        return {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "feed_forward": self.feed_forward}

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts().values())

    def forward(self, ctx, residual, entry, owns_cache=True):
        x = self.norm1.forward(ctx, residual, ctx.dtype, lazy=self.mixer.accepts_lazy_norm)
        self.mixer.forward(ctx, x, residual, entry, owns_cache)
        x = self.norm2.forward(ctx, residual, ctx.dtype, lazy=self.feed_forward.accepts_lazy_norm)
        self.feed_forward.forward(ctx, x, residual)
