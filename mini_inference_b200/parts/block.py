"""Pre-norm residual arrangement (engine/core/model_runner.py:120-131):
x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)).  Each addition is carried as a
pending delta into the next norm's kernel, which adds it to the residual stream (in float32,
stored back in the stream's dtype) and normalises in one pass."""
from __future__ import annotations

from .base import Part, register_block


@register_block("prenorm")
class PreNormBlock(Part):
    def __init__(self, spec, mixer, feed_forward, norm1, norm2, position):
        super().__init__(spec)
        self.mixer, self.feed_forward, self.norm1, self.norm2, self.position = mixer, feed_forward, norm1, norm2, position

    def forward(self, x, delta, ctx, cache, owns_cache=True):
        h = self.norm1.forward(x, delta, ctx)
        a = self.mixer.forward(h, ctx, cache, self.position, owns_cache)
        h = self.norm2.forward(x, a, ctx)
        return x, self.feed_forward.forward(h, ctx)
