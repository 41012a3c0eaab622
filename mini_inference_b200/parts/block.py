"""Pre-norm residual arrangement (engine/core/model_runner.py:120-131):
x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)).  Each addition is carried as a
pending delta into the next norm's kernel, which adds it to the residual stream (in float32,
stored back in the stream's dtype) and normalises in one pass.

What the parts offer of the optional protocol (parts/base.py) is read once at construction:
a mixer or feed-forward that can stop before its last product lets the block make that product
with defer=True when every norm of the model accepts deferred sums; a norm that takes the hint is
told which weight the following part streams first."""
from __future__ import annotations

from .base import Part, register_block


@register_block("prenorm")
class PreNormBlock(Part):
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm", "position": "position"}

    def __init__(self, spec, parts):
        super().__init__(spec)
        self.parts = dict(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.norm1, self.norm2, self.position = parts["norm1"], parts["norm2"], parts["position"]
        self.open_mixer = bool(self.mixer.offers_open)
        self.open_ffn = bool(self.feed_forward.offers_open)
        self.hint1 = bool(self.norm1.takes_next_weight)
        self.hint2 = bool(self.norm2.takes_next_weight)

    def norms(self):
        return [self.norm1, self.norm2]

    def forward(self, x, delta, ctx, cache, owns_cache=True):
        ops = ctx.ops
        w1 = self.mixer.first_weight if self.hint1 else None
        h = self.norm1.forward(x, delta, ctx, next_weight=w1) if w1 is not None else self.norm1.forward(x, delta, ctx)
        defer = ctx.defer_ok                   # the readers of `a` and of the returned delta are norms that accept it
        if self.open_mixer:
            rows, w_out = self.mixer.forward_open(h, ctx, cache, self.position, owns_cache)
            a = ops.linear(rows, w_out, defer=True) if defer else ops.linear(rows, w_out)
        else:
            a = self.mixer.forward(h, ctx, cache, self.position, owns_cache)
        w2 = self.feed_forward.first_weight if self.hint2 else None
        h = self.norm2.forward(x, a, ctx, next_weight=w2) if w2 is not None else self.norm2.forward(x, a, ctx)
        if self.open_ffn and defer:
            rows, w_out = self.feed_forward.forward_open(h, ctx)
            return x, ops.linear(rows, w_out, defer=True)
        return x, self.feed_forward.forward(h, ctx)
