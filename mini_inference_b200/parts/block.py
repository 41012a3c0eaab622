"""Pre-norm residual arrangement (engine/core/model_runner.py:120-131):
x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)).  Each addition is carried as a
pending delta into the next norm's kernel, which adds it to the residual stream (in float32,
stored back in the stream's dtype) and normalises in one pass.

When a step has few rows and the three parts offer the optional fast-path protocol (a mixer that
can stop before its output projection, a plain RMS norm, a silu-gated feed-forward), everything
after the mixer's core runs as one persistent kernel (ops.decode_chain); the kernel namespace
decides whether it takes the sizes, and the separate kernels run otherwise."""
from __future__ import annotations

from .base import Part, register_block


@register_block("prenorm")
class PreNormBlock(Part):
    def __init__(self, spec, mixer, feed_forward, norm1, norm2, position):
        super().__init__(spec)
        self.mixer, self.feed_forward, self.norm1, self.norm2, self.position = mixer, feed_forward, norm1, norm2, position

        self.chain = (hasattr(mixer, "forward_open") and hasattr(norm2, "rms_params")
                      and hasattr(feed_forward, "gated_weights"))

        self.open_mixer = hasattr(mixer, "forward_open")
        self.open_ffn = hasattr(feed_forward, "forward_open")
        # a norm that takes the hint is told which weight is streamed right after it
        self.hint1 = getattr(norm1, "takes_next_weight", False) and hasattr(mixer, "first_weight")
        self.hint2 = getattr(norm2, "takes_next_weight", False) and hasattr(feed_forward, "first_weight")

    def forward(self, x, delta, ctx, cache, owns_cache=True):
        ops = ctx.ops
        h = (self.norm1.forward(x, delta, ctx, next_weight=self.mixer.first_weight) if self.hint1
             else self.norm1.forward(x, delta, ctx))
        defer = ctx.defer_ok                   # the readers of `a` and of the returned delta are norms that accept it
        if self.open_mixer:
            rows, w_out = self.mixer.forward_open(h, ctx, cache, self.position, owns_cache)
            chain = getattr(ops, "decode_chain", None) if self.chain else None
            if chain is not None:
                norm_w, eps = self.norm2.rms_params()
                gate_up, down = self.feed_forward.gated_weights()
                out = chain(rows, w_out, x, norm_w, eps, gate_up, down)
                if out is not None:
                    return x, out
            a = ops.linear(rows, w_out, defer=True) if defer else ops.linear(rows, w_out)
        else:
            a = self.mixer.forward(h, ctx, cache, self.position, owns_cache)
        h = (self.norm2.forward(x, a, ctx, next_weight=self.feed_forward.first_weight) if self.hint2
             else self.norm2.forward(x, a, ctx))
        if self.open_ffn and defer:
            rows, w_out = self.feed_forward.forward_open(h, ctx)
            return x, ops.linear(rows, w_out, defer=True)
        return x, self.feed_forward.forward(h, ctx)
