"""RMSNorm: y = w * cast(x32 * rsqrt(mean(x32^2) + eps)), statistics in float32.  The
reference calls the loaded model's norm modules (engine/core/model_runner.py:120-121,133);
here the residual addition that precedes a norm is fused into the same kernel."""
from __future__ import annotations

from .base import Part, WeightSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    accepts_deferred = True      # delta goes to the kernel namespace untouched
    takes_next_weight = True     # and so does the hint about the weight that is read next

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec.get("size"))
        self.eps = float(spec.get("eps"))
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.size,), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"]

    def forward(self, x, delta, ctx, rows=None, next_weight=None):
        if next_weight is not None and ctx.hints_ok:
            return ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, rows, next_weight=next_weight)
        return ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, rows)
