"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)) (engine/core/model_runner.py:124-131).
gate and up are stored as one [2*inter, hidden] matrix so that one product serves both, as
the reference does with FUSED_PROJ (engine/core/fused_linear.py:173-177,196)."""
from __future__ import annotations

import torch

from .base import Part, WeightSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(Part):
    offers_open = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.get("hidden_size"))
        self.inter = int(spec.get("intermediate_size"))
        self.gate_up = self.down = None

    def weight_specs(self):
        return [WeightSpec("gate_proj", (self.inter, self.hidden)),
                WeightSpec("up_proj", (self.inter, self.hidden)),
                WeightSpec("down_proj", (self.hidden, self.inter))]

    def load(self, tensors, dtype, device):
        self.gate_up = torch.cat([tensors.pop("gate_proj"), tensors.pop("up_proj")], dim=0).contiguous()
        self.down = tensors.pop("down_proj")

    @property
    def open_weight(self):
        return self.down

    @property
    def first_weight(self):
        return self.gate_up

    @property
    def gated_weight(self):
        return self.gate_up

    def first_product_probe(self, ops, rows):
        x = torch.randn(rows, self.hidden, device=self.gate_up.device, dtype=self.gate_up.dtype)
        return lambda w: ops.gated_linear(x, w)

    def forward(self, h, ctx):
        rows, w = self.forward_open(h, ctx)
        return ctx.ops.linear(rows, w)

    def forward_open(self, h, ctx):
        """Everything but the last product: (silu(gate) * up, down weight)."""
        return ctx.ops.gated_linear(h, self.gate_up), self.down
