"""Rotary position encoding, rotate-half layout (engine/core/model_runner.py:6-8,151-152).
inv_freq_i = 1 / theta^(2i/D) is made once on the host in float32; the angle pos * inv_freq
and its cos/sin are computed in float32 inside the kernel that rotates q and k."""
from __future__ import annotations

import torch

from .base import Part, register_position


@register_position("rotary")
class RotaryEncoding(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(spec.get("head_dim"))
        self.theta = float(spec.get("theta"))
        self._inv_freq = None

    def load(self, tensors, dtype, device):
        D = self.head_dim
        inv = 1.0 / (self.theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        self._inv_freq = inv.to(device)

    def rotary_inv_freq(self):
        return self._inv_freq

    def on_embedding(self, x, ctx):
        return x


@register_position("none")
class NoPosition(Part):
    def rotary_inv_freq(self):
        return None

    def on_embedding(self, x, ctx):
        return x
