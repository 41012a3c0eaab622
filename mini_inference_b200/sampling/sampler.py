"""Greedy and temperature sampling of one token per logits row (engine/core/sampler.py:3-11
in the reference).  Temperature 0 is the argmax (ties: lowest id); otherwise the draw comes
from softmax(logits / max(T, 1e-5)) through the Gumbel-max kernel, driven by a counter-based
generator keyed on (request seed, tokens generated so far): the reference draws from the
library's global generator, so its results depend on batch composition; these do not."""
from __future__ import annotations

import torch


def request_seed(engine_seed: int, req) -> int:
    if req.params.seed is not None:
        return req.params.seed & 0xFFFFFFFF
    return (engine_seed * 0x9E3779B1 + req.id * 0x85EBCA6B + 0x27D4EB2F) & 0xFFFFFFFF


def _as_i32(values):
    return [v - (1 << 32) if v >= (1 << 31) else v for v in values]


class Sampler:
    def __init__(self, ops, engine_seed: int = 0):
        self.ops, self.engine_seed = ops, engine_seed

    def sample(self, logits, requests):
        """logits float32 [R, V], one row per request -> int32 device tensor [R]."""
        temps = [max(0.0, float(r.params.temperature)) for r in requests]
        if not any(t > 0 for t in temps):
            return self.ops.argmax(logits)
        dev = logits.device
        t = torch.tensor(temps, dtype=torch.float32, device=dev)
        seeds = torch.tensor(_as_i32([request_seed(self.engine_seed, r) for r in requests]), dtype=torch.int32, device=dev)
        counters = torch.tensor([len(r.output_ids) for r in requests], dtype=torch.int32, device=dev)
        return self.ops.sample(logits, t, seeds, counters)
