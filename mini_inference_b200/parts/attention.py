"""Grouped-query attention over the paged cache (engine/core/model_runner.py:137-196).

q, k, v come from one product on the concatenated weight [(H+2KV)*D, hidden]
(engine/core/fused_linear.py:167-169).  One kernel then applies the per-head q/k RMSNorm
(weights shared by all heads, :148-150), rotates q and k (:151-152) and writes k and v into
the step's pages BEFORE attention runs, so a portion attends to itself through the cache
(:156).  Attention reads the pages in place for prompt portions and decoded tokens alike."""
from __future__ import annotations

import numpy as np
from types import SimpleNamespace

import torch

from .base import KVCacheNeed, Part, WeightSpec, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Part):
    offers_open = True
    step_arrays_key = "paged_attention"

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H, self.KV, self.D = int(g("hidden_size")), int(g("num_heads")), int(g("num_kv_heads")), int(g("head_dim"))
        self.scale = float(g("scale"))
        self.qk_norm = bool(g("qk_norm", False))
        self.qk_eps = float(g("qk_norm_eps", 0.0))
        self.window = g("window")
        if self.H % self.KV:
            raise ValueError(f"{self.H} query heads are not a multiple of {self.KV} kv heads")
        self.qkv = self.o = self.q_norm = self.k_norm = None

    def weight_specs(self):
        H, KV, D, hid = self.H, self.KV, self.D, self.hidden
        specs = [WeightSpec("q_proj", (H * D, hid)), WeightSpec("k_proj", (KV * D, hid)),
                 WeightSpec("v_proj", (KV * D, hid)), WeightSpec("o_proj", (hid, H * D))]
        if self.qk_norm:
            specs += [WeightSpec("q_norm", (D,), kind="vector", init="norm"),
                      WeightSpec("k_norm", (D,), kind="vector", init="norm")]
        return specs

    def cache_need(self):
        return KVCacheNeed(self.KV, self.D, self.window)

    def load(self, tensors, dtype, device):
        self.qkv = torch.cat([tensors.pop("q_proj"), tensors.pop("k_proj"), tensors.pop("v_proj")], dim=0).contiguous()
        self.o = tensors.pop("o_proj")
        self.q_norm, self.k_norm = tensors.get("q_norm"), tensors.get("k_norm")

    @property
    def open_weight(self):
        return self.o

    @property
    def first_weight(self):
        return self.qkv

    def step_flops(self, rows, pairs):
        return 4 * self.H * self.D * pairs                 # q.k and p.v, a multiply and an add each

    def step_arrays(self, facts):
        """The attention kernels' work lists: the entries that feed one token (decode kernel), and for the longer
        entries one (entry, first row) pair per tile of query rows (prompt kernels; the tensor-core kernel takes
        tiles twice as tall)."""
        lens, tile = facts.lens, facts.tile
        decode = [i for i, n in enumerate(lens) if n == 1]
        tiles = [(i, r) for i, n in enumerate(lens) if n > 1 for r in range(0, n, tile)]
        tiles2 = [(i, r) for i, n in enumerate(lens) if n > 1 for r in range(0, n, 2 * tile)]
        as_i32 = lambda v, shape: np.asarray(v, dtype=np.int32).reshape(shape)      # noqa: E731
        return {"decode_segs": as_i32(decode, (-1,)), "prefill_tiles": as_i32(tiles, (-1, 2)),
                "prefill_tiles2": as_i32(tiles2, (-1, 2))}

    def forward(self, h, ctx, cache, position, owns_cache=True):
        o, w = self.forward_open(h, ctx, cache, position, owns_cache)
        return ctx.ops.linear(o, w)

    def forward_open(self, h, ctx, cache, position, owns_cache=True):
        """Everything but the output projection: (attention rows [T, H*D], o_proj weight)."""
        ops = ctx.ops
        meta = ctx.batch.group_view(cache.group, self.step_arrays_key)
        q = ops.qkv_project(h, self.qkv, self.H, self.KV, self.D, self.q_norm, self.k_norm, self.qk_eps,
                            position.rotary_inv_freq(), meta, cache.k if owns_cache else None, cache.v if owns_cache else None)
        o = ops.paged_attention(q, cache.k, cache.v, meta, self.H, self.KV, self.D, self.scale, self.window)
        return o, self.o

    def first_product_probe(self, ops, rows):
        """The projection with norm, rotation and cache write as forward_open runs it, on a made-up cache of its own."""
        dev, dt, page = self.qkv.device, self.qkv.dtype, 16
        x = torch.randn(rows, self.hidden, device=dev, dtype=dt)
        k = torch.zeros(((rows + page - 1) // page + 1, self.KV, page, self.D), device=dev, dtype=dt)
        v = torch.zeros_like(k)
        ar = torch.arange(rows, device=dev, dtype=torch.int32)
        meta = SimpleNamespace(positions=ar, slots=ar + page, page_size=page)
        inv_freq = torch.full((self.D // 2,), 0.01, device=dev, dtype=torch.float32)
        return lambda w: ops.qkv_project(x, w, self.H, self.KV, self.D, self.q_norm, self.k_norm, self.qk_eps, inv_freq, meta, k, v)
