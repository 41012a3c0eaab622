"""Plain PyTorch statement of every kernel the engine launches: the reference each CUDA
kernel is tested against, and a stand-in kernel namespace that lets the engine's batching
and cache logic run on the CPU inside the tests.  Not part of the product path: the package
never imports this file."""
from __future__ import annotations

import torch


class TorchRefOps:
    prefill_tile = 64

    # ---------------------------------------------------------------- elementwise / norms
    def scatter_i32(self, table, idx, val):
        table[idx.long()] = val

    def embedding(self, ids, table):
        return table[ids.long()]

    def add_rmsnorm(self, x, delta, weight, eps, rows=None):
        if rows is None:
            if delta is not None:
                x.copy_((x.float() + delta.float()).to(x.dtype))
            src = x
        else:
            src = x[rows.long()]
            if delta is not None:
                src = (src.float() + delta[rows.long()].float()).to(x.dtype)
        x32 = src.float()
        y = (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
        return (y.float() * weight.float()).to(x.dtype)

    def linear(self, x, w, out_dtype=None, defer=False):
        return (x.float() @ w.float().T).to(out_dtype or x.dtype)

    def gated_linear(self, x, w):
        return self.swiglu(self.linear(x, w))

    def swiglu(self, gate_up):
        g, u = gate_up.float().chunk(2, dim=-1)
        return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)

    # ---------------------------------------------------------------- q/k norm, rotation, cache write
    def qk_norm_rope_cache(self, qkv, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        T = qkv.shape[0]
        dt = qkv.dtype
        q, k, v = qkv.split([H * D, KV * D, KV * D], dim=-1)
        q, k, v = q.reshape(T, H, D), k.reshape(T, KV, D), v.reshape(T, KV, D)

        def norm(t, w):
            if w is None:
                return t
            t32 = t.float()
            y = (t32 * torch.rsqrt(t32.pow(2).mean(-1, keepdim=True) + eps)).to(dt)
            return (y.float() * w.float()).to(dt)

        def rope(t):
            if inv_freq is None:
                return t
            ang = meta.positions.float()[:, None] * inv_freq.float()[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            t32 = t.float()
            a, b = t32[..., :D // 2], t32[..., D // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(dt)

        q = rope(norm(q, q_weight))
        if k_cache is not None:
            k = rope(norm(k, k_weight))
            page, off = meta.slots.long() // meta.page_size, meta.slots.long() % meta.page_size
            k_cache[page, :, off, :] = k
            v_cache[page, :, off, :] = v
        return q.reshape(T, H * D)

    def qkv_project(self, h, w, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        return self.qk_norm_rope_cache(self.linear(h, w), H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache)

    # ---------------------------------------------------------------- attention over the pages
    def paged_attention(self, q, k_cache, v_cache, meta, H, KV, D, scale, window):
        T = q.shape[0]
        out = torch.empty_like(q)
        q = q.view(T, H, D)
        q_start = meta.seg_q_start.tolist()
        pos0, kv_len = meta.seg_pos0.tolist(), meta.seg_kv_len.tolist()
        ps = meta.page_size
        rows = getattr(meta, "table_rows", None)
        rows = list(range(len(pos0))) if rows is None else rows.tolist()
        for s in range(len(pos0)):
            a, b, L = q_start[s], q_start[s + 1], kv_len[s]
            j = torch.arange(L, device=q.device)
            pages = meta.block_table[rows[s], j // ps].long()
            k = k_cache[pages, :, j % ps, :].float()              # [L, KV, D]
            v = v_cache[pages, :, j % ps, :].float()
            k = k.repeat_interleave(H // KV, dim=1)
            v = v.repeat_interleave(H // KV, dim=1)
            p = pos0[s] + torch.arange(b - a, device=q.device)
            visible = j[None, :] <= p[:, None]
            if window is not None:
                visible &= j[None, :] > p[:, None] - window
            sc = torch.einsum("phd,jhd->hpj", q[a:b].float(), k) * scale
            sc = sc.masked_fill(~visible[None], float("-inf"))
            o = torch.einsum("hpj,jhd->phd", torch.softmax(sc, dim=-1), v)
            out[a:b] = o.reshape(b - a, H * D).to(q.dtype)
        return out

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        return logits.argmax(dim=-1).to(torch.int32)

    def sample(self, logits, temperatures, seeds, counters):
        from tests.ref_sampling import gumbel_sample_reference
        return gumbel_sample_reference(logits, temperatures, seeds, counters)
