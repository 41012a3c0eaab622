"""Pure-decode steps replayed as CUDA graphs, one graph per batch-size bucket.

The reference does the same for its decode steps (engine/core/cuda_graphs.py:8-139): fixed
device buffers, pinned staging, one graph per bucket, rows beyond the live batch padded with
harmless work (token 0, position 0, a one-key context on a scratch page).  Differences here:
all metadata of a step travels in ONE pinned buffer and one copy; sampling is inside the
graph, so a step returns token ids, not logits; padding rows use the cache's null page 0,
which no request ever owns.  The number of key splits of the attention kernel is fixed per
bucket from the longest sequence the cache admits, so the grid depends on the bucket only
(engine/core/cuda_graphs.py:55); each request still cuts its own length."""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from ..parts.base import StepContext
from .batch import GroupMeta

DEFAULT_BUCKETS = [1, 2, 4, 8, 12, 16, 24, 32, 40, 48, 56, 64, 80, 96, 112, 128, 160, 192, 224, 256]


class _StaticBatch:
    """The StepBatch of a decode-only step of exactly `bucket` rows, as views into one fixed
    device buffer that a pinned host buffer of the same layout is copied into before a replay."""

    def __init__(self, bucket: int, cache, device, max_kv_len: int, tile: int):
        B = bucket
        self.bucket = B
        self.num_tokens = self.num_segs = self.num_decode = self.num_logit_rows = B
        self.num_prefill_tiles = 0
        self.tile = tile
        self.max_kv_len = max_kv_len                  # fixes the split count for this bucket
        self.max_q_len = 1
        P = cache.max_pages_per_seq
        G = len(cache.kv_groups)
        fields = [("token_ids", B), ("positions", B), ("seg_pos0", B), ("seg_kv_len", B), ("seg_slot", B),
                  ("temps", B), ("seeds", B), ("counters", B)]
        fields += [(f"slots{g}", B) for g in range(G)] + [(f"table{g}", B * P) for g in range(G)]
        self.offsets, total = {}, 0
        for name, n in fields:
            self.offsets[name] = (total, n)
            total += (n + 3) // 4 * 4
        self.size = total
        self.dev = torch.zeros(total, dtype=torch.int32, device=device)
        ar = torch.arange(B + 1, dtype=torch.int32, device=device)
        self.token_seg = self.decode_segs = self.logit_rows = ar[:B]
        self.seg_q_start = ar
        self.prefill_tiles = torch.zeros((0, 2), dtype=torch.int32, device=device)
        for name in ("token_ids", "positions", "seg_pos0", "seg_kv_len", "seg_slot", "seeds", "counters"):
            setattr(self, name, self.view(name))
        self.temps = self.view("temps").view(torch.float32)
        self.groups = [GroupMeta(self, cache.page_size, self.view(f"slots{g}"), self.view(f"table{g}").view(B, P), P)
                       for g in range(G)]

    def view(self, name, buf=None):
        a, n = self.offsets[name]
        return (self.dev if buf is None else buf)[a:a + n]


class DecodeGraphs:
    RING = 4            # pinned staging buffers in flight

    def __init__(self, runner, max_batch: int, buckets: Optional[List[int]] = None):
        self.runner, self.cache, self.ops = runner, runner.cache, runner.ops
        self.device = runner.device
        self.buckets = [b for b in (buckets or DEFAULT_BUCKETS) if b < max_batch] + [max_batch]
        self.max_batch = max_batch
        self.batches, self.graphs, self.tokens_out, self.launches = {}, {}, {}, {}
        self.staging, self.events, self._turn = {}, {}, {}
        self.out_host, self._out_turn = {}, {}
        self.replays = self.eager_steps = 0
        self.capture_s = 0.0

    # ---------------------------------------------------------------- capture
    def _forward(self, batch):
        ctx = StepContext(self.ops, batch, self.runner.dtype, self.device)
        logits = self.runner.model.forward(ctx, self.cache.layer_caches)
        return self.ops.sample(logits, batch.temps, batch.seeds, batch.counters)

    def capture(self):
        import time
        t0 = time.perf_counter()
        max_len = self.cache.max_pages_per_seq * self.cache.page_size
        pool = None
        for B in sorted(self.buckets, reverse=True):            # largest first: smaller graphs reuse its pool
            batch = _StaticBatch(B, self.cache, self.device, max_len, self.ops.prefill_tile)
            batch.view("seg_kv_len").fill_(1)                    # harmless rows: one key on the null page
            self.staging[B] = [torch.zeros(batch.size, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
            self.out_host[B] = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
            self._out_turn[B] = 0
            self.events[B] = [None] * self.RING
            self._turn[B] = 0
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):                               # warm up library workspaces outside the capture
                    self._forward(batch)
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = self.ops.launches
            with torch.cuda.graph(graph, pool=pool):
                out = self._forward(batch)
            self.launches[B] = self.ops.launches - before
            pool = pool or graph.pool()
            self.batches[B], self.graphs[B], self.tokens_out[B] = batch, graph, out
        torch.cuda.synchronize(self.device)
        self.capture_s = time.perf_counter() - t0

    # ---------------------------------------------------------------- replay
    def bucket_for(self, n: int) -> Optional[int]:
        for b in self.buckets:
            if b >= n:
                return b
        return None

    def fill(self, B, seqs, tokens, temps=None, seeds=None, counters=None):
        """Write one decode step's metadata for the live rows (and padding) into the next pinned
        buffer and start its copy.  tokens=None keeps the token ids already on the device (the
        previous step's samples, see feed_back)."""
        batch = self.batches[B]
        turn = self._turn[B]
        self._turn[B] = (turn + 1) % self.RING
        if self.events[B][turn] is not None:
            self.events[B][turn].synchronize()                   # its last copy has left the buffer
        host = self.staging[B][turn]
        h = host.numpy()
        n = len(seqs)
        pos = np.fromiter((s.num_tokens for s in seqs), dtype=np.int32, count=n)

        def put(name, values, pad):
            a, m = batch.offsets[name]
            h[a:a + n] = values
            h[a + n:a + B] = pad
        put("positions", pos, 0)
        put("seg_pos0", pos, 0)
        put("seg_kv_len", pos + 1, 1)
        put("seg_slot", [s.slot for s in seqs], 0)
        a, _ = batch.offsets["temps"]
        h[a:a + B] = 0
        if temps is not None:
            h[a:a + n] = np.asarray(temps, dtype=np.float32).view(np.int32)
            put("seeds", np.asarray(seeds, dtype=np.uint32).view(np.int32), 0)
            put("counters", np.asarray(counters, dtype=np.int32), 0)
        P = self.cache.max_pages_per_seq
        for g in range(len(self.cache.kv_groups)):
            put(f"slots{g}", [self.cache.slots_for(g, s, int(p), int(p) + 1)[0] for s, p in zip(seqs, pos)], 0)
            a, _ = batch.offsets[f"table{g}"]
            h[a:a + n * P] = self.cache.table_rows(g, seqs, P).reshape(-1)
            h[a + n * P:a + B * P] = 0
        a_tok, _ = batch.offsets["token_ids"]
        end = a_tok + (B + 3) // 4 * 4
        if tokens is not None:
            h[a_tok:a_tok + n] = tokens
            h[a_tok + n:a_tok + B] = 0
            batch.dev.copy_(host, non_blocking=True)
        else:                                                    # everything but the token ids
            batch.dev[end:].copy_(host[end:], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.events[B][turn] = ev
        return batch.size * 4 if tokens is not None else (batch.size - end) * 4

    def feed_back(self, B):
        """Next step's token ids = this step's samples, without leaving the device."""
        self.batches[B].token_ids.copy_(self.tokens_out[B])

    def replay(self, B):
        self.graphs[B].replay()
        self.replays += 1
        self.ops.launches += self.launches[B]

    def can_run(self, chunks) -> bool:
        """A pure decode step that fits a bucket (engine/core/cuda_graphs.py:87)."""
        return all(e - s == 1 and s > 0 for _, s, e in chunks) and self.bucket_for(len(chunks)) is not None

    def launch(self, chunks, sampler, on_device_tokens: bool = False):
        """Start one decode step and the copy of its sampled tokens to pinned host memory; returns a
        handle for read().  on_device_tokens: the input tokens are the previous step's samples,
        which are still on the device (same requests in the same rows); then nothing of the previous
        step has to be known on the host, and each request's sample counter is one ahead of its
        delivered tokens.  The cache's bookkeeping moves on at once: what the step wrote is ordered on
        the stream before anything that could use those pages."""
        n = len(chunks)
        B = self.bucket_for(n)
        reqs = [r for r, _, _ in chunks]
        seqs = [r.seq for r in reqs]
        tokens = None if on_device_tokens else [r.token_at(s) for r, s, _ in chunks]
        temps = [max(0.0, float(r.params.temperature)) for r in reqs]
        if any(t > 0 for t in temps):
            from ..sampling.sampler import request_seed
            ahead = 1 if on_device_tokens else 0
            self.fill(B, seqs, tokens, temps, [request_seed(sampler.engine_seed, r) for r in reqs],
                      [len(r.output_ids) + ahead for r in reqs])
        else:
            self.fill(B, seqs, tokens)
        if on_device_tokens:
            self.feed_back(B)
        self.replay(B)
        turn = self._out_turn[B]
        self._out_turn[B] = (turn + 1) % self.RING
        host = self.out_host[B][turn]
        host[:n].copy_(self.tokens_out[B][:n], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        for (r, s, e), seq in zip(chunks, seqs):
            self.cache.commit(seq, e)
        return (host, ev, n)

    def read(self, handle) -> List[int]:
        """The step's sampled tokens (waits for that step only: its one device->host sync)."""
        host, ev, n = handle
        ev.synchronize()
        return host[:n].tolist()

    def run(self, chunks, sampler) -> Optional[List[int]]:
        """The engine's decode step.  None when the step is not a pure decode step that fits a bucket."""
        if not self.can_run(chunks):
            self.eager_steps += 1
            return None
        return self.read(self.launch(chunks, sampler))

    def stats(self):
        return {"graph_replays": self.replays, "graph_eager_steps": self.eager_steps, "graph_buckets": len(self.buckets)}
