"""Pure-decode steps replayed as CUDA graphs, one graph per batch-size bucket.

The reference does the same for its decode steps (engine/core/cuda_graphs.py:8-139): fixed
device buffers, pinned staging, one graph per bucket, rows beyond the live batch padded with
harmless work (token 0, position 0, a one-key context on a scratch page).  Differences here:
all metadata of a step travels in ONE pinned buffer and one copy, laid out and filled by the
same builder as an eager step's (engine/batch.py: BatchBuilder.static / refill); the block
tables stay on the device and only their changed entries ride along; sampling is inside the
graph, so a step returns token ids, not logits; padding rows use the cache's null page 0,
which no request ever owns.  The number of key splits of the attention kernel is fixed per
bucket from the longest sequence the cache admits, so the grid depends on the bucket only
(engine/core/cuda_graphs.py:55); each request still cuts its own length."""
from __future__ import annotations

from typing import List, Optional

import torch


DEFAULT_BUCKETS = [1, 2, 4, 8, 12, 16, 24, 32, 40, 48, 56, 64, 80, 96, 112, 128, 160, 192, 224, 256]


class DecodeGraphs:
    RING = 4            # pinned staging buffers in flight

    def __init__(self, runner, max_batch: int, buckets: Optional[List[int]] = None):
        self.runner, self.cache, self.ops = runner, runner.cache, runner.ops
        self.builder = runner.builder
        self.device = runner.device
        self.buckets = [b for b in (buckets or DEFAULT_BUCKETS) if b < max_batch] + [max_batch]
        self.max_batch = max_batch
        self.batches, self.graphs, self.tokens_out, self.logits_out, self.launches = {}, {}, {}, {}, {}
        self.last_h2d_bytes = 0
        self.out_host, self._out_turn = {}, {}
        self.replays = self.eager_steps = 0
        self.capture_s = 0.0

    # ---------------------------------------------------------------- capture
    def _forward(self, batch):
        logits = self.runner.forward(batch)
        return self.ops.sample(logits, batch.temps, batch.seeds, batch.counters), logits

    def capture(self):
        import time
        t0 = time.perf_counter()
        max_len = self.cache.max_pages_per_seq * self.cache.page_size
        pool = None
        for B in sorted(self.buckets, reverse=True):            # largest first: smaller graphs reuse its pool
            batch = self.builder.static(B, max_len)              # harmless rows: one key on the null page
            self.out_host[B] = [torch.zeros(B, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
            self._out_turn[B] = 0
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
                out, logits = self._forward(batch)
            self.launches[B] = self.ops.launches - before
            pool = pool or graph.pool()
            self.batches[B], self.graphs[B], self.tokens_out[B] = batch, graph, out
            self.logits_out[B] = logits                          # float32 [B, vocab] of the last replay (valid until the next)
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
        previous step's samples, see feed_back).  Returns the bytes copied."""
        sampling = None if temps is None else (temps, seeds, counters)
        self.last_h2d_bytes = self.builder.refill(self.batches[B], seqs, tokens, sampling)
        return self.last_h2d_bytes

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
