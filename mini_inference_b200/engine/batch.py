"""The flat, unpadded batch of one step, and the ONE builder that makes it for eager steps and
for graph-replayed decode steps alike.

The reference builds a BatchMetadata per step (engine/core/model_runner.py:11-57) and a second,
padded set of buffers for its CUDA graphs (engine/core/cuda_graphs.py:93-122).  Here both are
the same thing: a table of int32 fields laid out in one buffer,

  per token    token_ids, positions, token_seg (which entry it belongs to),
               per cache group: slots (page * page_size + offset it is written to)
  per entry    seg_q_start (S+1 prefix sums), seg_pos0 (position of its first fed token),
               seg_kv_len (keys it sees at its last token), seg_slot (state slot = row of the
               request in the device block tables)
  logit_rows   flat rows whose logits are wanted
  sampling     temps, seeds, counters per entry (graph steps sample on the device)
  per group    tab_idx, tab_val: block-table entries that changed since the last step
               (cache/manager.py keeps the tables on the device; only changes travel)
  per part     whatever arrays the model's parts ask for through step_arrays (the attention
               mixer's kernel work lists, a toy mixer's own per-entry array, ...)

filled on the host in a pinned staging buffer taken from a small ring and sent to the device in
one copy.  An eager step sizes the fields to the step; a graph bucket fixes them once (a decode
step of B rows) and refills the same device buffer before every replay.

Only wanted rows reach the final norm and the head; the reference computes a row per chunk
and drops those of unfinished prompts (engine/custom_engine.py:139,155-157)."""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


class StepEntry:
    """A request's next tokens.  want: indices among these tokens whose logits are wanted."""
    __slots__ = ("seq", "tokens", "want")

    def __init__(self, seq, tokens: Sequence[int], want: Sequence[int] = ()):
        self.seq, self.tokens, self.want = seq, list(tokens), list(want)
        if not self.tokens:
            raise ValueError("a step entry needs at least one token")
        for w in self.want:
            if not 0 <= w < len(self.tokens):
                raise ValueError(f"want index {w} outside the entry's {len(self.tokens)} tokens")


class StepFacts:
    """What is known of a step on the host before anything is laid out: per entry its number of
    fed tokens, the position of the first, the keys it sees, its state slot.  This is what a
    part's step_arrays(facts) computes its own arrays from."""

    def __init__(self, lens, pos0, slots, tile: int):
        self.lens = np.asarray(lens, dtype=np.int32)
        self.pos0 = np.asarray(pos0, dtype=np.int32)
        self.slots = np.asarray(slots, dtype=np.int32)
        self.kv_len = self.pos0 + self.lens
        self.q_start = np.zeros(len(self.lens) + 1, dtype=np.int32)
        np.cumsum(self.lens, out=self.q_start[1:])
        self.num_entries, self.num_tokens = len(self.lens), int(self.q_start[-1])
        self.tile = tile


class BatchLayout:
    """Field name -> (offset, count) in the step's int32 buffer; every field starts on 16 bytes."""

    def __init__(self, fields):
        self.fields: Dict[str, tuple] = {}
        total = 0
        for name, count in fields:
            self.fields[name] = (total, count)
            total += (count + 3) // 4 * 4
        self.size = max(total, 4)

    def view(self, buf, name):
        a, n = self.fields[name]
        return buf[a:a + n]


class GroupView:
    """A mixer's view of the step for one cache group: the group's own arrays (slots, the device
    block table and which row of it each entry reads), the arrays its step_arrays hook asked
    for, and behind them everything the batch holds."""

    def __init__(self, batch, own: dict):
        self.__dict__.update(own)
        self.batch = batch

    def __getattr__(self, name):
        return getattr(self.__dict__["batch"], name)


class StepBatch:
    """Device views of one step's fields, plus the host-side facts."""

    def __init__(self, layout: BatchLayout, dev: torch.Tensor, cache, facts: StepFacts, shapes: dict,
                 num_logit_rows: int, max_kv_len: int, sampling: bool):
        self.layout, self.dev, self.cache = layout, dev, cache
        self.num_tokens, self.num_segs, self.tile = facts.num_tokens, facts.num_entries, facts.tile
        self.num_logit_rows = num_logit_rows
        self.max_kv_len, self.max_q_len = max_kv_len, int(facts.lens.max())
        self.host = {"seg_q_start": facts.q_start, "seg_pos0": facts.pos0, "seg_kv_len": facts.kv_len,
                     "seg_slot": facts.slots.tolist(), "lens": facts.lens}
        for name in ("token_ids", "positions", "token_seg", "seg_q_start", "seg_pos0", "seg_kv_len", "seg_slot", "logit_rows"):
            setattr(self, name, layout.view(dev, name))
        if sampling:
            self.temps = layout.view(dev, "temps").view(torch.float32)
            self.seeds, self.counters = layout.view(dev, "seeds"), layout.view(dev, "counters")
        self.extras: Dict[str, Dict[str, torch.Tensor]] = {}
        self.extras_host: Dict[str, Dict[str, np.ndarray]] = {}
        for (key, name), shape in shapes.items():
            self.extras.setdefault(key, {})[name] = layout.view(dev, f"x:{key}:{name}").view(shape)
        self._views = {}
        self.h2d_bytes = 0

    def group_view(self, group: int, key: Optional[str] = None) -> GroupView:
        """Arrays of cache group `group` (slots, block_table [rows, max_pages], table_rows) with the step arrays of
        the part key `key` beside them."""
        v = self._views.get((group, key))
        if v is None:
            g = self.cache.kv_groups[group]
            own = {"slots": self.layout.view(self.dev, f"slots{group}"), "block_table": g.device_table,
                   "table_rows": self.seg_slot, "max_pages": self.cache.max_pages_per_seq, "page_size": self.cache.page_size}
            own.update(self.extras.get(key, {}))
            v = self._views[(group, key)] = GroupView(self, own)
        return v

    def apply_table_updates(self, ops) -> None:
        """Write the changed block-table entries this step brought into the device tables (before any kernel reads them)."""
        for gi, g in enumerate(self.cache.kv_groups):
            idx = self.layout.view(self.dev, f"tab_idx{gi}")
            if idx.numel():
                ops.scatter_i32(g.device_table.view(-1), idx, self.layout.view(self.dev, f"tab_val{gi}"))


class BatchBuilder:
    RING = 4            # pinned staging buffers in flight

    def __init__(self, cache, device, hooks=None, tile: int = 64, vocab_size: Optional[int] = None):
        self.cache, self.device = cache, torch.device(device)
        self.hooks = dict(hooks or {})                # {key: step_arrays} of the model's parts
        self.tile, self.vocab_size = tile, vocab_size
        self.pinned = self.device.type == "cuda"
        self._ring: List[Optional[torch.Tensor]] = [None] * self.RING
        self._events: List[Optional[torch.cuda.Event]] = [None] * self.RING
        self._turn = 0
        # host-side range checks of everything a kernel will index with (positions, cache slots, table entries)
        self.debug_checks = os.environ.get("MI_DEBUG_CHECKS", "0") == "1"

    # ---------------------------------------------------------------- layout
    def _part_arrays(self, facts: StepFacts):
        arrays = {}
        for key, hook in self.hooks.items():
            for name, a in hook(facts).items():
                arrays[(key, name)] = np.ascontiguousarray(a, dtype=np.int32)
        return arrays

    def _layout(self, T, S, R, sampling, updates, part_arrays) -> BatchLayout:
        G = len(self.cache.kv_groups)
        fields = [("token_ids", T), ("positions", T), ("token_seg", T), ("seg_q_start", S + 1), ("seg_pos0", S),
                  ("seg_kv_len", S), ("seg_slot", S), ("logit_rows", R)]
        if sampling:
            fields += [("temps", S), ("seeds", S), ("counters", S)]
        for g in range(G):
            fields += [(f"slots{g}", T), (f"tab_idx{g}", updates[g]), (f"tab_val{g}", updates[g])]
        fields += [(f"x:{key}:{name}", a.size) for (key, name), a in part_arrays.items()]
        return BatchLayout(fields)

    def _staging(self, size: int):
        """The next pinned host buffer of the ring, at least `size` ints, free of its previous copy."""
        turn = self._turn
        self._turn = (turn + 1) % self.RING
        if self._events[turn] is not None:
            self._events[turn].synchronize()
            self._events[turn] = None
        buf = self._ring[turn]
        if buf is None or buf.numel() < size:
            buf = torch.zeros(max(size, 1024) * 5 // 4, dtype=torch.int32)
            if self.pinned:
                buf = buf.pin_memory()
            self._ring[turn] = buf
        return turn, buf

    def _send(self, turn, host, dev, start=0):
        if self.pinned:
            dev[start:].copy_(host[start:dev.numel()], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._events[turn] = ev
        else:
            dev[start:].copy_(host[start:dev.numel()])
        return (dev.numel() - start) * 4

    # ---------------------------------------------------------------- filling
    def _fill(self, layout, h, facts, seqs, token_ids, logit_rows, sampling, part_arrays, take_updates=True):
        """Write one step into the host array h (a numpy view of a staging buffer).  seqs: the live requests; entries
        of `facts` behind them are padding (graph buckets): position 0, one key on the null page, slot 0."""
        def put(name, values):
            a, n = layout.fields[name]
            h[a:a + n] = values
        S = facts.num_entries
        if token_ids is not None:
            put("token_ids", token_ids)
        positions = np.concatenate([np.arange(p, p + n, dtype=np.int32) for p, n in zip(facts.pos0, facts.lens)])
        put("positions", positions)
        put("token_seg", np.repeat(np.arange(S, dtype=np.int32), facts.lens))
        put("seg_q_start", facts.q_start)
        put("seg_pos0", facts.pos0)
        put("seg_kv_len", facts.kv_len)
        put("seg_slot", facts.slots)
        put("logit_rows", logit_rows)
        if sampling is not None:
            temps, seeds, counters = sampling
            put("temps", np.asarray(temps, dtype=np.float32).view(np.int32))
            put("seeds", np.asarray(seeds, dtype=np.uint32).view(np.int32))
            put("counters", np.asarray(counters, dtype=np.int32))
        elif "temps" in layout.fields:
            put("temps", 0)
        live = len(seqs)
        ps = self.cache.page_size
        for gi in range(len(self.cache.kv_groups)):
            slots = [self.cache.slots_for(gi, s, int(p), int(p + n)) for s, p, n in zip(seqs, facts.pos0, facts.lens)]
            if live < S:
                slots.append(np.zeros(int(facts.lens[live:].sum()), dtype=np.int32))
            put(f"slots{gi}", np.concatenate(slots))
            a, cap = layout.fields[f"tab_idx{gi}"]
            idx, val = self.cache.take_table_updates(gi, cap if take_updates else 0)
            h[a:a + len(idx)] = idx
            h[a + len(idx):a + cap] = 0
            b, _ = layout.fields[f"tab_val{gi}"]
            h[b:b + len(val)] = val
            h[b + len(val):b + cap] = 0
            if self.debug_checks:
                flat = np.concatenate(slots)
                assert flat.min() >= 0 and flat.max() < (self.cache.num_pages + 1) * ps, "a cache slot outside the pool"
                assert (val >= 0).all() and (val <= self.cache.num_pages).all(), "a block-table entry outside the pool"
                assert (idx >= 0).all() and (idx < (self.cache.max_seqs + 1) * self.cache.max_pages_per_seq).all()
        for (key, name), a in part_arrays.items():
            put(f"x:{key}:{name}", a.reshape(-1))
        if self.debug_checks:
            limit = self.cache.max_pages_per_seq * ps
            assert positions.min() >= 0 and facts.kv_len.max() <= limit, "a position beyond the longest sequence the cache admits"
            assert facts.slots.min() >= 0 and facts.slots.max() <= self.cache.max_seqs, "a state slot outside the slot table"

    def _check_tokens(self, ids):
        if self.vocab_size is not None and ids.size and (ids.min() < 0 or ids.max() >= self.vocab_size):
            raise ValueError(f"token id outside [0, {self.vocab_size})")

    # ---------------------------------------------------------------- eager steps
    def build(self, entries: List[StepEntry]) -> StepBatch:
        """The batch of an eager step: fields sized to the step, a fresh device buffer, one copy."""
        lens = [len(e.tokens) for e in entries]
        facts = StepFacts(lens, [e.seq.num_tokens for e in entries], [e.seq.slot for e in entries], self.tile)
        ids = np.fromiter((t for e in entries for t in e.tokens), dtype=np.int64, count=facts.num_tokens)
        self._check_tokens(ids)
        rows = np.asarray([int(facts.q_start[i]) + w for i, e in enumerate(entries) for w in e.want], dtype=np.int32)
        arrays = self._part_arrays(facts)
        updates = [self.cache.pending_table_updates(g) for g in range(len(self.cache.kv_groups))]
        layout = self._layout(facts.num_tokens, facts.num_entries, rows.size, False, updates, arrays)
        turn, host = self._staging(layout.size)
        self._fill(layout, host.numpy(), facts, [e.seq for e in entries], ids.astype(np.int32), rows, None, arrays)
        dev = torch.empty(layout.size, dtype=torch.int32, device=self.device)
        batch = StepBatch(layout, dev, self.cache, facts, {k: a.shape for k, a in arrays.items()}, rows.size,
                          int(facts.kv_len.max()), False)
        batch.h2d_bytes = self._send(turn, host, dev)
        batch.extras_host = self._host_extras(arrays)
        batch.entries = entries
        return batch

    @staticmethod
    def _host_extras(arrays):
        out = {}
        for (key, name), a in arrays.items():
            out.setdefault(key, {})[name] = a
        return out

    # ---------------------------------------------------------------- graph buckets
    def static(self, bucket: int, max_kv_len: int) -> StepBatch:
        """A decode-only batch of exactly `bucket` rows over a fixed device buffer (what a CUDA graph is captured
        on); refill() rewrites it before each replay.  Up to 2 * bucket + 8 block-table changes per group ride
        along (a new and a released page per row); more are flushed beforehand."""
        facts = StepFacts([1] * bucket, [0] * bucket, [0] * bucket, self.tile)
        arrays = self._part_arrays(facts)
        updates = [2 * bucket + 8] * len(self.cache.kv_groups)
        layout = self._layout(bucket, bucket, bucket, True, updates, arrays)
        dev = torch.zeros(layout.size, dtype=torch.int32, device=self.device)
        batch = StepBatch(layout, dev, self.cache, facts, {k: a.shape for k, a in arrays.items()}, bucket, max_kv_len, True)
        batch.bucket = bucket
        batch.array_sizes = {k: a.size for k, a in arrays.items()}
        # harmless rows until the first refill: one key on the null page
        h = np.zeros(layout.size, dtype=np.int32)
        self._fill(layout, h, facts, [], np.zeros(bucket, dtype=np.int32), np.arange(bucket, dtype=np.int32), None, arrays,
                   take_updates=False)
        dev.copy_(torch.from_numpy(h))
        return batch

    def refill(self, batch: StepBatch, seqs, tokens, sampling=None) -> int:
        """One decode step for the live requests `seqs` (padding behind them) into a static batch's buffer.
        tokens=None keeps the token ids that are already on the device.  Returns the bytes copied."""
        B, n = batch.bucket, len(seqs)
        pos = [s.num_tokens for s in seqs] + [0] * (B - n)
        facts = StepFacts([1] * B, pos, [s.slot for s in seqs] + [0] * (B - n), self.tile)
        arrays = self._part_arrays(facts)
        for k, a in arrays.items():
            if a.size != batch.array_sizes.get(k):
                raise RuntimeError(f"step array {k} changed size between capture and replay ({batch.array_sizes.get(k)} -> {a.size})")
        for gi in range(len(self.cache.kv_groups)):          # what does not fit beside the step goes first, on its own
            cap = batch.layout.fields[f"tab_idx{gi}"][1]
            if self.cache.pending_table_updates(gi) > cap:
                self.flush_table_updates(gi, keep=cap)
        ids = None
        if tokens is not None:
            ids = np.zeros(B, dtype=np.int32)
            ids[:n] = tokens
        if sampling is not None:
            temps, seeds, counters = sampling
            pad = [0] * (B - n)
            sampling = (list(temps) + pad, list(seeds) + pad, list(counters) + pad)
        turn, host = self._staging(batch.layout.size)
        self._fill(batch.layout, host.numpy(), facts, list(seqs), ids, np.arange(B, dtype=np.int32), sampling, arrays)
        batch.host.update(seg_pos0=facts.pos0, seg_kv_len=facts.kv_len, seg_slot=facts.slots.tolist())
        batch.extras_host = self._host_extras(arrays)
        start = 0 if tokens is not None else batch.layout.fields["positions"][0]
        return self._send(turn, host, batch.dev, start)

    def flush_table_updates(self, gi: int, keep: int = 0, ops=None) -> None:
        """Send all but `keep` of group gi's pending block-table changes in a copy of their own."""
        n = self.cache.pending_table_updates(gi) - keep
        if n <= 0:
            return
        idx, val = self.cache.take_table_updates(gi, n)
        turn, host = self._staging(2 * n)
        h = host.numpy()
        h[:n], h[n:2 * n] = idx, val
        dev = torch.empty(2 * n, dtype=torch.int32, device=self.device)
        self._send(turn, host, dev)
        (ops or self.ops).scatter_i32(self.cache.kv_groups[gi].device_table.view(-1), dev[:n], dev[n:])

    ops = None          # set by the runner: the kernel namespace that applies flushed updates
