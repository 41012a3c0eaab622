"""Cache manager: pages of keys and values per cache group, a block table per request and
group, and slots for fixed-size per-request state.

What the reference does in one PagedAllocator + KVCache for one uniform tensor
(engine/core/kv_cache.py:124-301, 305-437) is done here per GROUP: execution steps whose
mixers need the same thing (kv heads, head size, window) share a pool of pages and one block
table per request.  A group with a window gives a page back as soon as every key in it lies
before the window of the next position.  Storage of a group is
[steps, 2 (k, v), pages + 1, kv_heads, page_size, head_dim]: one (page, kv head) is a
contiguous page_size x head_dim tile that a kernel can fetch in one bulk copy.

Call order for a request: admit -> (ensure -> commit)* -> free.
  ensure(seq, n)  pages for positions < n exist in every group, all or nothing
                  (the reference's reserve() keeps a partial grab, kv_cache.py:216-224)
  commit(seq, n)  n tokens are now cached; pages a window has passed are given back

Block tables live twice: a host array per group ([slots + 1, max pages], the truth) and a
device copy of the same shape that the attention kernels read, a request's row being its
state slot.  The reference rebuilds and copies a padded table every step
(kv_cache.py:403-420); here every change of a host entry is noted, and a step sends only the
entries that changed since the last one (take_table_updates): a decode step sends at most a
new page and a released page per request, whatever the context length.
"""
from __future__ import annotations

import math
from typing import List, Optional

import numpy as np
import torch

from ..parts.base import KVCacheNeed, LayerCache, StateNeed
from .page_pool import PagePool
from .state_slots import StateSlots


class SeqCache:
    """One live request's hold on the cache."""
    __slots__ = ("seq_id", "slot", "num_tokens", "num_pages", "first_live", "alive")

    def __init__(self, seq_id, slot, num_groups):
        self.seq_id, self.slot = seq_id, slot
        self.num_tokens = 0                              # tokens committed
        self.num_pages = [0] * num_groups                # table entries filled (by page index)
        self.first_live = [0] * num_groups               # first page index not yet given back
        self.alive = True


class _Group:
    def __init__(self, need, steps):
        self.need, self.steps = need, steps
        self.pool: Optional[PagePool] = None
        self.storage = None                              # kv groups
        self.tables: Optional[np.ndarray] = None         # [slots + 1, max_pages] int32 (host)
        self.device_table = None                         # the same on the device, kept current by update lists
        self.dirty: dict = {}                            # flat index -> None, in the order the entries changed


class CacheManager:
    def __init__(self, needs, page_size: int, num_pages: int, max_seqs: int, max_seq_len: int,
                 dtype=torch.bfloat16, device="cpu", watermark: float = 0.0, allocate: bool = True):
        """needs: per execution step a KVCacheNeed, a StateNeed or None (DecoderModel.cache_needs)."""
        self.page_size, self.num_pages, self.max_seqs = page_size, num_pages, max_seqs
        self.max_pages_per_seq = math.ceil(max_seq_len / page_size)
        self.dtype, self.device = dtype, torch.device(device)
        # engine/core/kv_cache.py:132: pages kept free at admission so running requests can grow
        self.watermark_pages = max(1, math.ceil(num_pages * watermark)) if watermark > 0 else 0
        self.slots = StateSlots(max_seqs)
        self.seqs = {}
        self.kv_groups: List[_Group] = []
        self.state_groups: List[_Group] = []
        self.layer_caches: List[Optional[LayerCache]] = [None] * len(needs)
        by_need = {}
        for step, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, KVCacheNeed):
                g = by_need.get(need)
                if g is None:
                    g = by_need[need] = _Group(need, [])
                    self.kv_groups.append(g)
                g.steps.append(step)
            elif isinstance(need, StateNeed):
                g = _Group(need, [step])
                self.state_groups.append(g)
            else:
                raise TypeError(f"execution step {step}: unknown cache need {need!r}")
        for gi, g in enumerate(self.kv_groups):
            g.pool = PagePool(num_pages)
            g.tables = np.zeros((max_seqs + 1, self.max_pages_per_seq), dtype=np.int32)
            if allocate:
                g.device_table = torch.zeros((max_seqs + 1, self.max_pages_per_seq), dtype=torch.int32, device=self.device)
                n = g.need
                g.storage = torch.zeros((len(g.steps), 2, num_pages + 1, n.num_kv_heads, page_size, n.head_dim),
                                        dtype=dtype, device=self.device)
            for j, step in enumerate(g.steps):
                k = g.storage[j, 0] if allocate else None
                v = g.storage[j, 1] if allocate else None
                self.layer_caches[step] = LayerCache(gi, k=k, v=v)
        for g in self.state_groups:
            if allocate:
                sd = dtype if g.need.dtype == "compute" else torch.float32
                g.storage = torch.zeros((max_seqs + 1, *g.need.shape), dtype=sd, device=self.device)
            self.layer_caches[g.steps[0]] = LayerCache(-1, state=g.storage)

    # ---------------------------------------------------------------- sizes
    @property
    def capacity_tokens(self) -> int:
        return self.num_pages * self.page_size

    def bytes_per_token(self) -> int:
        """Bytes of cache one token occupies over all groups (engine/core/kv_cache.py:22-30)."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * len(g.steps) * g.need.num_kv_heads * g.need.head_dim * el for g in self.kv_groups)

    def state_bytes_per_seq(self) -> int:
        """Bytes of fixed-size state one live request occupies over all state groups."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(math.prod(g.need.shape) * (el if g.need.dtype == "compute" else 4) for g in self.state_groups)

    def pages_for(self, num_tokens: int) -> int:
        return math.ceil(num_tokens / self.page_size)

    def peak_pages(self, g: "_Group", total_len: int, max_span: Optional[int]) -> int:
        """Most pages of group g that a request of total_len tokens holds at one time when no step feeds it more
        than max_span tokens (None: a step may feed all of them).  A windowed group keeps the pages that the
        window of the next position reaches plus those of the span being written."""
        full = self.pages_for(total_len)
        W = g.need.window
        if W is None or max_span is None:
            return full
        return min(full, self.pages_for(W + max_span) + 1)

    def _first_needed_page(self, g: _Group, num_cached: int) -> int:
        """First page index that holds a key some position >= num_cached may still read."""
        W = g.need.window
        if W is None:
            return 0
        return max(0, num_cached - W + 1) // self.page_size

    # ---------------------------------------------------------------- admission and growth
    def free_pages(self) -> int:
        return min((g.pool.num_free for g in self.kv_groups), default=self.num_pages)

    def can_admit(self, total_len: int, max_span: Optional[int] = None) -> bool:
        """engine/core/kv_cache.py:192-197: the pages the request will hold plus the watermark must be free, in
        every group (a windowed group is charged what it holds at its peak, see peak_pages), and a state slot."""
        if self.slots.num_free == 0 or total_len > self.max_pages_per_seq * self.page_size:
            return False
        return all(self.peak_pages(g, total_len, max_span) + self.watermark_pages <= g.pool.num_free
                   for g in self.kv_groups)

    def admit(self, seq_id, total_len: Optional[int] = None, max_span: Optional[int] = None) -> Optional[SeqCache]:
        if seq_id in self.seqs:
            raise RuntimeError(f"request {seq_id!r} is already admitted")
        if total_len is not None and not self.can_admit(total_len, max_span):
            return None
        slot = self.slots.claim()
        if slot is None:
            return None
        seq = SeqCache(seq_id, slot, len(self.kv_groups))
        self.seqs[seq_id] = seq
        for g in self.state_groups:
            if g.storage is not None:
                g.storage[slot].zero_()
        return seq

    def ensure(self, seq: SeqCache, num_tokens: int) -> bool:
        """Pages for positions < num_tokens in every group; takes nothing if any group is short."""
        want = self.pages_for(num_tokens)
        if want > self.max_pages_per_seq:
            return False
        for gi, g in enumerate(self.kv_groups):
            if want - seq.num_pages[gi] > g.pool.num_free:
                return False
        for gi, g in enumerate(self.kv_groups):
            row = g.tables[seq.slot]
            base = seq.slot * self.max_pages_per_seq
            for idx in range(seq.num_pages[gi], want):
                row[idx] = g.pool.take()
                g.dirty[base + idx] = None
            seq.num_pages[gi] = max(seq.num_pages[gi], want)
        return True

    def commit(self, seq: SeqCache, num_tokens: int) -> None:
        seq.num_tokens = num_tokens
        for gi, g in enumerate(self.kv_groups):
            keep_from = min(self._first_needed_page(g, num_tokens), seq.num_pages[gi])
            row = g.tables[seq.slot]
            base = seq.slot * self.max_pages_per_seq
            for idx in range(seq.first_live[gi], keep_from):
                g.pool.give(int(row[idx]))
                row[idx] = PagePool.NULL_PAGE
                g.dirty[base + idx] = None
            seq.first_live[gi] = max(seq.first_live[gi], keep_from)

    def free(self, seq: SeqCache) -> None:
        """Give back everything the request holds (finish, preemption, abort, failed admission:
        engine/core/scheduler.py:87,101,209-219)."""
        if not seq.alive:
            raise RuntimeError(f"request {seq.seq_id!r} freed twice")
        seq.alive = False
        for gi, g in enumerate(self.kv_groups):
            row = g.tables[seq.slot]
            base = seq.slot * self.max_pages_per_seq
            for idx in range(seq.first_live[gi], seq.num_pages[gi]):
                g.pool.give(int(row[idx]))
                row[idx] = PagePool.NULL_PAGE
                g.dirty[base + idx] = None
        self.slots.release(seq.slot)
        del self.seqs[seq.seq_id]

    # ---------------------------------------------------------------- what a step reads
    def slots_for(self, gi: int, seq: SeqCache, start: int, end: int) -> np.ndarray:
        """Flat cache positions page * page_size + offset of tokens start..end-1
        (engine/core/kv_cache.py:269-272)."""
        pos = np.arange(start, end, dtype=np.int64)
        pages = self.kv_groups[gi].tables[seq.slot, pos // self.page_size].astype(np.int64)
        return (pages * self.page_size + pos % self.page_size).astype(np.int32)

    def table_rows(self, gi: int, seqs, num_cols: int) -> np.ndarray:
        return self.kv_groups[gi].tables[[s.slot for s in seqs], :num_cols]

    def pending_table_updates(self, gi: int) -> int:
        return len(self.kv_groups[gi].dirty)

    def take_table_updates(self, gi: int, limit: Optional[int] = None):
        """(flat indices, values) of up to `limit` block-table entries of group gi whose host value changed since they
        were last taken, oldest change first; the caller writes them into the device table before the kernels of
        its step run.  An entry changed twice is sent once, with its current value."""
        g = self.kv_groups[gi]
        n = len(g.dirty) if limit is None else min(limit, len(g.dirty))
        if n == len(g.dirty):
            idx = np.fromiter(g.dirty, dtype=np.int64, count=n)
            g.dirty = {}
        else:
            keys = list(g.dirty)[:n]
            for k in keys:
                del g.dirty[k]
            idx = np.asarray(keys, dtype=np.int64)
        return idx.astype(np.int32), g.tables.reshape(-1)[idx]

    # ---------------------------------------------------------------- checks and numbers
    def check_invariants(self) -> None:
        """No page lost, none held twice, free list and tables disjoint (used by the tests)."""
        for gi, g in enumerate(self.kv_groups):
            held = []
            for seq in self.seqs.values():
                row = g.tables[seq.slot]
                live = [int(p) for p in row[seq.first_live[gi]:seq.num_pages[gi]]]
                assert all(p != 0 for p in live), f"group {gi}: a live table entry is the null page"
                assert not row[:seq.first_live[gi]].any() and not row[seq.num_pages[gi]:].any(), \
                    f"group {gi}: table entries outside the live range are not null"
                held += live
            for slot in range(g.tables.shape[0]):
                if slot not in {s.slot for s in self.seqs.values()}:
                    assert not g.tables[slot].any(), f"group {gi}: row {slot} belongs to nobody and is not null"
            if g.device_table is not None:
                mirror = g.device_table.cpu().numpy().reshape(-1).copy()
                for k in g.dirty:
                    mirror[k] = g.tables.reshape(-1)[k]
                assert (mirror == g.tables.reshape(-1)).all(), f"group {gi}: device table differs beyond the noted changes"
            free = list(g.pool.free)
            assert len(set(held)) == len(held), f"group {gi}: a page is held twice"
            assert len(set(free)) == len(free), f"group {gi}: a page is in the free list twice"
            assert not set(held) & set(free), f"group {gi}: a held page is also free"
            assert len(held) + len(free) == g.pool.num_pages, f"group {gi}: a page is lost"
            assert 0 not in free
            for p in range(1, g.pool.num_pages + 1):
                assert g.pool.ref[p] == (1 if p in set(held) else 0)

    def stats(self) -> dict:
        """Names after engine/core/kv_cache.py:283-301,427-437."""
        used = max((g.pool.num_used for g in self.kv_groups), default=0)
        stored = sum(s.num_tokens for s in self.seqs.values())
        return {
            "kv_capacity_tokens": self.capacity_tokens,
            "kv_reserved_tokens": used * self.page_size,
            "kv_used_tokens": stored,
            "kv_free_tokens": self.free_pages() * self.page_size,
            "kv_blocks_used": used,
            "kv_blocks_total": self.num_pages,
            "kv_block_size": self.page_size,
            "kv_groups": len(self.kv_groups),
            "state_slots_used": self.max_seqs - self.slots.num_free,
        }
