"""The cache manager alone: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; state slots; all-or-nothing growth."""
import random

import pytest

from mini_inference_b200.cache import CacheManager, PagePool, StateSlots
from mini_inference_b200.parts.base import KVCacheNeed, StateNeed

FULL = KVCacheNeed(2, 16, None)
WIN = KVCacheNeed(2, 16, 10)


def manager(needs, pages=12, page=4, seqs=4, watermark=0.0):
    return CacheManager(needs, page, pages, seqs, 4096, allocate=False, watermark=watermark)


def test_pages_fifo_and_counts():
    """engine/core/kv_cache.py: 20 tokens -> 2 pages of 16, 33 -> 3; freed pages go to the back."""
    m = manager([FULL], pages=8, page=16)
    s = m.admit("a")
    assert m.ensure(s, 20) and s.num_pages == [2]
    assert m.ensure(s, 33) and s.num_pages == [3]
    slots = m.slots_for(0, s, 0, 33)
    assert len(set(slots.tolist())) == 33
    assert list(m.kv_groups[0].tables[s.slot, :3]) == [1, 2, 3]
    m.free(s)
    assert m.free_pages() == 8
    t = m.admit("b")
    m.ensure(t, 16)
    assert m.kv_groups[0].tables[t.slot, 0] == 4            # FIFO: pages 1..3 wait at the back
    m.check_invariants()


def test_ensure_is_all_or_nothing_across_groups():
    m = manager([FULL, WIN, FULL], pages=3, page=4)
    assert len(m.kv_groups) == 2 and m.kv_groups[0].steps == [0, 2]
    a = m.admit("a")
    assert m.ensure(a, 8)
    b = m.admit("b")
    assert not m.ensure(b, 8)                                # needs 2 pages, 1 left
    assert b.num_pages == [0, 0] and m.free_pages() == 1
    assert m.ensure(b, 4)
    m.check_invariants()


def test_window_gives_pages_back():
    m = manager([WIN], pages=6, page=4)                      # window 10
    s = m.admit("a")
    for n in range(1, 41):
        assert m.ensure(s, n)
        m.commit(s, n)
        m.check_invariants()
        # the next position n reads keys > n - 10: pages wholly below are gone
        assert s.first_live[0] == max(0, n - 10 + 1) // 4
        assert m.kv_groups[0].pool.num_used <= 4
    m.free(s)
    assert m.free_pages() == 6


def test_double_free_and_double_admit_are_errors():
    m = manager([FULL])
    s = m.admit("a")
    with pytest.raises(RuntimeError):
        m.admit("a")
    m.free(s)
    with pytest.raises(RuntimeError):
        m.free(s)
    p = PagePool(2)
    x = p.take()
    p.give(x)
    with pytest.raises(RuntimeError):
        p.give(x)
    sl = StateSlots(1)
    k = sl.claim()
    assert sl.claim() is None
    sl.release(k)
    with pytest.raises(RuntimeError):
        sl.release(k)


def test_admission_watermark_and_slots():
    m = manager([FULL], pages=10, page=4, seqs=2, watermark=0.1)      # watermark 1 page
    assert m.can_admit(36) and not m.can_admit(37)
    a, b = m.admit("a", 8), m.admit("b", 8)
    assert a and b and m.admit("c", 4) is None                          # no state slot left
    m.free(a)
    assert m.admit("c", 4) is not None


def test_state_slots_are_zeroed_on_claim():
    import torch
    m = CacheManager([StateNeed((3,)), FULL], 4, 4, 2, 64, dtype=torch.float32, device="cpu")
    s = m.admit("a")
    state = m.layer_caches[0].state
    assert state.shape == (3, 3)
    state[s.slot] += 5
    m.free(s)
    t = m.admit("b")
    assert t.slot == s.slot and float(state[t.slot].abs().sum()) == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_invariants(seed):
    rng = random.Random(seed)
    m = manager([FULL, WIN, FULL], pages=20, page=4, seqs=5)
    live, n_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            s = m.admit(n_id)
            if s is not None:
                live[n_id] = s
            n_id += 1
        elif op < 0.8 and live:
            s = rng.choice(list(live.values()))
            n = s.num_tokens + rng.randint(1, 9)
            if m.ensure(s, n):
                m.commit(s, n)
        elif live:
            k = rng.choice(list(live))
            m.free(live.pop(k))
        m.check_invariants()
    for s in live.values():
        m.free(s)
    m.check_invariants()
    assert m.free_pages() == 20 and m.slots.num_free == 5


def test_block_table_changes_are_noted_and_taken_once():
    """The device copy of a block table is kept current by change lists: every entry that changed on the host since the
    last take comes out once, with its current value, oldest change first; a limit leaves the rest for the next take."""
    import numpy as np
    m = manager([FULL, WIN], pages=20, page=4, seqs=3)       # window 10
    P = m.max_pages_per_seq
    mirror = [np.zeros_like(g.tables).reshape(-1) for g in m.kv_groups]

    def sync(limit=None):
        for gi in range(2):
            idx, val = m.take_table_updates(gi, limit)
            assert len(set(idx.tolist())) == len(idx)
            mirror[gi][idx] = val
    a, b = m.admit("a"), m.admit("b")
    m.ensure(a, 9)
    m.ensure(b, 3)
    assert m.pending_table_updates(0) == 4 and m.pending_table_updates(1) == 4
    idx, val = m.take_table_updates(0, 3)                     # a limit: the oldest three
    assert idx.tolist() == [a.slot * P, a.slot * P + 1, a.slot * P + 2] and m.pending_table_updates(0) == 1
    mirror[0][idx] = val
    sync()
    assert all((mirror[gi] == m.kv_groups[gi].tables.reshape(-1)).all() for gi in range(2))
    for n in range(10, 40):                                   # growth: at most one new and (window) one released entry a step
        m.ensure(a, n)
        m.commit(a, n)
        assert m.pending_table_updates(0) <= 1 and m.pending_table_updates(1) <= 2
        sync()
        assert all((mirror[gi] == m.kv_groups[gi].tables.reshape(-1)).all() for gi in range(2))
    m.free(a)                                                 # its live entries become null: noted too
    assert m.pending_table_updates(0) == 10
    m.ensure(b, 5)
    sync()
    assert all((mirror[gi] == m.kv_groups[gi].tables.reshape(-1)).all() for gi in range(2))
    assert not m.kv_groups[0].tables[a.slot].any()
    m.check_invariants()


def test_admission_counts_what_a_request_holds_at_its_peak():
    """A windowed group holds at most the window plus one step's span in pages, so with a bounded span a long request
    is charged that, not its whole length; an unbounded step (whole prompts) is charged in full.  State is counted in bytes."""
    import torch
    m = CacheManager([FULL, WIN, StateNeed((3, 8), "float32"), StateNeed((5,), "compute")], 4, 30, 2, 4096,
                     dtype=torch.bfloat16, allocate=False)
    full, win = m.kv_groups
    assert m.peak_pages(full, 100, 8) == 25 and m.peak_pages(win, 100, None) == 25
    assert m.peak_pages(win, 100, 8) == 6                     # ceil((10 + 8) / 4) + 1
    assert m.peak_pages(win, 9, 8) == 3                       # never more than the request itself
    assert m.can_admit(100, 8)
    a = m.admit("a", 100, 8)
    m.ensure(a, 8)
    for g in m.kv_groups:                                     # leave 26 free pages in the full group, 5 in the windowed one
        pass
    while win.pool.num_free > 5:
        win.pool.take()
    assert not m.can_admit(100, 8) and m.can_admit(9, 8)      # 6 > 5 free pages in the windowed group; 3 fit
    assert m.state_bytes_per_seq() == 3 * 8 * 4 + 5 * 2
    assert m.bytes_per_token() == 2 * 2 * 2 * 16 * 2


def test_a_decode_step_sends_changes_not_tables():
    """The metadata of a graph-replayed decode step does not grow with the longest sequence the cache admits: the block
    tables stay on the device, a step carries the entries that changed (at most a new and a released page per row)."""
    import torch
    from mini_inference_b200.engine.batch import BatchBuilder
    from tests.ref_ops import TorchRefOps
    sizes = []
    for max_len in (2048, 32768):
        m = CacheManager([FULL, WIN], 16, 4096, 64, max_len, dtype=torch.float32, device="cpu")
        b = BatchBuilder(m, "cpu")
        b.ops = TorchRefOps()
        seqs = [m.admit(i) for i in range(8)]
        for i, s in enumerate(seqs):
            m.ensure(s, 1000 + 16 * i)
            m.commit(s, 1000 + 16 * i)
        batch = b.static(8, max_len)
        b.flush_table_updates(0), b.flush_table_updates(1)        # what prompts left behind travels before the first decode step
        for step in range(40):
            for s in seqs:
                assert m.ensure(s, s.num_tokens + 1)
            nbytes = b.refill(batch, seqs, [1] * 8)
            batch.apply_table_updates(b.ops)
            for s in seqs:
                m.commit(s, s.num_tokens + 1)
        m.check_invariants()                                       # the device tables equal the host's
        sizes.append(nbytes)
    assert sizes[0] == sizes[1] and sizes[1] < 1024, sizes
