"""mi_attn_decode_noalloc: the decode-attention entry point for callers that cannot allocate
device memory (embedders running inside another framework's memory plan, loops in which
allocation is forbidden after start-up, plug-ins that are only handed pointers).  Its scratch
is an 8 MiB array inside the library image, so the only memory it touches beyond its inputs
and outputs is that array.  Called here through its exported C symbol, twice in a row on
different problems (the array keeps the first call's contents), and compared with the
ordinary entry point, which takes its scratch from the framework's allocator.  This file sorts
last so that a run that stops at the first failure has already run every other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def problem(B, ctx_lens, H, KV, D, page, seed):
    import numpy as np
    from tests.test_kernels_gpu import make_meta
    g = torch.Generator().manual_seed(seed)
    meta = make_meta(page, [(n - 1, 1) for n in ctx_lens], 1 + sum(-(-n // page) for n in ctx_lens), seed=seed)
    pages = 2 + sum(-(-n // page) for n in ctx_lens)
    q = torch.randn(B, H * D, generator=g).to(torch.bfloat16).to(DEV)
    kc = torch.randn(pages, KV, page, D, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(pages, KV, page, D, generator=g).to(torch.bfloat16).to(DEV)
    return meta, q, kc, vc


def call_noalloc(lib, q, kc, vc, meta, H, KV, D, splits, window=0, check_free=False):
    """check_free: compare the DRIVER's free-memory figure around the call (it sees a cudaMalloc inside the library,
    which the framework allocator's counters cannot); only meaningful once the library's kernels are loaded, so the
    first call of a test runs without it."""
    out = torch.full((q.shape[0], H * D), float("nan"), dtype=torch.bfloat16, device=DEV)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    free_before = torch.cuda.mem_get_info()[0]
    rc = lib.mi_attn_decode_noalloc(p(q), q.stride(0), p(kc), p(vc), p(out), p(meta.decode_segs), meta.decode_segs.shape[0],
                                    p(meta.seg_q_start), p(meta.seg_kv_len), p(meta.block_table), meta.max_pages,
                                    H, KV, D, meta.page_size, splits, ctypes.c_float(D ** -0.5), window, stream)
    torch.cuda.synchronize()
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == before     # the call allocated nothing
    if check_free:
        assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated during the call"
    return rc, out


def test_no_alloc_decode_attention_matches_ordinary_entry_point():
    from mini_inference_b200.ops import get_ops, load_library
    from tests.ref_ops import TorchRefOps
    lib = load_library()
    lib.mi_attn_decode_noalloc_strerror.restype = ctypes.c_char_p
    ops = get_ops(DEV)
    H, KV, D, page = 32, 8, 128, 16
    # two calls in a row: the second is smaller and uses fewer splits, so stale partials of the
    # first call lie in the array beside and behind what the second call writes
    for call, (lens, splits, seed) in enumerate((([700, 33, 1, 260, 129], 5, 1), ([90, 517], 2, 2), ([300], 1, 3))):
        meta, q, kc, vc = problem(len(lens), lens, H, KV, D, page, seed)
        rc, got = call_noalloc(lib, q, kc, vc, meta, H, KV, D, splits, check_free=call > 0)
        assert rc == 0, lib.mi_attn_decode_noalloc_strerror(rc).decode()
        ops.force_splits = splits
        try:
            want = ops.paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, None)
        finally:
            ops.force_splits = None
        ref = TorchRefOps().paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, None)
        assert not torch.isnan(got.float()).any()
        assert ((got.float() - want.float()).abs().max() / want.float().abs().max()).item() < 1.6e-2
        assert ((got.float() - ref.float()).abs().max() / ref.float().abs().max()).item() < 1.6e-2
    # refusals: too large for the built-in scratch; a shape the kernel does not take
    meta, q, kc, vc = problem(2, [40, 50], H, KV, D, page, 4)
    rc, _ = call_noalloc(lib, q, kc, vc, meta, H, KV, D, splits=300)
    assert rc == -3 and b"8 MiB" in lib.mi_attn_decode_noalloc_strerror(rc)
    meta2, q2, kc2, vc2 = problem(1, [40], 4, 2, 48, page, 5)
    rc, _ = call_noalloc(lib, q2, kc2, vc2, meta2, 4, 2, 48, splits=2)
    assert rc == -2 and b"head size" in lib.mi_attn_decode_noalloc_strerror(rc)
