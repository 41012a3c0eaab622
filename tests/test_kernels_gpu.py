"""Each CUDA kernel alone against its plain PyTorch reference (tests/ref_ops.py), at sizes
other than the engine's tiny configurations: widths and vocabularies that are no power of
two, head sizes in steps of 16, odd head counts and groups."""
import types

import numpy as np
import pytest
import torch

from tests.ref_ops import TorchRefOps
from tests.ref_sampling import perturbed_scores

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def ops():
    from mini_inference_b200.ops import get_ops
    return get_ops(DEV)


def tol(dtype):
    return 2e-6 if dtype == torch.float32 else 1.6e-2


def close(a, b, dtype, scale=None):
    a, b = a.float(), b.float()
    s = scale if scale is not None else b.abs().max().clamp_min(1e-6)
    err = ((a - b).abs().max() / s).item()
    assert err < tol(dtype), f"relative error {err}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(72, 301), (2560, 1000), (100, 77)])
def test_embedding(ops, dtype, hidden, vocab):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, hidden, generator=g).to(dtype).to(DEV)
    ids = torch.randint(0, vocab, (37,), generator=g).to(torch.int32).to(DEV)
    assert torch.equal(ops.embedding(ids, table), TorchRefOps().embedding(ids, table))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 2560, 1001])
@pytest.mark.parametrize("w32", [False, True])
def test_add_rmsnorm(ops, dtype, hidden, w32):
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(19, hidden, generator=g) * 3).to(dtype).to(DEV)
    d = torch.randn(19, hidden, generator=g).to(dtype).to(DEV)
    w = (torch.rand(hidden, generator=g) + 0.5).to(torch.float32 if w32 else dtype).to(DEV)
    ref = TorchRefOps()
    for delta in (None, d):
        x1, x2 = x.clone(), x.clone()
        y1 = ops.add_rmsnorm(x1, delta, w, 1e-5)
        y2 = ref.add_rmsnorm(x2, delta, w, 1e-5)
        assert torch.equal(x1, x2)
        close(y1, y2, dtype)
        rows = torch.tensor([3, 0, 18, 7], dtype=torch.int32, device=DEV)
        x3 = x.clone()
        y3 = ops.add_rmsnorm(x3, delta, w, 1e-5, rows)
        assert torch.equal(x3, x)
        close(y3, ref.add_rmsnorm(x.clone(), delta, w, 1e-5, rows), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [64, 2560, 4096, 5120, 1001])
def test_add_rmsnorm_many_rows(ops, dtype, hidden):
    """Row counts at which the one-warp-per-row kernel is used (from 1,024 rows), and just below."""
    g = torch.Generator().manual_seed(11)
    ref = TorchRefOps()
    w = (torch.rand(hidden, generator=g) + 0.5).to(dtype).to(DEV)
    for n in (203, 1027):
        x = (torch.randn(n, hidden, generator=g) * 2).to(dtype).to(DEV)
        d = torch.randn(n, hidden, generator=g).to(dtype).to(DEV)
        x1, x2 = x.clone(), x.clone()
        close(ops.add_rmsnorm(x1, d, w, 1e-6), ref.add_rmsnorm(x2, d, w, 1e-6), dtype)
        assert torch.equal(x1, x2)
        rows = torch.arange(0, n, 2, dtype=torch.int32, device=DEV)
        close(ops.add_rmsnorm(x.clone(), None, w, 1e-6, rows), ref.add_rmsnorm(x.clone(), None, w, 1e-6, rows), dtype)
    rows = torch.arange(0, 2 * 1100, 2, dtype=torch.int32, device=DEV) % 1027      # many selected rows of few
    close(ops.add_rmsnorm(x.clone(), d, w, 1e-6, rows), ref.add_rmsnorm(x.clone(), d, w, 1e-6, rows), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,D,page", [(4, 2, 16, 8), (32, 8, 128, 16), (5, 1, 48, 16)])
def test_qk_norm_rope_cache_long_prompt(ops, dtype, H, KV, D, page):
    """Token counts at which the one-block-per-token kernel is used."""
    g = torch.Generator().manual_seed(12)
    meta = make_meta(page, [(3, 300), (100, 41)], 64, seed=5)
    qkv = torch.randn(meta.num_tokens, (H + 2 * KV) * D, generator=g).to(dtype).to(DEV)
    qw = (torch.rand(D, generator=g) + 0.5).to(dtype).to(DEV)
    kw = (torch.rand(D, generator=g) + 0.5).to(dtype).to(DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(DEV)
    shape = (65, KV, page, D)
    k1, v1 = torch.zeros(shape, dtype=dtype, device=DEV), torch.zeros(shape, dtype=dtype, device=DEV)
    k2, v2 = k1.clone(), v1.clone()
    q1 = ops.qk_norm_rope_cache(qkv.clone(), H, KV, D, qw, kw, 1e-6, inv_freq, meta, k1, v1)
    q2 = TorchRefOps().qk_norm_rope_cache(qkv.clone(), H, KV, D, qw, kw, 1e-6, inv_freq, meta, k2, v2)
    close(q1, q2, dtype)
    close(k1, k2, dtype)
    assert torch.equal(v1, v2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, dtype):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(13, 2 * 223, generator=g) * 4).to(dtype).to(DEV)
    close(ops.swiglu(gu), TorchRefOps().swiglu(gu), dtype)


@pytest.mark.parametrize("M,N,K", [(1, 517, 96), (37, 130, 250), (64, 64, 16), (129, 65, 33)])
def test_gemm_f32(ops, M, N, K):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(M, K + 5, generator=g).to(DEV)[:, :K]          # strided rows
    w = torch.randn(N, K, generator=g).to(DEV)
    want = x.double() @ w.double().T
    got = ops.linear(x, w)
    assert ((got.double() - want).abs().max() / want.abs().max()).item() < 2e-6
    # a row's result does not depend on the other rows of the batch
    assert torch.equal(ops.linear(x[:1], w), got[:1])


@pytest.mark.parametrize("M,N,K", [(5, 301, 80), (64, 2560, 4096)])
def test_linear_bf16(ops, M, N, K):
    g = torch.Generator().manual_seed(4)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ref = TorchRefOps()
    close(ops.linear(x, w), ref.linear(x, w), torch.bfloat16)
    out = ops.linear(x, w, out_dtype=torch.float32)
    assert out.dtype == torch.float32
    want = ref.linear(x, w, out_dtype=torch.float32)
    assert ((out - want).abs().max() / want.abs().max()).item() < 1e-4


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", [(2560, 4096), (6144, 2560), (100, 64), (517, 96), (19456, 2560), (2560, 9728)])
def test_gemm_skinny(ops, request, M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :K]      # strided rows
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ops.skinny_max_rows, ops.skinny_max_cols, ops.stream_gemm = 64, 1 << 30, False     # this test is about the skinny kernel
    request.addfinalizer(lambda: (setattr(ops, "skinny_max_rows", 16), setattr(ops, "skinny_max_cols", 4096),
                                  setattr(ops, "stream_gemm", True)))
    before = ops.launches
    got = ops.linear(x, w, out_dtype=torch.float32)
    assert ops.launches == before + 1                     # the package's own kernel ran
    want = x.double() @ w.double().T
    assert ((got.double() - want).abs().max() / want.abs().max()).item() < 1e-5
    got16 = ops.linear(x, w)
    assert got16.dtype == torch.bfloat16
    close(got16, want, torch.bfloat16)
    # a token's result does not depend on the rest of the batch (same bits alone and in company)
    assert torch.equal(ops.linear(x[:1], w, out_dtype=torch.float32), got[:1])
    if M > 8:
        assert torch.equal(ops.linear(x[5:9], w, out_dtype=torch.float32), got[5:9])


@pytest.mark.parametrize("M", [1, 5, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(2560, 4096), (6144, 2560), (100, 64), (517, 192), (19456, 2560), (2560, 9728), (128, 64)])
def test_gemm_stream(ops, M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :K]      # strided rows
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    got = ops._gemm_stream(x, w, torch.float32)
    assert got is not None
    ops.check_errors()
    want = x.double() @ w.double().T
    assert ((got.double() - want).abs().max() / want.abs().max()).item() < 1e-5
    got16 = ops._gemm_stream(x, w, torch.bfloat16)
    close(got16, want, torch.bfloat16)
    # same bits on a second call (the split's summation order is fixed) and alone vs in company
    assert torch.equal(ops._gemm_stream(x, w, torch.float32), got)
    assert torch.equal(ops._gemm_stream(x[:1], w, torch.float32), got[:1])
    if M > 8:
        assert torch.equal(ops._gemm_stream(x[5:9], w, torch.float32), got[5:9])
    ops.check_errors()


@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (512, 512, 128), (700, 517 + 3, 192), (2048, 2560, 4096), (2048, 6144, 2560),
                                   (513, 304, 640), (1027, 2560, 9728), (128, 128, 128), (129, 296, 640), (1, 256, 64), (300, 6144, 2560),
                                   (256, 2560, 4096), (4096, 2560, 1024), (1500, 1288, 448)])
def test_gemm_tc2(ops, M, N, K):
    """The two-block (cta_group::2) tcgen05 product: 256-row tiles shared by a cluster of two blocks."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K + 8, generator=g).to(torch.bfloat16).to(DEV)[:, :K]
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    before = ops.launches
    got = ops._gemm_tc(x, w, torch.bfloat16)
    assert got is not None and ops.launches == before + 1
    again = ops._gemm_tc(x, w, torch.bfloat16)
    ops.check_errors()
    want = x.double() @ w.double().T
    close(got, want, torch.bfloat16)
    assert torch.equal(got, again)
    assert int(ops._tc2_counters.abs().sum()) == 0               # tiles cut along K leave their arrival counters at zero
    assert ops._gemm_tc(x, w, torch.float32) is None             # bfloat16 results only: the caller takes another kernel


def test_gemm_tc2_random_shapes(ops):
    """Shapes drawn at random: rows from 128 to 5,000, widths that are multiples of 8, depths that are multiples of 64, among them
    many whose left-over tiles are cut along K (few tiles, long K) and many with ragged last tiles in both directions."""
    rng = np.random.default_rng(11)
    for case in range(24):
        M = int(rng.integers(128, 5000)) if case % 3 else int(rng.integers(128, 700))
        N = 8 * int(rng.integers(16, 900)) if case % 2 else 8 * int(rng.integers(16, 120))
        K = 64 * int(rng.integers(1, 160)) if case % 4 else 64 * int(rng.integers(40, 200))
        if M * N > 6e6:
            N = max(128, 8 * int(6e6 / M / 8))
        g = torch.Generator().manual_seed(case)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        w = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16).to(DEV)
        got = ops._gemm_tc(x, w, torch.bfloat16)
        assert got is not None, (M, N, K)
        ops.check_errors()
        want = x.float() @ w.float().T
        err = ((got.float() - want).abs().max() / want.abs().max()).item()
        assert err < 1e-2, (M, N, K, err)
        assert int(ops._tc2_counters.abs().sum()) == 0, (M, N, K)
        if N % 16 == 0:
            saved = ops.tc_gemm
            ops.tc_gemm = True
            try:
                act = ops.gated_linear(x, w)
            finally:
                ops.tc_gemm = saved
            ops.check_errors()
            ref = TorchRefOps()
            want_act = ref.swiglu(ref.linear(x, w)).float()
            err = ((act.float() - want_act).abs().max() / want_act.abs().max().clamp_min(1e-6)).item()
            assert err < 2e-2, (M, N, K, err)


@pytest.mark.parametrize("M,inter,K", [(512, 128, 64), (700, 264, 192), (2048, 9728, 2560), (600, 1000, 640), (513, 40, 128), (129, 64, 128),
                                       (256, 1024, 2560), (1024, 648, 512)])
def test_gemm_tc2_swiglu(ops, M, inter, K):
    """The same with the gate rows loaded by the even block and the up rows by the odd one, silu(gate) * up in the epilogue."""
    g = torch.Generator().manual_seed(M + inter)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * inter, K, generator=g) * K ** -0.5).to(torch.bfloat16).to(DEV)
    saved = ops.tc_gemm
    ops.tc_gemm = True
    try:
        before = ops.launches
        got = ops.gated_linear(x, w)
        assert ops.launches == before + 1
    finally:
        ops.tc_gemm = saved
    ops.check_errors()
    ref = TorchRefOps()
    close(got, ref.swiglu(ref.linear(x, w)), torch.bfloat16)


def make_meta(page_size, segs, num_pages, seed, tile=64, indirect=False, window=None):
    """segs: list of (pos0, n).  Builds block tables with shuffled pages; returns an object with the arrays the
    engine's group view gives a mixer.  indirect: the table has more rows than entries, in another order, and
    table_rows says which row an entry reads (the engine's device-resident tables); otherwise entry i reads row i.
    window: pages that lie wholly before the window of an entry's FIRST fed position hold the null page, as after
    the cache manager has given them back."""
    rng = np.random.default_rng(seed)
    free = list(rng.permutation(np.arange(1, num_pages + 1)))
    S = len(segs)
    kv_len = [p + n for p, n in segs]
    max_pages = max(-(-L // page_size) for L in kv_len)
    rows = list(range(S))
    R = S
    if indirect:
        R = S + 3
        rows = [int(r) for r in rng.permutation(np.arange(1, R))[:S]]
    table = np.zeros((R, max_pages), dtype=np.int32)
    for s, L in enumerate(kv_len):
        first_live = 0 if window is None else max(0, segs[s][0] - window + 1) // page_size
        for i in range(-(-L // page_size)):
            page = free.pop()
            table[rows[s], i] = page if i >= first_live else 0
    q_start = np.zeros(S + 1, dtype=np.int32)
    q_start[1:] = np.cumsum([n for _, n in segs])
    positions = np.concatenate([np.arange(p, p + n) for p, n in segs]).astype(np.int32)
    slots = np.concatenate([table[rows[s], np.arange(p, p + n) // page_size] * page_size + np.arange(p, p + n) % page_size
                            for s, (p, n) in enumerate(segs)]).astype(np.int32)
    decode = [s for s, (_, n) in enumerate(segs) if n == 1]
    tiles = [(s, r) for s, (_, n) in enumerate(segs) if n > 1 for r in range(0, n, tile)]
    tiles2 = [(s, r) for s, (_, n) in enumerate(segs) if n > 1 for r in range(0, n, 2 * tile)]
    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device=DEV)
    return types.SimpleNamespace(
        page_size=page_size, tile=tile, positions=t(positions), slots=t(slots), block_table=t(table),
        table_rows=t(rows) if indirect else None, rows=rows,
        max_pages=max_pages, seg_q_start=t(q_start), seg_pos0=t([p for p, _ in segs]), seg_kv_len=t(kv_len),
        decode_segs=t(decode), prefill_tiles=t(tiles).view(-1, 2), prefill_tiles2=t(tiles2).view(-1, 2),
        max_kv_len=max(kv_len), num_tokens=int(q_start[-1]))


ATTN_SHAPES = [  # H, KV, D, page
    (4, 2, 16, 8), (6, 3, 32, 4), (5, 1, 48, 16), (8, 8, 64, 16), (32, 8, 128, 16), (3, 3, 80, 32), (2, 1, 256, 16),
    (5, 1, 64, 16), (12, 1, 128, 32), (16, 1, 64, 16), (6, 2, 128, 8), (20, 1, 128, 16)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,D,page", ATTN_SHAPES)
def test_qk_norm_rope_cache(ops, dtype, H, KV, D, page):
    g = torch.Generator().manual_seed(5)
    segs = [(0, 9), (37, 1), (5, 70)]
    meta = make_meta(page, segs, 64, seed=1)
    T = meta.num_tokens
    qkv = torch.randn(T, (H + 2 * KV) * D, generator=g).to(dtype).to(DEV)
    qw = (torch.rand(D, generator=g) + 0.5).to(dtype).to(DEV)
    kw = (torch.rand(D, generator=g) + 0.5).to(dtype).to(DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(DEV)
    shape = (65, KV, page, D)
    for use_norm, use_rope in ((True, True), (False, True), (True, False)):
        k1, v1 = torch.zeros(shape, dtype=dtype, device=DEV), torch.zeros(shape, dtype=dtype, device=DEV)
        k2, v2 = k1.clone(), v1.clone()
        a = (qw, kw) if use_norm else (None, None)
        f = inv_freq if use_rope else None
        q1 = ops.qk_norm_rope_cache(qkv.clone(), H, KV, D, *a, 1e-6, f, meta, k1, v1)
        q2 = TorchRefOps().qk_norm_rope_cache(qkv.clone(), H, KV, D, *a, 1e-6, f, meta, k2, v2)
        close(q1, q2, dtype)
        close(k1, k2, dtype)
        assert torch.equal(v1, v2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,D,page", ATTN_SHAPES)
@pytest.mark.parametrize("window", [None, 13])
def test_paged_attention(ops, dtype, H, KV, D, page, window):
    g = torch.Generator().manual_seed(6)
    segs = [(0, 70), (150, 1), (31, 1), (40, 29), (0, 1), (299, 1), (3, 2)]
    # rows of a larger table in another order, and (with a window) null entries where pages were given back
    meta = make_meta(page, segs, 200, seed=2, indirect=True, window=window)
    T = meta.num_tokens
    q = torch.randn(T, H * D, generator=g).to(dtype).to(DEV)
    kc = torch.randn(201, KV, page, D, generator=g).to(dtype).to(DEV)
    vc = torch.randn(201, KV, page, D, generator=g).to(dtype).to(DEV)
    # make one far key of the long decode stand out, so that a lost or misplaced key shows
    far = 2 * page + 3 if window is None else 299 - 7             # (inside the window when there is one)
    kc[meta.block_table[meta.rows[5], far // page].long(), :, far % page, :] *= 4.0
    kc[0], vc[0] = 1e4, 1e4                                       # the null page: reading it as a key would show
    want = TorchRefOps().paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, window)
    # splits merged by a cluster through shared memory / by the last block to finish / by a merge kernel (also when the
    # cluster switch is on) / generic kernels
    for fast, fused, cluster in ((True, True, True), (True, True, False), (True, False, False), (True, False, True),
                                 (False, False, False)):
        for splits in (None, 1, 3):
            ops.force_splits, ops.fast_attention, ops.fused_merge, ops.cluster_merge = splits, fast, fused, cluster
            ops.tc_attention = splits != 3               # prompt portions: tcgen05 kernel, and the mma.sync kernel
            ops.bulk_decode = splits != 1                # decoded tokens: bulk-copy ring, and register streaming
            try:
                got = ops.paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, window)
                got2 = ops.paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, window)    # counters were left clean
            finally:
                ops.force_splits, ops.fast_attention, ops.fused_merge, ops.tc_attention = None, True, True, True
                ops.bulk_decode = ops.cluster_merge = True
            close(got, want, dtype)
            assert torch.equal(got, got2)
            ops.check_errors()


@pytest.mark.parametrize("H,KV,D,page", [(8, 2, 128, 16), (4, 4, 64, 8), (6, 1, 128, 32), (2, 2, 64, 64)])
@pytest.mark.parametrize("window", [None, 200])
def test_prefill_attention_long(ops, H, KV, D, page, window):
    """Portions of hundreds of rows with offsets: whole tiles, diagonal tiles, a far key that stands out."""
    g = torch.Generator().manual_seed(9)
    segs = [(0, 300), (517, 260), (64, 129), (1000, 2)]
    meta = make_meta(page, segs, 400, seed=3, indirect=True, window=window)
    q = torch.randn(meta.num_tokens, H * D, generator=g).to(torch.bfloat16).to(DEV)
    kc = torch.randn(401, KV, page, D, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(401, KV, page, D, generator=g).to(torch.bfloat16).to(DEV)
    far = 3 * page + 5 if window is None else 517 - 150
    kc[meta.block_table[meta.rows[1], far // page].long(), :, far % page, :] *= 3.0
    want = TorchRefOps().paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, window)
    for tc in (True, False):
        ops.tc_attention = tc
        try:
            got = ops.paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, window)
        finally:
            ops.tc_attention = True
        ops.check_errors()
        close(got, want, torch.bfloat16)


def test_sampling(ops):
    g = torch.Generator().manual_seed(7)
    V = 1543
    logits = (torch.randn(6, V, generator=g) * 3).to(DEV)
    logits[2, 100] = logits[2, 900] = logits[2].max() + 1          # a tie: the lowest index wins
    assert torch.equal(ops.argmax(logits).cpu(), logits.argmax(-1).to(torch.int32).cpu())
    assert int(ops.argmax(logits)[2]) == 100
    temps = torch.tensor([0.0, 0.8, 1.5, 0.3, 0.0, 1.0], device=DEV)
    seeds = torch.tensor([1, 2, 3, -5, 5, 6], dtype=torch.int32, device=DEV)
    counters = torch.tensor([0, 1, 2, 3, 4, 70000], dtype=torch.int32, device=DEV)
    got = ops.sample(logits, temps, seeds, counters).cpu().long()
    scores = perturbed_scores(logits.cpu(), temps.cpu(), seeds.cpu(), counters.cpu())
    top = scores.max(-1).values
    # the chosen token's perturbed score is the row's maximum (up to the rounding of log)
    assert ((top - scores[torch.arange(6), got]).abs() < 1e-4 * top.abs().clamp_min(1)).all()
    assert got[0] == logits[0].argmax().item() and got[4] == logits[4].argmax().item()


def test_sampling_large_vocabulary(ops):
    """The several-blocks-per-row path: same tokens as the reference, ties to the lowest index, twice in a row."""
    g = torch.Generator().manual_seed(8)
    V = 151936
    logits = (torch.randn(5, V, generator=g) * 2).to(DEV)
    logits[1, 70000] = logits[1, 150000] = logits[1, 9] = logits[1].max() + 1
    temps = torch.tensor([0.0, 0.0, 0.9, 1.3, 0.0], device=DEV)
    seeds = torch.tensor([3, 4, 5, 6, 7], dtype=torch.int32, device=DEV)
    counters = torch.tensor([0, 9, 2, 30, 4], dtype=torch.int32, device=DEV)
    for _ in range(2):
        got = ops.sample(logits, temps, seeds, counters).cpu().long()
        assert got[1] == 9 and got[0] == logits[0].argmax().item() and got[4] == logits[4].argmax().item()
        scores = perturbed_scores(logits.cpu(), temps.cpu(), seeds.cpu(), counters.cpu())
        top = scores.max(-1).values
        assert ((top - scores[torch.arange(5), got]).abs() < 1e-4 * top.abs().clamp_min(1)).all()
        assert torch.equal(ops.argmax(logits).cpu().long(), logits.argmax(-1).cpu())


def test_sampling_distribution(ops):
    """Draws at temperature T follow softmax(logits / T): compare frequencies over many counters."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -3.0]], device=DEV).repeat(4096, 1)
    temps = torch.full((4096,), 0.7, device=DEV)
    seeds = torch.full((4096,), 1234, dtype=torch.int32, device=DEV)
    counters = torch.arange(4096, dtype=torch.int32, device=DEV)
    got = ops.sample(logits, temps, seeds, counters).cpu().long()
    freq = torch.bincount(got, minlength=7).float() / 4096
    probs = torch.softmax(logits[0].cpu() / 0.7, -1)
    assert (freq - probs).abs().max() < 0.03


@pytest.mark.parametrize("M", [1, 5, 8, 13, 32])
@pytest.mark.parametrize("N,K", [(2560, 4096), (2560, 9728), (100, 64), (516, 192), (19456, 2560)])
def test_deferred_sums(ops, M, N, K):
    """A few-row product left as partial sums: adding them up gives the bits the GEMM's own fix-up stores, and the
    residual-add + norm that reads them directly matches the separate kernels."""
    from mini_inference_b200.ops import DeferredSum
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * K ** -0.5).to(torch.bfloat16).to(DEV)
    res = (torch.randn(M, N, generator=g) * 2).to(torch.bfloat16).to(DEV)
    nw = (torch.rand(N, generator=g) + 0.5).to(torch.bfloat16).to(DEV)
    saved = ops._linear_choice
    ops._linear_choice = {(ops._row_bucket(M), N, K): "stream"}
    try:
        plain_out = ops.linear(x, w)
        lazy = ops.linear(x, w, defer=True)
        assert isinstance(lazy, DeferredSum) and lazy.shape == (M, N)
        assert torch.equal(ops.materialize(lazy), plain_out)
        x1, x2 = res.clone(), res.clone()
        y1 = ops.add_rmsnorm(x1, lazy, nw, 1e-5)
        y2 = ops.add_rmsnorm(x2, plain_out, nw, 1e-5)
        ops.check_errors()
        assert torch.equal(x1, x2)
        close(y1, y2, torch.bfloat16)
        # a reader that normalises selected rows only gets the product itself
        rows = torch.tensor([M - 1, 0], dtype=torch.int32, device=DEV)
        x3 = res.clone()
        close(ops.add_rmsnorm(x3, lazy, nw, 1e-5, rows), ops.add_rmsnorm(res.clone(), plain_out, nw, 1e-5, rows), torch.bfloat16)
        assert torch.equal(x3, res)
        # the hint about the weight that is read next changes nothing but the kernel's grid: whole tensors, a few
        # bytes, a size that is no multiple of the request size, a view that starts off a 16-byte boundary
        odd = torch.randn(5000, generator=g).to(torch.bfloat16).to(DEV)
        for hint in (w, odd, odd[:4], odd[1:]):
            x4, x5 = res.clone(), res.clone()
            close(ops.add_rmsnorm(x4, lazy, nw, 1e-5, next_weight=hint), y1, torch.bfloat16)
            assert torch.equal(x4, x1)
            close(ops.add_rmsnorm(x5, plain_out, nw, 1e-5, next_weight=hint), y2, torch.bfloat16)
            assert torch.equal(x5, x2)
        ops.check_errors()
    finally:
        ops._linear_choice = saved


@pytest.mark.parametrize("H,KV,D,page", [(32, 8, 128, 16), (8, 2, 64, 64), (16, 1, 128, 256)])
@pytest.mark.parametrize("window", [None, 1000])
def test_decode_attention_long_context(ops, H, KV, D, page, window):
    """Decoded tokens at contexts of thousands of keys (many ring revolutions, many splits, the merge), requests of
    very different lengths in one launch, one far key that stands out."""
    g = torch.Generator().manual_seed(21)
    segs = [(4099, 1), (8999, 1), (17, 1), (1023, 1), (1024, 1), (0, 1)]
    pages = sum((p + 1 + page - 1) // page for p, _ in segs) + 2
    meta = make_meta(page, segs, pages, seed=6, indirect=True, window=window)
    T = meta.num_tokens
    q = torch.randn(T, H * D, generator=g).to(torch.bfloat16).to(DEV)
    kc = torch.randn(pages + 1, KV, page, D, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(pages + 1, KV, page, D, generator=g).to(torch.bfloat16).to(DEV)
    far = 5000 if window is None else 8999 - 700
    kc[meta.block_table[meta.rows[1], far // page].long(), :, far % page, :] *= 4.0
    want = TorchRefOps().paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, window)
    for bulk, cluster in ((True, True), (True, False), (False, False)):
        for splits in (None, 5, 8, 11):
            ops.bulk_decode, ops.cluster_merge, ops.force_splits = bulk, cluster, splits
            try:
                got = ops.paged_attention(q, kc, vc, meta, H, KV, D, D ** -0.5, window)
            finally:
                ops.bulk_decode, ops.cluster_merge, ops.force_splits = True, True, None
            ops.check_errors()
            close(got, want, torch.bfloat16)
