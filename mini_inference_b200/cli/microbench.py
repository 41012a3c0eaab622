"""Microbenchmarks of the decode step's bandwidth-bound kernels, in the manner of the
reference's bench/micro/bench_gemm.py (:35-170: every linear of a model at a few row counts,
ms, GB/s and share of peak, rotating weight copies to defeat the L2) and
bench/micro/bench_attention.py (:61-167: paged decode attention over batch x context).

    python -m mini_inference_b200.cli.microbench gemm      [--rows 1,8,64] [--size 4b]
    python -m mini_inference_b200.cli.microbench attention [--batch 1,8,64] [--ctx 4096]
    python -m mini_inference_b200.cli.microbench prefill   [--tokens 2048] [--ctx-before 0]

Each line: kernel, shape, microseconds (CUDA events, after warm-up), GB/s of the bytes the
kernel has to read, and that as a share of the measured copy bandwidth."""
from __future__ import annotations

import argparse
import json
import os
import sys
import types

import torch

from .run_engine import SIZES


def peak_gbs():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f)["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def timed(fn, iters, warmup=3):
    """Microseconds per call.  The calls are recorded into one CUDA graph (fn(i) for i in
    range(iters), each on different operands) and the graph is replayed, so the figure is the
    kernels' time on the device, not the host's launch cost."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(warmup):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i)
    graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / iters


def bench_gemm(args, ops, peak):
    cfg = SIZES[args.size]
    h, H, KV, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["intermediate_size"], cfg["vocab_size"])
    shapes = [("qkv", (H + 2 * KV) * D, h), ("o", h, H * D), ("gate_up", 2 * I, h), ("down", h, I), ("lm_head", V, h)]
    for name, N, K in shapes:
        if args.only and name not in args.only:
            continue
        copies = max(2, -(-args.rotate_mb * 2 ** 20 // (N * K * 2)))      # rotate >= rotate_mb of weights
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        for M in args.rows:
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            od = torch.float32 if name == "lm_head" else None
            ops.skinny_max_rows, ops.skinny_max_cols = 64, 1 << 30
            for label, stream, skinny, tc in (("stream", True, False, False), ("skinny", False, True, False),
                                              ("tcgen05 x2", False, False, True), ("library", False, False, False)):
                ops.stream_gemm, ops.skinny_gemm, ops.tc_gemm = stream, skinny, tc
                if (stream and M > 32) or (skinny and M > 64) or (tc and (M < 128 or od is not None)):
                    continue
                us = timed(lambda i: ops.linear(x, ws[i % copies], out_dtype=od), args.iters)
                gbs = N * K * 2 / us / 1e3
                tf = 2.0 * M * N * K / us / 1e6
                print(f"gemm {name:8s} M={M:<4d} N={N:<6d} K={K:<5d} {label:10s} {us:9.2f} us {gbs:8.1f} GB/s "
                      f"{100 * gbs / peak:5.1f} % of peak bandwidth {tf:8.1f} TFLOP/s", flush=True)
            ops.stream_gemm = ops.skinny_gemm = True
            ops.tc_gemm = False
        del ws


def bench_attention(args, ops, peak):
    cfg = SIZES[args.size]
    H, KV, D, ps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], args.page_size
    for B in args.batch:
        pages_per_seq = -(-args.ctx // ps)
        layers = max(2, -(-args.rotate_mb * 2 ** 20 // (B * pages_per_seq * ps * KV * D * 4)))
        num_pages = B * pages_per_seq
        kv = torch.randn(layers, 2, num_pages + 1, KV, ps, D, device="cuda", dtype=torch.bfloat16)
        perm = torch.randperm(num_pages, device="cuda").to(torch.int32) + 1
        table = perm.view(B, pages_per_seq).contiguous()
        ar = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        meta = types.SimpleNamespace(
            page_size=ps, tile=64, block_table=table, max_pages=pages_per_seq, seg_q_start=ar,
            seg_pos0=torch.full((B,), args.ctx - 1, dtype=torch.int32, device="cuda"),
            seg_kv_len=torch.full((B,), args.ctx, dtype=torch.int32, device="cuda"), decode_segs=ar[:B],
            table_rows=None, prefill_tiles=torch.zeros((0, 2), dtype=torch.int32, device="cuda"), prefill_tiles2=None,
            max_kv_len=args.ctx, num_tokens=B)
        q = torch.randn(B, H * D, device="cuda", dtype=torch.bfloat16)
        for label, flag in (("tensor-core", True), ("generic", False)):
            for splits in (args.splits or [None]):
                if splits and not flag:
                    continue
                ops.fast_attention, ops.force_splits = flag, splits
                us = timed(lambda i: ops.paged_attention(q, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, D,
                                                         D ** -0.5, None), args.iters)
                gbs = B * args.ctx * KV * D * 4 / us / 1e3
                print(f"decode attention B={B:<3d} ctx={args.ctx} heads {H}/{KV} D={D} {label:12s} "
                      f"{'splits ' + str(splits) if splits else 'splits chosen'} {us:9.2f} us {gbs:8.1f} GB/s {100 * gbs / peak:5.1f} % of peak",
                      flush=True)
        ops.fast_attention, ops.force_splits = True, None
        del kv


def bench_prefill_attention(args, ops, peak):
    """Prompt attention over the pages: one request of --tokens tokens whose first token is at position --ctx-before
    (a later portion of a long prompt when that is not 0), causal; TFLOP/s of the scores and weighted sums that count."""
    import numpy as np
    cfg = SIZES[args.size]
    H, KV, D, ps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], args.page_size
    T, p0 = args.tokens, args.ctx_before
    pages_per_seq = -(-(p0 + T) // ps)
    layers = max(2, -(-args.rotate_mb * 2 ** 20 // (pages_per_seq * ps * KV * D * 4)))
    kv = torch.randn(layers, 2, pages_per_seq + 1, KV, ps, D, device="cuda", dtype=torch.bfloat16)
    table = (torch.randperm(pages_per_seq, device="cuda").to(torch.int32) + 1).view(1, pages_per_seq).contiguous()
    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device="cuda")
    meta = types.SimpleNamespace(
        page_size=ps, tile=64, block_table=table, table_rows=None, max_pages=pages_per_seq, seg_q_start=t([0, T]), seg_pos0=t([p0]),
        seg_kv_len=t([p0 + T]), decode_segs=t([]), prefill_tiles=t([(0, r) for r in range(0, T, 64)]).view(-1, 2),
        prefill_tiles2=t([(0, r) for r in range(0, T, 128)]).view(-1, 2), max_kv_len=p0 + T, num_tokens=T)
    q = torch.randn(T, H * D, device="cuda", dtype=torch.bfloat16)
    flops = 4.0 * H * D * (T * p0 + T * (T + 1) / 2)
    for label, tc, fast in (("tcgen05", True, True), ("mma.sync", False, True)):
        ops.tc_attention, ops.fast_attention = tc, fast
        us = timed(lambda i: ops.paged_attention(q, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, D, D ** -0.5, None), args.iters)
        print(f"prompt attention T={T} from position {p0} heads {H}/{KV} D={D} page {ps} {label:9s} {us:9.2f} us "
              f"{flops / us / 1e6:8.1f} TFLOP/s", flush=True)
        if tc and hasattr(ops.lib, "mi_attn_tc_timing"):
            # a library built with MI_NVCC_EXTRA=-DMI_ATT_TIMING counts clocks of one softmax thread per block and key tile
            import ctypes
            ticks = (ctypes.c_ulonglong * 16)()
            ops.lib.mi_attn_tc_timing(ticks, 1)
            ops.paged_attention(q, kv[0, 0], kv[0, 1], meta, H, KV, D, D ** -0.5, None)
            torch.cuda.synchronize()
            ops.lib.mi_attn_tc_timing(ticks, 1)
            n = max(1, ticks[3])
            print(f"  softmax thread, clocks per 64-key tile over {n} tiles: wait for scores {ticks[0] / n:.0f}, "
                  f"maximum + exponentials + P store {ticks[1] / n:.0f}, wait for the previous PV + hand-over {ticks[2] / n:.0f}", flush=True)
            print(f"  MMA thread, clocks per tile: wait for the next keys + issue of their scores {ticks[4] / n:.0f}, wait for P {ticks[5] / n:.0f}, "
                  f"wait for the values {ticks[6] / n:.0f}", flush=True)
            print(f"  of the middle part: score load {ticks[8] / n:.0f}, mask + maximum {ticks[9] / n:.0f}, exponentials + sums + packing {ticks[10] / n:.0f}, "
                  f"P store {ticks[11] / n:.0f}", flush=True)
    ops.tc_attention = ops.fast_attention = True
    ops.check_errors()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["gemm", "attention", "prefill"])
    ap.add_argument("--size", default="4b", choices=sorted(SIZES))
    ap.add_argument("--rows", default="1,8,64", type=lambda s: [int(v) for v in s.split(",")])
    ap.add_argument("--batch", default="1,8,64", type=lambda s: [int(v) for v in s.split(",")])
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048, help="prefill: tokens of the portion")
    ap.add_argument("--ctx-before", type=int, default=0, help="prefill: tokens of the request already in the cache")
    ap.add_argument("--only", default=None, type=lambda s: s.split(","), help="gemm: only these (qkv,o,gate_up,down,lm_head)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--splits", default=None, type=lambda s: [int(v) for v in s.split(",")],
                    help="attention: time these numbers of key splits instead of the chosen one")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--rotate-mb", type=int, default=512, help="rotate through at least this many MB of operands")
    args = ap.parse_args(argv)
    from ..ops import get_ops
    ops = get_ops("cuda:0")
    peak, src = peak_gbs()
    print(f"# peak {peak} GB/s ({src})")
    {"gemm": bench_gemm, "attention": bench_attention, "prefill": bench_prefill_attention}[args.what](args, ops, peak)
    return 0


if __name__ == "__main__":
    sys.exit(main())
