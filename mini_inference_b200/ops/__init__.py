"""Kernel namespace of the engine: thin Python entry points over the hand-written sm_100a
kernels in csrc/ (built into _kernels.so, called through its C interface).

There is no CPU path and no silent fall-back: get_ops() raises when there is no CUDA device
or the library cannot be built or loaded.  Matrix products of the bfloat16 path go to the
library GEMM, as the reference's do (engine/core/fused_linear.py:29-34); the float32 path
uses this package's own float32 GEMM kernel, which never uses a reduced-precision mode.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

_LIB = None
_c = ctypes


def load_library():
    global _LIB
    if _LIB is None:
        from .build import build
        path = build()
        _LIB = ctypes.CDLL(path)
    return _LIB


_CODES = {torch.float32: 0, torch.bfloat16: 1}


def _code(dtype):
    try:
        return _CODES[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} is not supported by the kernels (float32, bfloat16)") from None


def _raw_stream(device_index):
    getter = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if getter is not None:
        return getter(device_index)
    return torch.cuda.current_stream(device_index).cuda_stream


def _p(t):
    return _c.c_void_p(0 if t is None else t.data_ptr())


def _check(err, what):
    if err != 0:
        if err == -1:
            raise TypeError(f"{what}: unsupported combination of dtypes")
        if err == -2:
            raise ValueError(f"{what}: size not supported by this kernel")
        raise RuntimeError(f"{what}: CUDA error {err} at launch")


class DeferredSum:
    """A product [M, N] that the few-row GEMM left as partial sums (csrc/gemm_stream.cu, deferred mode).  Only
    add_rmsnorm (as its `delta`) and CudaOps.materialize understand it; a part that gets one must pass it on untouched."""
    __slots__ = ("ws", "M", "N", "K", "grid", "max_contrib", "tok", "device")

    def __init__(self, ws, M, N, K, grid, max_contrib, tok):
        self.ws, self.M, self.N, self.K, self.grid, self.max_contrib, self.tok = ws, M, N, K, grid, max_contrib, tok
        self.device = ws.device

    @property
    def shape(self):
        return (self.M, self.N)


class CudaOps:
    prefill_tile = 64
    deferred = True                          # linear(..., defer=True) may answer with a DeferredSum
    takes_hints = True                       # add_rmsnorm(..., next_weight=) is understood
    MAX_ROWS = 4096                          # decode rows x kv heads that the attention merge counters cover

    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError("mini_inference_b200 runs on a CUDA device only (no CPU path); "
                               f"device '{device}' is not one")
        self.lib = load_library()
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.NUM_SMS = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        self.force_splits = None             # tests set this to exercise the split merge on short contexts
        # many-row bfloat16 products on this package's two-block tcgen05 kernel (csrc/gemm_tc2.cu) instead of the library GEMM:
        # MI_TC_GEMM=1 all of them, 0 none; otherwise ("auto") those that tune_many_rows found faster on this model's weights
        self.tc_mode = os.environ.get("MI_TC_GEMM", "auto")
        self.tc_gemm = self.tc_mode == "1"
        self._many_choice = {}               # {(row bucket, N, K): "tc2"} from tune_many_rows; anything else: library
        self.tc_min_rows = 128
        # scratch of the own GEMM for the tiles it cuts along K (the shares of a last, partly filled wave of tiles)
        self._tc2_ws = torch.empty(20 << 20, dtype=torch.uint8, device=self.device)
        self._tc2_counters = torch.zeros(512, dtype=torch.int32, device=self.device)
        self.tc_attention = os.environ.get("MI_TC_ATTENTION", "1") == "1"    # prompt attention on the tcgen05 kernel
        self.stream_gemm = True              # few-row products on the persistent TMA weight-streaming kernel
        self.stream_max_cols = int(os.environ.get("MI_STREAM_MAX_COLS", 1 << 30))
        self._sample_slots = torch.zeros(4096, dtype=torch.int64, device=self.device)
        self._sample_arrivals = torch.zeros(4096, dtype=torch.int32, device=self.device)
        # decode attention stages K/V through shared memory with swizzled TMA tiles and per-warp mbarrier rings (31 vs
        # 33 us at batch 8, 168 vs 202 us at batch 64, context 4096, against streaming them into registers);
        # MI_BULK_DECODE=0 selects the register-streaming variant
        self.bulk_decode = os.environ.get("MI_BULK_DECODE", "1") == "1"
        self.fused_merge = True              # the last split block to finish merges the splits (no merge launch)
        # 2..8 splits of a (request, kv head): one thread-block cluster, merged through distributed shared memory
        self.cluster_merge = os.environ.get("MI_CLUSTER_MERGE", "1") == "1"
        self._cluster_fit = {}
        self._linear_choice = None           # {(row bucket, N, K): "library" | "stream" | "skinny"} from tune_linear
        self._stream_plans = {}
        # Scratch that kernels address directly and that captured graphs keep the address of: allocated here, once, at
        # fixed sizes; a call that needs more raises instead of moving them.
        self._merge_counters = torch.zeros(self.MAX_ROWS * 8, dtype=torch.int32, device=self.device)
        self._stream_counters = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self._stream_error = torch.zeros(1, dtype=torch.int32, device=self.device)
        # a few-row product whose only reader is the next residual-add + norm is left as partial sums for that kernel
        # to add up (no fix-up tail in the GEMM); MI_DEFER_SUMS=0 turns it off
        self.defer_sums = os.environ.get("MI_DEFER_SUMS", "1") == "1"
        # few rows: the residual-add + norm kernel's idle blocks request the first bytes of the weight that the next
        # product streams into L2 (MI_L2_AHEAD_MB=0 turns it off)
        self.l2_ahead_bytes = int(float(os.environ.get("MI_L2_AHEAD_MB", "32")) * (1 << 20))
        self.l2_ahead_max_rows = 64
        self.skinny_gemm = True              # few-row products on this package's weight-streaming kernel ...
        self.skinny_max_rows, self.skinny_max_cols = 16, 4096    # ... where it is at least as fast as the library's
        self.fast_attention = True           # tests clear this to run the generic attention kernels in bfloat16
        self.launches = 0                    # kernels of this package launched so far

    def _stream(self):
        # the raw handle of torch's current stream on this device: one C call (torch.cuda.current_stream builds a
        # Stream object every time, which at ~10 launches per layer was a fifth of an eager decode step's host time)
        return _c.c_void_p(_raw_stream(self._device_index))

    # ---------------------------------------------------------------- elementwise / norms
    def scatter_i32(self, table, idx, val):
        """table[idx[i]] = val[i]: the block-table entries that changed since the last step (cache/manager.py)."""
        n = idx.shape[0]
        if n:
            _check(self.lib.mi_scatter_i32(_p(table), _p(idx), _p(val), n, _c.c_longlong(table.numel()), self._stream()),
                   "scatter_i32")
            self.launches += 1

    def embedding(self, ids, table):
        T, hidden = ids.shape[0], table.shape[1]
        out = torch.empty((T, hidden), dtype=table.dtype, device=table.device)
        _check(self.lib.mi_embedding(_p(ids), _p(table), _p(out), T, hidden, table.shape[0], _code(table.dtype),
                                     self._stream()), "embedding")
        self.launches += 1
        return out

    def add_rmsnorm(self, x, delta, weight, eps, rows=None, next_weight=None):
        """x += delta (if any), y = rmsnorm(x) * weight.  next_weight: the tensor that the caller's next kernel streams; at
        few rows the kernel's idle blocks ask for its first bytes to be brought into L2 (a hint, never needed)."""
        hidden = x.shape[-1]
        ahead, ahead_bytes = None, 0
        if next_weight is not None and self.l2_ahead_bytes and x.shape[0] <= self.l2_ahead_max_rows and next_weight.is_contiguous():
            ahead, ahead_bytes = next_weight, min(next_weight.numel() * next_weight.element_size(), self.l2_ahead_bytes)
        if isinstance(delta, DeferredSum):
            if rows is None and x.dtype == torch.bfloat16 and x.is_contiguous() and hidden % 4 == 0 and delta.shape == tuple(x.shape):
                y = torch.empty_like(x)
                rc = self.lib.mi_deferred_add_rmsnorm(_p(x), _p(delta.ws), _p(weight), _p(y), delta.M, delta.N, delta.K, delta.grid,
                                                      delta.max_contrib, delta.tok, _c.c_float(eps), _code(weight.dtype),
                                                      _p(ahead), _c.c_longlong(ahead_bytes), self._stream())
                if rc == 0:
                    self.launches += 1
                    return y
                if rc != -2:
                    _check(rc, "deferred_add_rmsnorm")
            delta = self.materialize(delta)
        assert x.is_contiguous() and (delta is None or delta.is_contiguous())
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, hidden), dtype=x.dtype, device=x.device)
        _check(self.lib.mi_add_rmsnorm_ahead(_p(x), _p(delta), _p(weight), _p(y), _p(rows), n, hidden, _c.c_float(eps),
                                             _code(x.dtype), _code(weight.dtype), _p(ahead), _c.c_longlong(ahead_bytes),
                                             self._stream()), "add_rmsnorm")
        self.launches += 1
        return y

    def gated_linear(self, x, w):
        """silu(g) * u with [g | u] = x @ w.T (w = [gate rows | up rows]).  Many rows with the own tcgen05 GEMM chosen for this shape:
        one kernel whose epilogue applies the activation (csrc/gemm_tc2.cu), so the [M, 2 I] product is never written;
        otherwise product, then swiglu (or, for a few rows, the activation kernel that adds the product's partial sums)."""
        M, K = x.shape
        inter = w.shape[0] // 2
        if (self._use_tc(M, w.shape[0], K) and K % 64 == 0 and inter % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            act = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
            rc = self.lib.mi_gemm_tc2_swiglu(_p(x), x.stride(0), _p(w), _p(act), M, inter, K, *self._tc2_scratch(), _p(self._stream_error), self._stream())
            if rc == 0:
                self.launches += 1
                return act
            if rc != -2:
                _check(rc, "gemm_tc2_swiglu")
        gu = self.linear(x, w, defer=True)
        if isinstance(gu, DeferredSum):          # the few-row product left its partial sums: the activation kernel adds them
            act = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
            rc = self.lib.mi_deferred_swiglu(_p(gu.ws), _p(act), M, inter, gu.K, gu.grid, gu.max_contrib, gu.tok, self._stream())
            if rc == 0:
                self.launches += 1
                return act
            if rc != -2:
                _check(rc, "deferred_swiglu")
            gu = self.materialize(gu)
        return self.swiglu(gu)

    def materialize(self, value):
        """The bfloat16 tensor behind a DeferredSum (anything else is returned as it is)."""
        if not isinstance(value, DeferredSum):
            return value
        out = torch.empty((value.M, value.N), dtype=torch.bfloat16, device=value.device)
        _check(self.lib.mi_deferred_reduce(_p(value.ws), _p(out), value.M, value.N, value.K, value.grid, value.max_contrib,
                                           value.tok, self._stream()), "deferred_reduce")
        self.launches += 1
        return out

    def swiglu(self, gate_up):
        rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
        assert gate_up.is_contiguous()
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
        _check(self.lib.mi_swiglu(_p(gate_up), _p(out), rows, inter, _code(gate_up.dtype), self._stream()), "swiglu")
        self.launches += 1
        return out

    # ---------------------------------------------------------------- matrix products
    def linear(self, x, w, out_dtype=None, defer=False):
        """x [M, K] (rows may be strided), w [N, K] -> [M, N].  defer=True: the caller will use the result only as the
        `delta` of add_rmsnorm (or pass it through materialize); the answer may then be a DeferredSum."""
        if x.dtype == torch.float32:
            M, K = x.shape
            N = w.shape[0]
            assert x.stride(1) == 1 and w.is_contiguous() and w.dtype == torch.float32
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            _check(self.lib.mi_gemm_f32_nt(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, self._stream()), "gemm_f32")
            self.launches += 1
            return out
        M, K = x.shape
        if (self._use_tc(M, w.shape[0], K) and K % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            out = self._gemm_tc(x, w, out_dtype or x.dtype)
            if out is not None:
                return out
        choice = self._linear_choice.get((self._row_bucket(M), w.shape[0], K)) if self._linear_choice else None
        if choice == "library":
            return self._library_linear(x, w, out_dtype)
        if (self.stream_gemm and choice in (None, "stream") and M <= 32 and w.shape[0] <= self.stream_max_cols and K % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            out = self._gemm_stream(x, w, out_dtype or x.dtype, defer=defer and self.defer_sums and choice == "stream"
                                    and out_dtype in (None, torch.bfloat16) and w.shape[0] % 4 == 0)
            if out is not None:
                return out
        if (self.skinny_gemm and (choice == "skinny" or (choice is None and M <= self.skinny_max_rows
                                                         and w.shape[0] <= self.skinny_max_cols)) and M <= 64 and K % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            N = w.shape[0]
            od = out_dtype or x.dtype
            out = torch.empty((M, N), dtype=od, device=x.device)
            err = self.lib.mi_gemm_skinny(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, _code(od), self._stream())
            if err == 0:
                self.launches += 1
                return out
            if err != -2:
                _check(err, "gemm_skinny")
        return self._library_linear(x, w, out_dtype)

    @staticmethod
    def _library_linear(x, w, out_dtype):
        if out_dtype is not None and out_dtype != x.dtype:
            try:
                return torch.mm(x, w.t(), out_dtype=out_dtype)
            except TypeError:
                return torch.mm(x, w.t()).to(out_dtype)
        return torch.mm(x, w.t())

    ROW_BUCKETS = (1, 2, 4, 8, 16, 32)
    MANY_BUCKETS = (256, 512, 1024, 2048, 4096)

    def _many_bucket(self, M):
        for b in self.MANY_BUCKETS:
            if M <= b:
                return b
        return self.MANY_BUCKETS[-1]

    def _use_tc(self, M, N, K):
        if M < self.tc_min_rows:
            return False
        return self.tc_gemm or self._many_choice.get((self._many_bucket(M), N, K)) == "tc2"

    def tune_many_rows(self, weights, probes=None, iters=6, min_bytes=64 << 20):
        """Per weight shape and bucket of many rows (prompt steps), time the own two-block tcgen05 GEMM against the library
        GEMM on the model's own weights and remember where the own kernel wins.  probes: {(N, K): probe(rows) -> run(weight)}
        for products that run together with what follows them (gate/up with its activation, q/k/v with norm, rotation and
        cache write: own kernel with that in its epilogue against library product + separate kernel).  Shapes of less than
        min_bytes in all are left to the library (tiny models).  Returns the timings in microseconds."""
        probes = probes or {}
        report = {}
        if self.tc_mode != "auto":
            return report
        groups = {}
        for w in weights:
            if w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous() and w.shape[1] % 64 == 0 and w.shape[0] % 8 == 0:
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        saved, table = self.tc_gemm, {}
        try:
            self._many_choice = {}
            for (N, K), ws in groups.items():
                if len(ws) * N * K * 2 < min_bytes:
                    continue
                for M in self.MANY_BUCKETS:
                    if M * N * 2 > 512 << 20:              # a vocabulary-wide product never has this many rows
                        continue
                    x = torch.randn(M, K, device=ws[0].device, dtype=torch.bfloat16)
                    times = {}
                    for name in ("library", "tc2"):
                        self.tc_gemm = name == "tc2"
                        if (N, K) in probes:
                            probe = probes[(N, K)](M)
                            run = lambda i: probe(ws[i % len(ws)])
                        else:
                            run = lambda i: self.linear(x, ws[i % len(ws)])
                        times[name] = min(self._time_in_graph(run, iters) for _ in range(2))
                    if times["tc2"] < 0.97 * times["library"]:
                        table[(M, N, K)] = "tc2"
                    report[f"{N}x{K} M<={M}"] = {k: round(v, 1) for k, v in times.items()} | {"best": table.get((M, N, K), "library")}
        finally:
            self.tc_gemm = saved
        self._many_choice = table
        self.check_errors()
        return report

    def _row_bucket(self, M):
        for b in self.ROW_BUCKETS:
            if M <= b:
                return b
        return 0

    def tune_linear(self, weights, out_dtypes=None, iters=16, min_bytes=256 << 20, deferrable=(), gated=()):
        """Per weight shape and row-count bucket, time this package's few-row kernels against the
        library GEMM on the model's own weights and remember the fastest.  The reference does the
        same kind of start-up timing to choose a weight layout per shape
        (engine/core/fused_linear.py:51-94); rotating over the layers' real weights keeps the L2
        from flattering anyone.  weights: bfloat16 [N, K] tensors; out_dtypes: {(N, K): dtype}."""
        groups = {}
        for w in weights:
            if w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous():
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        saved = (self.stream_gemm, self.skinny_gemm, self.skinny_max_rows, self.skinny_max_cols, self.stream_max_cols)
        table, report = {}, {}
        try:
            self._linear_choice = None
            for (N, K), ws in groups.items():
                od = (out_dtypes or {}).get((N, K))
                # one weight cannot defeat the L2 by rotation; leave such shapes to the default rule
                if len(ws) * N * K * 2 < min_bytes:
                    continue
                for M in self.ROW_BUCKETS:
                    x = torch.randn(M, K, device=ws[0].device, dtype=torch.bfloat16)
                    times = {}
                    for name in ("library", "stream", "skinny"):
                        if name == "stream" and K % 64:
                            continue
                        if name == "skinny" and K % 32:
                            continue
                        self.stream_gemm, self.skinny_gemm = name == "stream", name == "skinny"
                        self.skinny_max_rows, self.skinny_max_cols, self.stream_max_cols = 64, 1 << 30, 1 << 30
                        run = lambda i: self.linear(x, ws[i % len(ws)], out_dtype=od)
                        if (N, K) in gated:
                            # a gate/up product is read by the activation only: the pair is timed, as it runs in a step
                            self._linear_choice = {(M, N, K): name}
                            run = lambda i: self.gated_linear(x, ws[i % len(ws)])
                        elif name == "stream" and (N, K) in deferrable and self.defer_sums and od in (None, torch.bfloat16):
                            # these products are read by a norm kernel that adds the partial sums itself
                            run = lambda i: self._gemm_stream(x, ws[i % len(ws)], torch.bfloat16, defer=True)
                        times[name] = min(self._time_in_graph(run, iters) for _ in range(2))
                        self._linear_choice = None
                    best = min(times, key=times.get)
                    if times[best] > 0.95 * times["library"]:      # an own kernel has to win clearly
                        best = "library"
                    table[(M, N, K)] = best
                    report[f"{N}x{K} M<={M}"] = {k: round(v, 2) for k, v in times.items()} | {"best": best}
        finally:
            self.stream_gemm, self.skinny_gemm, self.skinny_max_rows, self.skinny_max_cols, self.stream_max_cols = saved
        self._linear_choice = table
        self.check_errors()
        return report

    def _time_in_graph(self, fn, iters):
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            fn(0)
            fn(1)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(i)
        graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(self.device)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize(self.device)
        return start.elapsed_time(stop) * 1e3 / iters

    def _gemm_stream(self, x, w, od, defer=False):
        """Persistent TMA weight-streaming product (csrc/gemm_stream.cu); None if the shape is not taken."""
        M, K = x.shape
        N = w.shape[0]
        plan = self._stream_plans.get((M, N, K))
        if plan is None:
            g, rt, mc = _c.c_int(), _c.c_int(), _c.c_int()
            rc = self.lib.mi_gemm_stream_plan(M, N, K, _c.byref(g), _c.byref(rt), _c.byref(mc))
            plan = self._stream_plans[(M, N, K)] = None if rc else (g.value, rt.value, mc.value)
        if not plan:
            return None
        grid, row_tiles, max_contrib = plan
        if row_tiles > self._stream_counters.numel():
            return None                      # more row tiles than the fixed counters cover: another kernel takes it
        tok = 8 if M <= 8 else 16 if M <= 16 else 32
        workspace = torch.empty(row_tiles * max_contrib * 128 * tok, dtype=torch.float32, device=x.device)
        if defer:
            rc = self.lib.mi_gemm_stream_deferred(_p(x), x.stride(0), _p(w), M, N, K, _p(workspace), _p(self._stream_error),
                                                  self._stream())
            if rc == 0:
                self.launches += 1
                return DeferredSum(workspace, M, N, K, grid, max_contrib, tok)
            if rc != -2:
                _check(rc, "gemm_stream_deferred")
        out = torch.empty((M, N), dtype=od, device=x.device)
        rc = self.lib.mi_gemm_stream(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, _code(od), _p(workspace),
                                     _p(self._stream_counters), _p(self._stream_error), self._stream())
        if rc == -2:
            return None
        _check(rc, "gemm_stream")
        self.launches += 1
        return out

    def _gemm_tc(self, x, w, od):
        """Two-block tcgen05 + TMA product for many rows (csrc/gemm_tc2.cu), bfloat16 result; None if the shape or the
        result type is not taken."""
        M, K = x.shape
        N = w.shape[0]
        if od != torch.bfloat16 or N % 8:
            return None
        out = torch.empty((M, N), dtype=od, device=x.device)
        rc = self.lib.mi_gemm_tc2(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, *self._tc2_scratch(), _p(self._stream_error), self._stream())
        if rc == -2:
            return None
        _check(rc, "gemm_tc2")
        self.launches += 1
        return out

    def _tc2_scratch(self):
        return (_p(self._tc2_ws), _c.c_longlong(self._tc2_ws.numel()), _p(self._tc2_counters), self._tc2_counters.numel())

    def check_errors(self):
        """Raises if a bounded wait inside a kernel ran out (synchronises the device)."""
        code = int(self._stream_error.item())
        if code != 0:
            self._stream_error.zero_()
            self._tc2_counters.zero_()
            raise RuntimeError(f"a pipeline wait inside a kernel ran out (code {code}: 1-2 gemm_stream, 21+ attention, 51-55 gemm_tc2)")

    # ---------------------------------------------------------------- q/k norm, rotation, cache write
    def qk_norm_rope_cache(self, qkv, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        T = qkv.shape[0]
        assert qkv.is_contiguous() and qkv.shape[1] == (H + 2 * KV) * D
        w_dtype = q_weight.dtype if q_weight is not None else qkv.dtype
        _check(self.lib.mi_qk_norm_rope_cache(
            _p(qkv), _p(q_weight), _p(k_weight), _p(inv_freq), _p(meta.positions), _p(meta.slots),
            _p(k_cache), _p(v_cache), T, H, KV, D, meta.page_size, _c.c_float(eps), _code(qkv.dtype),
            _code(w_dtype), self._stream()), "qk_norm_rope_cache")
        self.launches += 1
        return qkv[:, :H * D]

    # ---------------------------------------------------------------- attention over the pages
    def _cluster_fits(self, D, S, clusters):
        """Whether `clusters` clusters of S blocks of the staged decode kernel are resident at once, with the margin the
        kernel itself asks for (clusters are placed whole inside a GPC; a second wave costs more than the merge saves)."""
        key = (D, S)
        if key not in self._cluster_fit:
            self._cluster_fit[key] = int(self.lib.mi_attn_decode_cluster_fit(D, S))
        return clusters * 100 <= self._cluster_fit[key] * 92

    def choose_splits(self, ctas, max_kv_len, per_sm=2, cluster=False, head_dim=128):
        """Enough blocks to fill the GPU about twice, never more splits than the longest
        request has 256-key pieces (kernels/paged_attention/decode_triton.py:114-120).
        cluster: up to 8 splits can merge through distributed shared memory, which is worth more
        than finer splits while a split stays within ~1,000 keys (12.5 vs 14.8 us at batch 1, context 4096)."""
        if self.force_splits:
            return self.force_splits
        slots = per_sm * self.NUM_SMS                      # blocks resident at once
        most = max(1, min(math.ceil(max_kv_len / 256), 32))
        if ctas * most <= slots:
            return 8 if cluster and most > 8 and max_kv_len <= 8 * 1024 and self._cluster_fits(head_dim, 8, ctas) else most
        # more blocks than fit at once: take the fewest splits whose last wave is at least 85 % full
        best, best_eff = 1, 0.0
        for S in range(1, most + 1):
            total = ctas * S
            eff = total / (math.ceil(total / slots) * slots)
            if eff >= 0.85:
                # one split fewer if that lets the splits merge as clusters
                if cluster and 2 < S <= 8 and not self._cluster_fits(head_dim, S, ctas) and self._cluster_fits(head_dim, S - 1, ctas):
                    return S - 1
                return S
            if eff > best_eff:
                best, best_eff = S, eff
        return best

    def qkv_project(self, h, w, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        """q [T, H D] (a strided view is allowed) = rotated(normed(h @ w_q.T)); rotated(normed(k)) and v go to the rows' slots
        of the caches (None: this layer writes none).  The product, then the norm / rotation / cache-write kernel; one entry,
        so that the start-up timing of kernels sees the pair (a version with all of it in the GEMM's epilogue was measured
        and dropped: 76-92 us against 59 us for the pair at 2,048 rows)."""
        return self.qk_norm_rope_cache(self.linear(h, w), H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache)

    def paged_attention(self, q, k_cache, v_cache, meta, H, KV, D, scale, window):
        """meta: the step's arrays for this cache group.  seg_q_start, seg_pos0, seg_kv_len per entry; decode_segs (entries
        that feed one token), prefill_tiles / prefill_tiles2 ((entry, first row) per tile of meta.tile / 2 * meta.tile query
        rows); block_table [rows, max_pages] with entry i reading row table_rows[i] (row i when table_rows is None)."""
        T = q.shape[0]
        assert q.stride(1) == 1
        out = torch.empty((T, H * D), dtype=q.dtype, device=q.device)
        code, win = _code(q.dtype), int(window or 0)
        rows = getattr(meta, "table_rows", None)
        num_decode, num_tiles = meta.decode_segs.shape[0], meta.prefill_tiles.shape[0]
        tiles2 = getattr(meta, "prefill_tiles2", None)
        num_tiles2 = 0 if tiles2 is None else tiles2.shape[0]
        fast = (self.fast_attention and q.dtype == torch.bfloat16 and D in (64, 128) and q.stride(0) % 8 == 0
                and q.data_ptr() % 16 == 0)
        tc = (fast and self.tc_attention and num_tiles and meta.tile == 64 and meta.page_size % 8 == 0
              and 64 % meta.page_size == 0 and num_tiles2)
        if tc:
            rc = self.lib.mi_attn_prefill_tc(
                _p(q), q.stride(0), T, _p(k_cache), _p(v_cache), _c.c_longlong(k_cache.shape[0] * KV * meta.page_size),
                _p(out), _p(tiles2), num_tiles2, _p(meta.seg_q_start), _p(meta.seg_pos0),
                _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D, meta.page_size, 128, _c.c_float(scale), win,
                _p(self._stream_error), self._stream())
            _check(rc, "attn_prefill_tc")
            self.launches += 1
        elif num_tiles and fast and meta.tile == 64:
            _check(self.lib.mi_attn_prefill_mma(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(meta.prefill_tiles), num_tiles,
                _p(meta.seg_q_start), _p(meta.seg_pos0), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D,
                meta.page_size, meta.tile, _c.c_float(scale), win, self._stream()), "attn_prefill_mma")
            self.launches += 1
        elif num_tiles:
            _check(self.lib.mi_attn_prefill_generic(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(meta.prefill_tiles), num_tiles,
                _p(meta.seg_q_start), _p(meta.seg_pos0), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D,
                meta.page_size, meta.tile, _c.c_float(scale), win, code, self._stream()), "attn_prefill")
            self.launches += 1
        if not num_decode:
            return out
        fast_decode = fast and H // KV <= 16 and meta.page_size % 16 == 0
        S = self.choose_splits(num_decode * (KV if fast_decode else math.ceil(H / 4)), meta.max_kv_len,
                               (2 if self.bulk_decode else 3) if fast_decode else 2,
                               cluster=fast_decode and self.bulk_decode and self.cluster_merge, head_dim=D)
        o_part = lse = None
        if S > 1:
            o_part = torch.empty((num_decode, H, S, D), dtype=torch.float32, device=q.device)
            lse = torch.empty((num_decode, H, S), dtype=torch.float32, device=q.device)
        if fast_decode:
            counters = None
            if S > 1 and self.fused_merge:
                if num_decode * KV > self._merge_counters.numel():
                    raise ValueError(f"attn_decode: {num_decode} rows x {KV} kv heads exceed the {self._merge_counters.numel()} "
                                     "merge counters allocated at start-up")
                counters = self._merge_counters
            # without counters the splits stay in o_part / lse for the merge launch below: the cluster merge must be off too
            cluster = int(self.cluster_merge and counters is not None)
            _check(self.lib.mi_attn_decode_mma_rows(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(o_part), _p(lse), _p(meta.decode_segs),
                num_decode, _p(meta.seg_q_start), _p(meta.seg_kv_len), _p(meta.block_table), _p(rows), meta.max_pages,
                H, KV, D, meta.page_size, S, _c.c_float(scale), win, _p(counters),
                _p(self._stream_error if self.bulk_decode else None), k_cache.shape[0], cluster, self._stream()),
                "attn_decode_mma")
            self.launches += 1
            if S > 1 and counters is None:
                _check(self.lib.mi_attn_decode_merge(_p(o_part), _p(lse), _p(out), _p(meta.decode_segs), num_decode,
                                                     _p(meta.seg_q_start), H, D, S, code, self._stream()), "attn_merge")
                self.launches += 1
        else:
            _check(self.lib.mi_attn_decode_generic(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(o_part), _p(lse), _p(meta.decode_segs),
                num_decode, _p(meta.seg_q_start), _p(meta.seg_kv_len), _p(meta.block_table), _p(rows), meta.max_pages,
                H, KV, D, meta.page_size, S, _c.c_float(scale), win, code, self._stream()), "attn_decode")
            self.launches += 2 if S > 1 else 1
        return out

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        return self.sample(logits, None, None, None)

    def sample(self, logits, temperatures, seeds, counters):
        """logits float32 [R, V]; temperatures float32 [R] (0 = greedy); seeds, counters: int32
        tensors read as unsigned.  Returns int32 [R]."""
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if V >= 16384 and R <= 4096:                     # several blocks per row
            _check(self.lib.mi_sample_split(_p(logits), logits.stride(0), R, V, _p(temperatures), _p(seeds), _p(counters),
                                            _p(out), _p(self._sample_slots), _p(self._sample_arrivals), self._stream()),
                   "sample")
            self.launches += 1
            return out
        _check(self.lib.mi_sample(_p(logits), logits.stride(0), R, V, _p(temperatures), _p(seeds), _p(counters),
                                  _p(out), self._stream()), "sample")
        self.launches += 1
        return out


_OPS = {}


def get_ops(device) -> CudaOps:
    device = torch.device(device)
    key = (device.type, device.index)
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]
