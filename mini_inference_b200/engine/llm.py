"""The Python entry point: model folder in, generated token ids out.

The reference's CustomEngine (engine/custom_engine.py:19-330) wires loader, cache, runner,
scheduler and sampler and runs the step loop on a background thread for its HTTP server.  The
same wiring and the same loop body live here, driven synchronously by the caller:
add_request() / step() / has_work(), or generate() for a list of prompts.  Token ids are the
native interface (there is no tokenizer in this engine)."""
from __future__ import annotations

import contextlib
import time
from typing import List, Optional, Sequence, Union

import torch

from ..cache.manager import CacheManager
from ..config.engine_args import EngineArgs
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .factory import DTYPES, load_model
from .request import RUNNING, Request, SamplingParams
from .runner import ModelRunner
from .scheduler import Scheduler, Span


class LLM:
    def __init__(self, model_dir: Optional[str], args: Optional[EngineArgs] = None, ops=None,
                 random_config: Optional[dict] = None, random_seed: int = 0, random_std: float = 0.02,
                 random_draw_dtype: Optional[str] = None, **overrides):
        """model_dir: a folder with config.json and model.safetensors.  With model_dir=None and
        random_config (a config.json dict) the weights are drawn on the device instead (random_draw_dtype: the type
        they are drawn in before they are cast to the engine's, so that a float32 engine can hold exactly the values
        of a bfloat16 one)."""
        args = args or EngineArgs()
        for k, v in overrides.items():
            if not hasattr(args, k):
                raise TypeError(f"unknown engine setting '{k}'")
            setattr(args, k, v)
        args.__post_init__()
        self.args = args
        t0 = time.perf_counter()
        if model_dir is not None:
            self.config, self.model, self.load_info = load_model(model_dir, args.dtype, args.device)
        else:
            from ..config.registry import resolve
            from ..parts.model import DecoderModel
            from ..weights.random_init import init_random_on_device
            arch = resolve(random_config)
            self.config = arch.config_class.from_dict(random_config)
            self.model = DecoderModel(arch.build_spec(self.config))
            self.load_info = init_random_on_device(self.model, DTYPES[args.dtype], args.device, random_seed, random_std,
                                                   draw_dtype=DTYPES[random_draw_dtype] if random_draw_dtype else None)
        self.load_info["load_time_s"] = round(time.perf_counter() - t0, 3)
        self.model_dir = model_dir
        self.device, self.dtype = self.model.device, DTYPES[args.dtype]
        # engine/custom_engine.py:28: the model's own limit, capped by MAX_MODEL_LEN
        self.max_model_len = min(self.model.spec.max_position, args.max_model_len)
        needs = self.model.cache_needs()
        probe = CacheManager(needs, args.kv_block_size, 1, 1, args.kv_block_size, dtype=self.dtype, allocate=False)
        tokens = self._kv_budget_tokens(probe.bytes_per_token(), args.max_num_seqs * probe.state_bytes_per_seq())
        num_pages = max(1, tokens // args.kv_block_size)
        self.cache = CacheManager(needs, args.kv_block_size, num_pages, args.max_num_seqs,
                                  min(self.max_model_len, num_pages * args.kv_block_size),
                                  dtype=self.dtype, device=self.device, watermark=args.kv_watermark)
        self.runner = ModelRunner(self.model, self.cache, ops)
        self.ops = self.runner.ops
        self.scheduler = Scheduler(self.cache, args.max_num_seqs, args.max_batched_tokens, self.max_model_len,
                                   chunked_prefill=args.chunked_prefill)
        self.sampler = Sampler(self.ops, args.seed)
        self.eos_ids = set(self.model.spec.eos_token_ids)
        self.graphs = None
        self.linear_tuning = None
        # which kernel runs the many-row products of prompt steps is timed on this model's weights (the few-row products
        # of decode steps are timed when the decode graphs are made)
        self.many_row_tuning = None
        if self.dtype == torch.bfloat16 and hasattr(self.ops, "tune_many_rows"):
            self.many_row_tuning = self.ops.tune_many_rows(self.model.matrix_weights(), self.model.first_product_probes(self.ops))
        if args.cuda_graphs:
            self.enable_cuda_graphs()
        self.last_error = None
        self._ahead = None               # (chunks, handle) of a decode step launched but not yet delivered
        # step wall time split by kind (engine/custom_engine.py:69,140-142)
        self.step_time = {"decode": [0, 0.0], "other": [0, 0.0]}
        # what those steps had to move and to compute, by the byte model of profiling/analyze.py:111-117 in the reference:
        # a decode step reads every weight once and the cache of its requests; a step with prompt tokens is counted in flops
        self.step_work = {"decode_bytes": 0, "other_flops": 0}
        self._weight_bytes = int(self.load_info.get("weight_bytes", 0))
        self._kv_bytes_per_token = self.cache.bytes_per_token()

    # ---------------------------------------------------------------- setup
    def enable_cuda_graphs(self):
        """Time the few-row GEMM kernels on this model's weights and capture the decode graphs (what cuda_graphs=True
        does at construction; may also be called later, between steps)."""
        if self.graphs is not None:
            return
        if self.dtype == torch.bfloat16 and hasattr(self.ops, "tune_linear"):
            self.linear_tuning = self.ops.tune_linear(self.model.matrix_weights(),
                                                      {tuple(self.model.lm_head.shape): torch.float32},
                                                      deferrable=self.model.deferrable_shapes(),
                                                      gated=self.model.gated_shapes())
        from .graphs import DecodeGraphs
        self.graphs = DecodeGraphs(self.runner, self.args.max_num_seqs)
        self.graphs.capture()
        self.args.cuda_graphs = True

    def _kv_budget_tokens(self, bytes_per_token: int, state_bytes: int = 0) -> int:
        """engine/custom_engine.py:105-121: fixed token count, fixed megabytes, or what the GPU
        has left after the weights and a reserve for activations.  A memory budget first pays for the
        fixed-size state of max_num_seqs requests (state_bytes); pages get the rest."""
        a = self.args
        if a.kv_cache_tokens:
            return a.kv_cache_tokens
        if a.kv_cache_mb:
            return int(max(a.kv_cache_mb * 1024 ** 2 - state_bytes, 0) // max(bytes_per_token, 1))
        if self.device.type != "cuda":
            return 32768
        free, total = torch.cuda.mem_get_info(self.device)
        budget = total * a.gpu_memory_utilization - (total - free) - a.activation_reserve_gb * 1024 ** 3 - state_bytes
        return max(int(max(budget, 0) // max(bytes_per_token, 1)), 1024)

    # ---------------------------------------------------------------- requests
    def add_request(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None) -> Request:
        ids = [int(t) for t in prompt_ids]
        if not ids:
            raise ValueError("the prompt is empty")                       # engine/custom_engine.py:189-190
        if min(ids) < 0 or max(ids) >= self.model.spec.vocab_size:
            raise ValueError(f"token id outside [0, {self.model.spec.vocab_size})")
        limit = min(self.max_model_len, self.cache.capacity_tokens)
        if len(ids) >= limit:
            raise ValueError(f"prompt is {len(ids)} tokens; the limit is {limit - 1}")   # :191-193
        params = params or SamplingParams(max_new_tokens=self.args.max_new_tokens)
        params = SamplingParams(max_new_tokens=min(params.max_new_tokens, limit - len(ids)),
                                temperature=params.temperature, seed=params.seed, ignore_eos=params.ignore_eos)
        req = Request(prompt_ids=ids, params=params)
        self.scheduler.add(req)
        return req

    # ---------------------------------------------------------------- the loop body
    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._ahead is not None

    def step(self) -> List[Request]:
        """Schedule, run, sample, deliver (engine/custom_engine.py:124-170).  Returns the
        requests that finished in this step.

        With CUDA graphs and overlap_decode a decode step is delivered one call after it was
        launched: the call launches the step after it first (its input tokens are this step's
        samples, still on the device), then waits for this step's tokens and does the bookkeeping
        while the GPU already runs the next one."""
        start = time.perf_counter()
        if self._ahead is not None:
            chunks, handle = self._ahead
            self._ahead = None
        else:
            chunks = self.scheduler.schedule(start)
            if not chunks:
                return self._fail_unschedulable()
            handle = None
            try:
                with self._label(chunks):
                    if self.graphs is not None and self.graphs.can_run(chunks):
                        handle = self.graphs.launch(chunks, self.sampler)
                    else:
                        tokens = self._run(chunks)
            except Exception as e:
                return self._abort(e)
            if handle is None:
                self._time_step(chunks, start)
                return self._deliver(chunks, tokens)
        try:
            nxt = self._launch_ahead(chunks)
            tokens = self.graphs.read(handle)
        except Exception as e:
            return self._abort(e)
        self._time_step(chunks, start)
        done = self._deliver(chunks, tokens)
        self._ahead = nxt
        return done

    def _launch_ahead(self, chunks):
        """The decode step after the one in flight, for the same requests in the same rows, if it is
        certain that all of them go on (nobody waits to be admitted, nobody reaches a length limit,
        everybody gets a page); a request that turns out to have stopped on EOS is skipped at delivery."""
        if not self.args.overlap_decode or self.scheduler.waiting:
            return None
        reqs = [r for r, _, _ in chunks]
        if len(reqs) != len(self.scheduler.running) or any(a is not b for a, b in zip(reqs, self.scheduler.running)):
            return None
        for req, _, end in chunks:
            if req.state != RUNNING or end != req.total_len:
                return None                                              # a row of the step in flight is already dead
            if len(req.output_ids) + 2 > req.params.max_new_tokens or end + 2 > self.max_model_len:
                return None                                              # it finishes with the step in flight
        for req, _, end in chunks:
            if not self.cache.ensure(req.seq, end + 1):
                return None                                              # out of pages: the scheduler decides who yields
        ahead = [Span(req, end, end + 1) for req, _, end in chunks]
        self.scheduler.count_decode_step(len(ahead))
        return ahead, self.graphs.launch(ahead, self.sampler, on_device_tokens=True)

    def _time_step(self, chunks, start):
        kind = "decode" if all(e - s == 1 and s > 0 for _, s, e in chunks) else "other"
        self.step_time[kind][0] += 1
        self.step_time[kind][1] += (time.perf_counter() - start) * 1e3
        if kind == "decode":
            self.step_work["decode_bytes"] += self._weight_bytes + self._kv_bytes_per_token * sum(e for _, _, e in chunks)
        else:
            rows = sum(e - s for _, s, e in chunks)
            pairs = sum((e - s) * (s + e + 1) // 2 for _, s, e in chunks)          # (query, visible key) pairs
            heads = sum(1 for r, _, e in chunks if e == r.total_len)
            self.step_work["other_flops"] += self.model.step_flops(rows, pairs, heads)

    def _abort(self, e):
        """Fail this batch, keep serving."""
        self.last_error = f"{type(e).__name__}: {e}"
        self._ahead = None
        done = self.scheduler.abort_all()
        for r in done:
            r.close("error", error=self.last_error)
        return done

    def _deliver(self, chunks, tokens) -> List[Request]:
        now = time.perf_counter()
        done, row = [], 0
        for req, _, end in chunks:
            if req.state != RUNNING:                                     # stopped while this step was already in flight
                row += 1
                continue
            req.num_computed = end
            if end < req.total_len:                                      # prompt not finished yet
                continue
            tok = tokens[row]
            row += 1
            req.deliver(tok, now)
            eos = tok in self.eos_ids and not req.params.ignore_eos
            if eos or len(req.output_ids) >= req.params.max_new_tokens or req.total_len >= self.max_model_len:
                self.scheduler.finish(req)
                req.close("stop" if eos else "length")
                done.append(req)
        return done

    def _run(self, chunks) -> List[int]:
        if self.graphs is not None:
            out = self.graphs.run(chunks, self.sampler)
            if out is not None:
                return out
        entries, sampled = [], []
        for req, s, e in chunks:
            last = e == req.total_len
            entries.append(StepEntry(req.seq, req.span(s, e), [e - s - 1] if last else []))
            if last:
                sampled.append(req)
        logits = self.runner.step(entries, ensure=False)
        if logits is None:
            return []
        return self.sampler.sample(logits, sampled).tolist()             # the step's one device->host sync

    def _label(self, plan):
        """A profiler range per step, in the reference's wording (engine/core/model_runner.py:98-102):
        forward(T=tokens, decode=rows, prefill=rows, ctx=keys).  Only with NVTX=1 (the reference's switch)."""
        if not self.args.nvtx or self.device.type != "cuda":
            return contextlib.nullcontext()
        dec = sum(1 for s in plan if s.is_decode)
        return torch.cuda.nvtx.range(f"forward(T={plan.num_tokens}, decode={dec}, prefill={len(plan) - dec}, "
                                     f"ctx={sum(s.end for s in plan)})")

    def _fail_unschedulable(self):
        """Nothing could be scheduled.  If nothing runs either, the request at the head of the
        queue can never fit (its pages plus the watermark exceed the pool): fail it instead of
        spinning."""
        if self.scheduler.running or not self.scheduler.waiting:
            return []
        req = self.scheduler.waiting.popleft()
        req.close("error", error=f"request of {req.total_len} tokens does not fit in the cache "
                                 f"({self.cache.capacity_tokens} tokens)")
        return [req]

    # ---------------------------------------------------------------- public API
    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[List[int]]:
        """Token ids in, generated token ids out, one list per prompt."""
        if params is None or isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.has_work():
            self.step()
        for r in reqs:
            if r.error:
                raise RuntimeError(f"request {r.id} failed: {r.error}")
        if hasattr(self.ops, "check_errors"):
            self.ops.check_errors()                    # a bounded wait inside a kernel ran out: the tokens cannot be trusted
        return [list(r.output_ids) for r in reqs]

    def score(self, token_ids: Sequence[int]) -> torch.Tensor:
        """float32 logits for every position, through the paged cache (engine/custom_engine.py:279-296)."""
        seq = self.cache.admit(("score", id(token_ids)), len(token_ids))
        if seq is None:
            raise RuntimeError("not enough free cache to score this sequence")
        try:
            return self.runner.step([StepEntry(seq, token_ids, range(len(token_ids)))])
        finally:
            self.cache.free(seq)

    def stats(self) -> dict:
        t = {"decode_steps_timed": self.step_time["decode"][0],
             "decode_step_ms_total": round(self.step_time["decode"][1], 3),
             "other_steps_timed": self.step_time["other"][0],
             "other_step_ms_total": round(self.step_time["other"][1], 3),
             "decode_bytes_total": self.step_work["decode_bytes"], "other_flops_total": self.step_work["other_flops"]}
        g = self.graphs.stats() if self.graphs is not None else {}
        return {**self.scheduler.stats(), **self.cache.stats(), **g, **t}

    def info(self) -> dict:
        """What the reference records in every result file (engine/base.py:35-49,
        engine/custom_engine.py:298-321)."""
        return {
            "engine": "mini_inference_b200", "model": self.model_dir, "architecture": self.config.architecture,
            "dtype": self.args.dtype, "max_model_len": self.max_model_len, "scheduler": "continuous",
            "kv_cache": "paged", "kv_block_size": self.args.kv_block_size, "kv_watermark": self.args.kv_watermark,
            "kv_capacity_tokens": self.cache.capacity_tokens,
            "kv_cache_mb": round(self.cache.capacity_tokens * self.cache.bytes_per_token() / 1024 ** 2, 1),
            "max_num_seqs": self.args.max_num_seqs, "max_batched_tokens": self.args.max_batched_tokens,
            "chunked_prefill": self.args.chunked_prefill, "cuda_graphs": self.graphs is not None,
            "weights": self.load_info,
        }


def create_engine(model_dir: str, **settings) -> LLM:
    """Counterpart of the reference's create_engine() (engine/factory.py:5-10)."""
    return LLM(model_dir, **settings)
