"""A small, bounded run of one kind of step for a profiler (ncu --profile-from-start off
captures only what lies between cudaProfilerStart and cudaProfilerStop):

    python -m mini_inference_b200.cli.profile_step decode|prefill --size 4b --layers 2 --batch 8 --ctx 4096 --steps 2

decode: no prefill runs before the decode steps (the cache holds zeros at the given context
length), one graph bucket, few launches.  Which kernel runs each product is timed at start-up;
under a profiler those timings are distorted, so a plain run can save its table (--choices FILE)
and the profiled run of the same command reads it back.  The reference wraps its measured runs
in the framework's profiler instead (bench/run_engine.py:126-131, profiling/torch_profiler.py)."""
from __future__ import annotations

import argparse
import json
import os
import sys

from .run_engine import SIZES


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("kind", choices=["decode", "prefill"])
    ap.add_argument("--size", default="4b", choices=sorted(SIZES))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048, help="prefill: tokens of the prompt")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--choices", default=None, help="decode: file to keep the start-up choice of GEMM kernels in")
    a = ap.parse_args(argv)

    import torch

    from ..engine.batch import StepEntry
    from ..engine.graphs import DecodeGraphs
    from ..engine.llm import LLM

    cfg = dict(dict(architectures=["Qwen3ForCausalLM"], rms_norm_eps=1e-6, max_position_embeddings=40960), **SIZES[a.size])
    if a.layers:
        cfg["num_hidden_layers"] = a.layers
    vocab = cfg["vocab_size"]
    llm = LLM(None, random_config=cfg, random_seed=0, dtype="bfloat16", device="cuda:0", kv_block_size=a.page_size,
              kv_cache_tokens=a.batch * a.ctx + 4096, kv_watermark=0.0, max_num_seqs=a.batch, max_model_len=a.ctx,
              max_batched_tokens=max(4096, a.tokens), cuda_graphs=False)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.kind == "prefill":
        g = torch.Generator().manual_seed(7)
        ids = torch.randint(0, vocab, (a.tokens,), generator=g).tolist()

        def run(i):
            seq = llm.cache.admit(("prefill", i), a.tokens)
            llm.runner.step([StepEntry(seq, ids, [a.tokens - 1])])
            llm.cache.free(seq)
        for i in range(a.warmup):
            run(i)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        start.record()
        for i in range(a.steps):
            run(a.warmup + i)
        stop.record()
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(f"prefill {a.tokens} tokens: {start.elapsed_time(stop) / a.steps:.3f} ms")
        own = sorted(k for k, v in (llm.many_row_tuning or {}).items() if v["best"] == "tc2")
        print("many-row products on the own tcgen05 GEMM:", ", ".join(own) if own else "none")
        llm.ops.check_errors()
        return 0
    if a.choices and os.path.isfile(a.choices):
        with open(a.choices) as f:
            llm.ops._linear_choice = {tuple(int(v) for v in k.split(",")): c for k, c in json.load(f).items()}
    else:
        llm.ops.tune_linear(llm.model.matrix_weights(), {tuple(llm.model.lm_head.shape): torch.float32},
                            deferrable=llm.model.deferrable_shapes(), gated=llm.model.gated_shapes())
        if a.choices:
            with open(a.choices, "w") as f:
                json.dump({",".join(str(v) for v in k): c for k, c in llm.ops._linear_choice.items()}, f)
    llm.graphs = DecodeGraphs(llm.runner, a.batch, buckets=[a.batch])
    llm.graphs.capture()
    seqs = []
    for i in range(a.batch):
        seq = llm.cache.admit(("p", i), a.ctx)
        llm.cache.ensure(seq, a.ctx - a.steps - a.warmup - 1)
        llm.cache.commit(seq, a.ctx - a.steps - a.warmup - 1)
        seqs.append(seq)
    G, B = llm.graphs, a.batch
    for i in range(a.warmup + a.steps):
        if i == a.warmup:
            torch.cuda.profiler.start()
            start.record()
        for s in seqs:
            llm.cache.ensure(s, s.num_tokens + 1)
        G.fill(B, seqs, [1] * B if i == 0 else None)
        G.replay(B)
        G.feed_back(B)
        for s in seqs:
            llm.cache.commit(s, s.num_tokens + 1)
    stop.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print(f"decode b{B} ctx{a.ctx}: {start.elapsed_time(stop) / a.steps:.3f} ms/step, {G.launches[B]} own kernels per step")
    llm.ops.check_errors()
    return 0


if __name__ == "__main__":
    sys.exit(main())
