#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200 at Qwen3-4B sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests at a context of 4,096 tokens, random
weights, bfloat16.  Prints ONE JSON line:
  value        decoded tokens per second, K steps timed on the device with CUDA events (graph
               replays; sampled tokens fed back on the device, metadata copied from pinned memory)
  e2e          the same through the Python entry point (LLM.step): host token ids in, host
               token ids out, every step
  prefill      one 2,048-token prompt: tokens/s, ms, and flops / time / measured bf16 peak
  roofline     the decode step's bytes (every weight once + the cache of the live requests)
               / its time, against the measured copy bandwidth
  points       decode tokens/s at batch 1 and 64 (context 4,096), and BASELINE's workload (512-token prompts + 256
               greedy tokens through the scheduler) at batch 1, 8 and 64
  check        logits of decode steps in the timed configuration against a float32 engine with the same weights
The weights (8 GB) and the cache are far larger than the 126 MB L2, so nothing is flushed
between steps.  More than one GPU is outside this engine: --gpus N>1 says so and exits 2.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 2560, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960,
}
FULL_LAYERS = 36


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), [x.strip() for x in line.split(",")]))

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            self.proc.wait()

    def summary(self, t0=None, t1=None):
        rows = [r for t, r in self.samples if (t0 is None or t0 <= t <= t1) and len(r) >= 6] or \
               [r for _, r in self.samples if len(r) >= 6]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(float(r[0]) for r in rows), "sm_max_mhz": float(rows[0][1]), "reasons": reasons}


def model_numbers(cfg, layers):
    h, H, KV, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["intermediate_size"], cfg["vocab_size"])
    per_layer = h * (H + 2 * KV) * D + H * D * h + 3 * h * I + 2 * h + 2 * D
    head = V * h
    return {"layer_params": per_layer, "head_params": head,
            "weight_bytes": 2 * (layers * per_layer + head + h), "kv_bytes_per_token": 2 * layers * KV * D * 2,
            "gemm_params": layers * (per_layer - 2 * h - 2 * D)}


def decode_device(llm, torch, batch, ctx, steps, warmup, vocab, clocks=None):
    """K graph-replayed decode steps at context ~ctx, timed with CUDA events.  The requests are
    prefilled through the engine itself; sampled tokens go back into the next step on the device."""
    from mini_inference_b200.engine.batch import StepEntry
    g = torch.Generator().manual_seed(batch)
    total = warmup + steps
    prompt_len = ctx - total - 1
    seqs = []
    for i in range(batch):
        seq = llm.cache.admit(("bench", batch, i), prompt_len + total + 1)
        assert seq is not None, "cache too small for the benchmark"
        ids = torch.randint(0, vocab, (prompt_len,), generator=g).tolist()
        for a in range(0, prompt_len, 2048):                       # the engine's own prefill, 2,048 tokens a step
            llm.runner.step([StepEntry(seq, ids[a:a + 2048], [])])
        seqs.append(seq)
    G = llm.graphs
    B = G.bucket_for(batch)
    first = torch.randint(0, vocab, (batch,), generator=g).tolist()
    launches0 = llm.ops.launches
    h2d = 0
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = t1 = None
    for i in range(total):
        if i == warmup:
            torch.cuda.synchronize()
            launches0 = llm.ops.launches
            t0 = time.perf_counter()
            start.record()
        for s in seqs:
            assert llm.cache.ensure(s, s.num_tokens + 1)
        h2d = G.fill(B, seqs, first if i == 0 else None)
        G.replay(B)
        G.feed_back(B)
        for s in seqs:
            llm.cache.commit(s, s.num_tokens + 1)
    stop.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = start.elapsed_time(stop) / steps
    launches = llm.ops.launches - launches0
    mean_ctx = sum(s.num_tokens for s in seqs) / batch - steps / 2
    for s in seqs:
        llm.cache.free(s)
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "launches": launches, "h2d": h2d, "ctx": mean_ctx, "t": (t0, t1)}


def decode_e2e(llm, torch, batch, ctx, steps, warmup, vocab):
    """The same decode steps through LLM.step(): scheduler, metadata from the host, graph replay,
    sampled tokens read back to the host, every step."""
    from mini_inference_b200.engine.request import SamplingParams
    g = torch.Generator().manual_seed(1000 + batch)
    total = warmup + steps
    # requests are admitted one a step (each prompt fills the token budget), so the first ones
    # already decode while the last are prefilled: leave room for those extra tokens
    prompt_len = ctx - total - batch - 4
    reqs = [llm.add_request(torch.randint(0, vocab, (prompt_len,), generator=g).tolist(),
                            SamplingParams(max_new_tokens=total + batch + 2, ignore_eos=True)) for _ in range(batch)]
    while any(not r.output_ids for r in reqs):
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        llm.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    while llm.has_work():
        llm.step()
    return {"tok_s": batch * steps / dt, "h2d": llm.graphs.last_h2d_bytes, "d2h": 4 * batch}


def prefill(llm, torch, tokens, vocab, warmup=3, reps=3, pause=0.0):
    """Best time of one prompt step.  pause: idle seconds before each timed repetition.  Back-to-back repetitions
    bring the GPU under its power cap within a few of them (14.2, 15.3, 16.2, 16.3 ms measured in a row); the bf16 peak
    this step is compared with is the burst figure of an idle GPU, so the step is timed the same way."""
    from mini_inference_b200.engine.batch import StepEntry
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, vocab, (tokens,), generator=g).tolist()
    times = []
    for i in range(warmup + reps):
        seq = llm.cache.admit(("prefill", i), tokens)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if pause and i >= warmup:
            time.sleep(pause)
        start.record()
        llm.runner.step([StepEntry(seq, ids, [tokens - 1])])
        stop.record()
        torch.cuda.synchronize()
        llm.cache.free(seq)
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    return min(times)


def generate_workload(llm, torch, batch, prompt_len, new_tokens, vocab):
    """BASELINE's decode workload through the scheduler: `batch` concurrent requests, each a prompt_len-token random
    prompt and new_tokens greedy tokens.  Decode rate = tokens delivered after the last request's first token / the
    time from then to the end."""
    from mini_inference_b200.engine.request import SamplingParams
    g = torch.Generator().manual_seed(2000 + batch)
    reqs = [llm.add_request(torch.randint(0, vocab, (prompt_len,), generator=g).tolist(),
                            SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)) for _ in range(batch)]
    while llm.has_work():
        llm.step()
    torch.cuda.synchronize()
    assert all(r.error is None and len(r.output_ids) == new_tokens for r in reqs)
    t0 = max(r.times.tokens[0] for r in reqs)
    t1 = max(r.times.finished for r in reqs)
    tokens = sum(sum(1 for t in r.times.tokens if t > t0) for r in reqs)
    return tokens / (t1 - t0)


def logit_check(llm, torch, LLM, cfg, vocab, prompt_len=512, steps=8):
    """One request in the state the decode timing runs in (start-up choice of GEMM kernels, partial sums handed to the
    norm kernels, weight prefetch hints, graph replay from a bucket) against a float32 engine holding the same weights:
    relative error of the decode steps' logits, and how many of the float32 argmax tokens the bfloat16 path picks."""
    from mini_inference_b200.engine.batch import StepEntry
    g = torch.Generator().manual_seed(99)
    ids = torch.randint(0, vocab, (prompt_len + steps,), generator=g).tolist()
    G = llm.graphs
    B = G.bucket_for(1)
    seq = llm.cache.admit(("check", 0), prompt_len + steps + 1)
    llm.runner.step([StepEntry(seq, ids[:prompt_len], [])])
    got = []
    for k in range(steps):
        assert llm.cache.ensure(seq, seq.num_tokens + 1)
        G.fill(B, [seq], [ids[prompt_len + k]])
        G.replay(B)
        got.append(G.logits_out[B][0].float().clone())
        llm.cache.commit(seq, seq.num_tokens + 1)
    llm.cache.free(seq)
    got = torch.stack(got)
    # the same steps on the plainest bfloat16 path (eager, library products, nothing deferred): what 16-bit rounding
    # alone costs at this depth, to read the timed path's error against
    saved = (llm.ops._linear_choice, llm.ops.defer_sums, llm.ops.stream_gemm, llm.ops.skinny_gemm)
    llm.ops._linear_choice, llm.ops.defer_sums, llm.ops.stream_gemm, llm.ops.skinny_gemm = None, False, False, False
    try:
        seq = llm.cache.admit(("check", 1), prompt_len + steps + 1)
        llm.runner.step([StepEntry(seq, ids[:prompt_len], [])])
        base = torch.cat([llm.runner.step([StepEntry(seq, [ids[prompt_len + k]], [0])]).float() for k in range(steps)])
        llm.cache.free(seq)
    finally:
        llm.ops._linear_choice, llm.ops.defer_sums, llm.ops.stream_gemm, llm.ops.skinny_gemm = saved
    ref_llm = LLM(None, random_config=cfg, random_seed=0, dtype="float32", device="cuda:0", kv_block_size=16,
                  kv_cache_tokens=2048, kv_watermark=0.0, max_num_seqs=1, max_model_len=2048, cuda_graphs=False,
                  random_draw_dtype="bfloat16")
    ref = ref_llm.score(ids)[prompt_len:].float()
    del ref_llm
    err = ((got - ref).abs().max() / ref.abs().max()).item()
    agree = int((got.argmax(-1) == ref.argmax(-1)).sum())
    base_err = ((base - ref).abs().max() / ref.abs().max()).item()
    return {"logit_rel_err_vs_fp32": round(err, 5), "library_bf16_path_rel_err_vs_fp32": round(base_err, 5),
            "argmax_agree": f"{agree}/{steps}", "rows": steps, "context": prompt_len}


def reference_arm(args):
    """The unmodified reference engine on the same workload (baseline/reference_arm.py drives the copy of its checkout
    under baseline/_ref through its own switches and public calls); its JSON line is passed on as it is."""
    pk = peaks()
    cmd = [sys.executable, os.path.join(ROOT, "baseline", "reference_arm.py"), "--steps", str(args.steps), "--warmup",
           str(args.warmup), "--batch", str(args.batch), "--ctx", str(args.ctx), "--layers", str(args.layers),
           "--peak-tflops", str(pk["bf16_tflops"]), "--peak-gbs", str(pk["hbm_gbs"])]
    if args.skip_points:
        cmd.append("--skip-points")
    with ClockSampler() as clocks:
        try:
            r = subprocess.run(cmd, stdout=subprocess.PIPE, text=True, timeout=1500)
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
            out = json.loads(lines[-1]) if lines else {"impl": "reference", "unavailable":
                                                       f"the reference arm printed no result (exit code {r.returncode})"}
        except subprocess.TimeoutExpired:
            out = {"impl": "reference", "unavailable": "the reference arm did not finish within 25 minutes"}
        if "unavailable" not in out:
            out["clocks"] = clocks.summary()
            out["gpu_launches"] = None
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-check", action="store_true", help="leave out the logits check against the float32 path")
    args = ap.parse_args()
    if args.gpus > 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported (use --gpus 1)")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    from mini_inference_b200.engine.llm import LLM

    cfg = dict(QWEN3_4B, num_hidden_layers=args.layers)
    vocab = cfg["vocab_size"]
    pk = peaks()
    nums = model_numbers(cfg, args.layers)
    kv_tokens = max(64, args.batch) * args.ctx + 4096
    llm = LLM(None, random_config=cfg, random_seed=0, dtype="bfloat16", device="cuda:0", kv_block_size=16,
              kv_cache_tokens=kv_tokens, kv_watermark=0.0, max_num_seqs=max(64, args.batch), max_model_len=args.ctx,
              max_batched_tokens=4096, cuda_graphs=False)

    # the prompt step first, then the start-up work of the decode path (kernel timing, graph capture): seconds of
    # back-to-back GEMMs put the GPU under its power cap, and the peak this step is compared with is a burst figure.
    # It is an eager step of ~330 launches: the clock sampler's queries (which belong to the decode run) start after it
    pre_ms = prefill(llm, torch, 2048, vocab, warmup=3, reps=5, pause=0.25)
    with ClockSampler() as clocks:
        llm.enable_cuda_graphs()
        main_run = decode_device(llm, torch, args.batch, args.ctx, args.steps, args.warmup, vocab)
        clock_summary = clocks.summary(*main_run["t"])
        e2e = decode_e2e(llm, torch, args.batch, args.ctx, args.steps, args.warmup, vocab)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                r = decode_device(llm, torch, b, args.ctx, max(16, args.steps // 4), args.warmup, vocab)
                points[f"decode_b{b}"] = round(r["tok_s"], 1)
            # BASELINE.json's own decode workload: 512-token prompts + 256 greedy tokens, through the scheduler
            for b in (1, 8, 64):
                points[f"gen512_256_b{b}"] = round(generate_workload(llm, torch, b, 512, 256, vocab), 1)
        check = None if args.skip_check else logit_check(llm, torch, LLM, cfg, vocab)

    step_bytes = nums["weight_bytes"] + args.batch * main_run["ctx"] * nums["kv_bytes_per_token"]
    achieved = step_bytes / (main_run["ms"] * 1e-3) / 1e9
    H, D, L = cfg["num_attention_heads"], cfg["head_dim"], args.layers
    T = 2048
    pre_flops = 2 * T * nums["gemm_params"] + 2 * nums["head_params"] + L * 4 * H * D * T * (T + 1) / 2
    out = {
        "metric": "Qwen3-4B decode tok/s at batch 8, context 4096 (prefill tok/s at 2,048 tokens in 'prefill')",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights (seeded), uniform-random token ids",
        "config": {
            "model": "Qwen3-4B-size", "layers": args.layers, "model_layers": FULL_LAYERS, "hidden": cfg["hidden_size"],
            "q_heads": H, "kv_heads": cfg["num_key_value_heads"], "head_dim": D, "intermediate": cfg["intermediate_size"],
            "vocab": vocab, "tied": True, "global_batch": args.batch, "seq_len": args.ctx, "page_size": 16,
            "parallelism": "single GPU", "cuda_graphs": True, "l2": "inputs larger than L2 (8 GB weights + cache)",
            "peaks": pk["source"], "prefill_timing": "best of 5, each after 0.25 s idle (burst, like the bf16 peak)",
        },
        "clocks": clock_summary,
        "e2e": {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(T / (pre_ms * 1e-3), 1), "tokens": T, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "check": check,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
