"""Run the engine directly from the command line, in the manner of the reference's
bench/run_engine.py (flags :31-77, summary :164-203): N prompts, C at a time, through the
Python entry point; prints per-request timings and a summary, optionally writes JSON.

Option names and meanings follow the reference where it has them (-n/--num-prompts,
-c/--concurrency, --warmup, --max-new-tokens, --cuda-graphs, --chunked-prefill,
--max-batched-tokens, --kv-tokens, --model, --out).  Prompts are seeded random token ids of
--prompt-len tokens (this engine has no tokenizer; the reference's --prompt/--prompt-words
build text).  --model is a model folder; --random-weights SIZE (or --config FILE, a config.json)
draws weights on the device.  --roofline adds what the reference's profiling report computes
from its byte model (profiling/analyze.py:111-117,271-277): bytes a decode step has to read
(every weight once + the cache of its requests) over its time, flops of the steps with prompt
tokens over theirs, each as a fraction of this GPU's measured peaks."""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time

SIZES = {
    "tiny": dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                 intermediate_size=128, vocab_size=256, rope_theta=10000.0, tie_word_embeddings=True),
    "tinyA": dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                  intermediate_size=128, vocab_size=256, rope_theta=10000.0, tie_word_embeddings=True),
    "tinyB": dict(hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3, head_dim=32,
                  intermediate_size=224, vocab_size=512, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False),
    "4b": dict(hidden_size=2560, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=9728, vocab_size=151936, rope_theta=1e6, tie_word_embeddings=True),
    "8b": dict(hidden_size=4096, num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=12288, vocab_size=151936, rope_theta=1e6, tie_word_embeddings=False),
    "14b": dict(hidden_size=5120, num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=8, head_dim=128,
                intermediate_size=17408, vocab_size=151936, rope_theta=1e6, tie_word_embeddings=False),
}


def parse_len(text):
    lo, _, hi = text.partition(":")
    return (int(lo), int(hi or lo))


def measured_peaks():
    """MEASURED_PEAKS.json (copy bandwidth in GB/s, bf16 GEMM TFLOP/s of this GPU) from the working directory or from
    beside the package; else an earlier measurement of a B200, marked as a fall-back."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    for d in (os.getcwd(), here):
        path = os.path.join(d, "MEASURED_PEAKS.json")
        if os.path.isfile(path):
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "source": "fallback"}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="Run the engine directly")
    p.add_argument("-n", "--num-prompts", type=int, default=3)
    p.add_argument("-c", "--concurrency", type=int, default=1, help="requests in flight at once")
    p.add_argument("--warmup", type=int, default=2, help="warmup runs, not measured")
    p.add_argument("--max-new-tokens", type=int, default=128)
    p.add_argument("--prompt-len", default="32", help="prompt length in tokens, N or lo:hi (uniform)")
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--sampling-seed", type=int, default=0)
    p.add_argument("--model", default=None, help="model folder (config.json + model.safetensors)")
    p.add_argument("--random-weights", default=None, choices=sorted(SIZES), help="draw weights of this size instead")
    p.add_argument("--config", default=None, help="draw weights for this config.json file instead")
    p.add_argument("--layers", type=int, default=None, help="with random weights: fewer layers than the size has")
    p.add_argument("--backend", default="cuda", choices=["cuda"],
                   help="kernels: this package's CUDA kernels (there is no other backend)")
    p.add_argument("--roofline", action="store_true", help="add achieved GB/s, TFLOP/s and their fractions of the measured peaks")
    p.add_argument("--seed", type=int, default=0, help="seed of the random weights and prompts")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    p.add_argument("--cuda-graphs", default=None, choices=["on", "off"])
    p.add_argument("--chunked-prefill", default=None, choices=["on", "off"])
    p.add_argument("--overlap-decode", default=None, choices=["on", "off"],
                   help="with CUDA graphs: launch the next decode step before reading this one's tokens (default on)")
    p.add_argument("--max-batched-tokens", type=int, default=None, help="per-step token budget")
    p.add_argument("--max-num-seqs", type=int, default=None)
    p.add_argument("--max-model-len", type=int, default=None)
    p.add_argument("--kv-tokens", type=int, default=None, help="fix the cache pool size in tokens")
    p.add_argument("--kv-mb", type=float, default=None)
    p.add_argument("--page-size", type=int, default=None)
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--out", default=None, help="optional JSON file for the results")
    a = p.parse_args(argv)
    if sum(x is not None for x in (a.model, a.random_weights, a.config)) != 1:
        p.error("give exactly one of --model DIR, --random-weights SIZE and --config FILE")

    from ..engine.llm import LLM
    from ..engine.request import SamplingParams

    settings = dict(dtype=a.dtype, device=a.device, seed=a.sampling_seed)
    for key, val in (("cuda_graphs", None if a.cuda_graphs is None else a.cuda_graphs == "on"),
                     ("chunked_prefill", None if a.chunked_prefill is None else a.chunked_prefill == "on"),
                     ("overlap_decode", None if a.overlap_decode is None else a.overlap_decode == "on"),
                     ("max_batched_tokens", a.max_batched_tokens), ("max_num_seqs", a.max_num_seqs),
                     ("max_model_len", a.max_model_len), ("kv_cache_tokens", a.kv_tokens), ("kv_cache_mb", a.kv_mb),
                     ("kv_block_size", a.page_size)):
        if val is not None:
            settings[key] = val
    if a.model:
        engine = LLM(a.model, **settings)
    else:
        if a.config:
            with open(a.config) as f:
                cfg = json.load(f)
        else:
            cfg = dict(dict(architectures=["Qwen3ForCausalLM"], rms_norm_eps=1e-6, max_position_embeddings=40960),
                       **SIZES[a.random_weights])
        if a.layers:
            cfg["num_hidden_layers"] = a.layers
        engine = LLM(None, random_config=cfg, random_seed=a.seed, **settings)
    vocab = engine.model.spec.vocab_size
    rng = random.Random(a.seed)
    lo, hi = parse_len(a.prompt_len)

    def prompt():
        return [rng.randrange(vocab) for _ in range(rng.randint(lo, hi))]

    sp = lambda n: SamplingParams(max_new_tokens=n, temperature=a.temperature, ignore_eos=True)  # noqa: E731
    for _ in range(a.warmup):
        engine.generate([prompt()], sp(min(a.max_new_tokens, 10)))
    before = engine.stats()
    print(f"Running {a.num_prompts} prompt(s), {a.concurrency} at a time, max_new_tokens={a.max_new_tokens}", file=sys.stderr)

    pending = [prompt() for _ in range(a.num_prompts)]
    live, finished = [], []
    start = time.perf_counter()
    while pending or engine.has_work():
        while pending and len(live) < a.concurrency:
            live.append(engine.add_request(pending.pop(0), sp(a.max_new_tokens)))
        for r in engine.step():
            live.remove(r)
            finished.append(r)
    wall = time.perf_counter() - start

    runs = []
    for i, r in enumerate(finished):
        tl, n = r.times, len(r.times.tokens)
        itl = tl.gaps_ms()
        r4 = lambda v, d=4: None if v is None else round(v, d)           # noqa: E731
        runs.append({"prompt_tokens": len(r.prompt_ids), "generated_tokens": n, "latency_s": r4(tl.latency_s()),
                     "ttft_s": r4(tl.ttft_s()), "tpot_ms": r4(tl.tpot_ms(), 3),
                     "itl_ms_max": round(max(itl), 3) if itl else None, "preemptions": r.preemptions, "error": r.error})
        print(f"[{i}] tokens={n} latency={runs[-1]['latency_s']}s TTFT={runs[-1]['ttft_s']}s "
              f"TPOT={runs[-1]['tpot_ms']}ms max gap={runs[-1]['itl_ms_max']}ms")
    after = engine.stats()

    def avg(key):
        vals = [r[key] for r in runs if r.get(key) is not None]
        return round(sum(vals) / len(vals), 3) if vals else None

    total = sum(r["generated_tokens"] for r in runs)
    summary = {"engine": engine.info(), "concurrency": a.concurrency, "num_prompts": a.num_prompts,
               "wall_time_s": round(wall, 3), "throughput_tok_s": round(total / wall, 2),
               "avg_latency_s": avg("latency_s"), "avg_ttft_s": avg("ttft_s"), "avg_tpot_ms": avg("tpot_ms"),
               "max_itl_ms": max((r["itl_ms_max"] for r in runs if r["itl_ms_max"] is not None), default=None)}
    for key in ("steps", "preemptions", "prefill_chunks", "mixed_steps", "graph_replays", "graph_eager_steps"):
        if key in after:
            summary[key] = after[key] - before.get(key, 0)
    dn = after["decode_steps_timed"] - before["decode_steps_timed"]
    on = after["other_steps_timed"] - before["other_steps_timed"]
    if dn:
        summary["decode_step_ms"] = round((after["decode_step_ms_total"] - before["decode_step_ms_total"]) / dn, 3)
    if on:
        summary["prefill_or_mixed_step_ms"] = round((after["other_step_ms_total"] - before["other_step_ms_total"]) / on, 3)
    if a.roofline:
        pk = measured_peaks()
        d_ms = after["decode_step_ms_total"] - before["decode_step_ms_total"]
        o_ms = after["other_step_ms_total"] - before["other_step_ms_total"]
        d_bytes = after["decode_bytes_total"] - before["decode_bytes_total"]
        o_flops = after["other_flops_total"] - before["other_flops_total"]
        summary["peaks"] = pk["source"]
        if d_ms > 0:
            gbs = d_bytes / (d_ms * 1e-3) / 1e9
            summary["decode_achieved_gb_s"] = round(gbs, 1)
            summary["decode_fraction_of_hbm_peak"] = round(gbs / pk["hbm_gbs"], 4)
        if o_ms > 0:
            tf = o_flops / (o_ms * 1e-3) / 1e12
            summary["prefill_or_mixed_achieved_tflop_s"] = round(tf, 1)
            summary["prefill_or_mixed_fraction_of_bf16_peak"] = round(tf / pk["bf16_tflops"], 4)
    print("\n===== Summary =====")
    for k, v in summary.items():
        if k != "engine":
            print(f"{k:>24}: {v}")
    if a.out:
        with open(a.out, "w") as f:
            json.dump({"summary": summary, "runs": runs}, f, indent=2)
    return 0


if __name__ == "__main__":
    sys.exit(main())
