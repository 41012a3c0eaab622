"""Run the engine directly from the command line, in the manner of the reference's
bench/run_engine.py (flags :31-77, summary :164-203): N prompts, C at a time, through the
Python entry point; prints per-request timings and a summary, optionally writes JSON.

Option names and meanings follow the reference where it has them (-n/--num-prompts,
-c/--concurrency, --warmup, --max-new-tokens, --cuda-graphs, --chunked-prefill,
--max-batched-tokens, --kv-tokens, --model, --out).  Prompts are seeded random token ids of
--prompt-len tokens (this engine has no tokenizer; the reference's --prompt/--prompt-words
build text).  --model is a model folder; --random-weights SIZE draws weights on the device."""
from __future__ import annotations

import argparse
import json
import random
import sys
import time

SIZES = {
    "tiny": dict(hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                 intermediate_size=128, vocab_size=256, rope_theta=10000.0, tie_word_embeddings=True),
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
    if (a.model is None) == (a.random_weights is None):
        p.error("give exactly one of --model DIR and --random-weights SIZE")

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
        cfg = dict(SIZES[a.random_weights], architectures=["Qwen3ForCausalLM"], rms_norm_eps=1e-6,
                   max_position_embeddings=40960)
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
        t, n = r.token_times, len(r.token_times)
        itl = [round((y - x) * 1e3, 3) for x, y in zip(t, t[1:])]
        runs.append({"generated_tokens": n, "latency_s": round(r.finished_at - r.arrived, 4),
                     "ttft_s": round(t[0] - r.arrived, 4) if t else None,
                     "tpot_ms": round((t[-1] - t[0]) / (n - 1) * 1e3, 3) if n > 1 else None,
                     "itl_ms_max": max(itl) if itl else None, "preemptions": r.preemptions, "error": r.error})
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
