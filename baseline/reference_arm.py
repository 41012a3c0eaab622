#!/usr/bin/env python3
"""The reference arm of bench.py: davidjoyme/mini-inference's own engine, unmodified, on the
benchmark's workload.

The reference is a set of plain scripts (no setup.py / pyproject, so nothing to pip-install):
its checkout is copied to baseline/_ref and put on sys.path, as its own tests and bench
scripts do.  This program
  1. writes a random Qwen3-4B-size model folder (config.json, model.safetensors; the one
     thing it takes from this repository is the folder writer) plus a word-level tokenizer whose
     words "w<i>" map to token id i + 3, as tests/test_batching.py:31-36 of the reference builds one;
  2. configures the reference through its own switches (config.py: MODEL, DEVICE_MAP, DTYPE,
     ENGINE=custom, SCHEDULER=continuous, KV_CACHE=paged, ATTN_BACKEND=triton, CUDA_GRAPHS=1,
     FUSED_PROJ=1, KV_CACHE_TOKENS, MAX_NUM_SEQS, MAX_BATCHED_TOKENS, MAX_MODEL_LEN), the full
     stack of bench/run_engine.py:79-120;
  3. builds engine.custom_engine.CustomEngine and drives it through submit() (its public
     request call): B requests of ~context-length prompts decode together, and the K timed
     steps are read from the engine's own per-token timestamps (Request.token_times, taken
     after each step's device->host read of the sampled tokens), so the number is end to end
     by construction: host text in, host tokens out, every step;
  4. the 2,048-token prompt: first_token_at - first_scheduled of a request that runs alone.

Prints one JSON line on the last line of stdout.  Everything the reference prints goes to stderr.
"""
import argparse
import json
import os
import shutil
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")

QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 2560, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960, "hidden_act": "silu", "attention_bias": False,
}


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


def write_tokenizer(path, vocab):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    words = ["<unk>", "<pad>", "<eos>"] + [f"w{i}" for i in range(vocab - 3)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    # no eos token is declared: with random weights any id may come out, and generation must run its length
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", pad_token="<pad>").save_pretrained(path)


def text_prompt(rng, n, vocab):
    return " ".join(f"w{rng.randrange(vocab - 3)}" for _ in range(n))


def decode_run(engine, rng, batch, ctx, steps, warmup, vocab):
    """B requests decoding together at context ~ctx; K steps between the engine's own timestamps."""
    total = warmup + steps
    prompt_len = ctx - total - batch - 4          # the first requests already decode while the last are prefilled
    reqs = [engine.submit(text_prompt(rng, prompt_len, vocab), max_new_tokens=total + batch + 2) for _ in range(batch)]
    for r in reqs:
        for _ in engine._events(r):
            pass
    if any(r.finish_reason == "error" for r in reqs):
        raise RuntimeError(f"the reference engine failed a request: {engine.last_error}")
    all_in = max(r.token_times[0] for r in reqs)             # from here on every step decodes all B requests
    t = reqs[0].token_times
    first = next(i for i, x in enumerate(t) if x >= all_in)
    a, b = first + warmup, first + warmup + steps
    if b >= len(t):
        raise RuntimeError("the timed steps ran past the first request's tokens")
    ms = (t[b] - t[a]) * 1e3 / steps
    return {"ms": ms, "tok_s": batch * 1e3 / ms, "prompt_len": prompt_len}


def prefill_run(engine, rng, tokens, vocab, reps=5, warmup=2, pause=0.25):
    best = None
    for i in range(warmup + reps):
        if i >= warmup:
            time.sleep(pause)
        r = engine.submit(text_prompt(rng, tokens, vocab), max_new_tokens=1)
        for _ in engine._events(r):
            pass
        if r.finish_reason == "error":
            raise RuntimeError(f"the reference engine failed the prompt: {engine.last_error}")
        ms = (r.first_token_at - r.first_scheduled) * 1e3
        if i >= warmup:
            best = ms if best is None else min(best, ms)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--peak-tflops", type=float, default=None)
    ap.add_argument("--peak-gbs", type=float, default=None)
    args = ap.parse_args()
    if not os.path.isfile(os.path.join(REF, "engine", "custom_engine.py")):
        return unavailable(f"no copy of the reference under baseline/_ref (expected {REF}/engine/custom_engine.py)")
    real_stdout = os.dup(1)
    os.dup2(2, 1)                                   # the reference prints its progress on stdout: send it to stderr
    out = None
    tmp = tempfile.mkdtemp(prefix="ref_model_")
    try:
        try:
            import torch
            import transformers  # noqa: F401
            import triton  # noqa: F401
            import tokenizers  # noqa: F401
        except Exception as e:
            out = {"impl": "reference", "unavailable": f"import failed on this box: {type(e).__name__}: {e}"}
            raise SystemExit
        if not torch.cuda.is_available():
            out = {"impl": "reference", "unavailable": "no CUDA device"}
            raise SystemExit
        cfg = dict(QWEN3_4B, num_hidden_layers=args.layers)
        vocab = cfg["vocab_size"]
        sys.path.insert(0, ROOT)
        from mini_inference_b200.weights import write_random_model      # the folder writer only
        t0 = time.perf_counter()
        write_random_model(cfg, tmp, seed=0, std=0.02, norm_init="ones", store_dtype="bfloat16", device="cuda:0")
        with open(os.path.join(tmp, "config.json")) as f:
            saved = json.load(f)
        saved.update(model_type="qwen3", hidden_act="silu", attention_bias=False)
        with open(os.path.join(tmp, "config.json"), "w") as f:
            json.dump(saved, f)
        write_tokenizer(tmp, vocab)
        print(f"model folder written in {time.perf_counter() - t0:.1f} s", file=sys.stderr)
        sys.path.remove(ROOT)
        for name in [m for m in sys.modules if m.split(".")[0] == "mini_inference_b200"]:
            del sys.modules[name]                    # nothing of this repository stays importable past this point

        os.environ.update({
            "HF_HUB_OFFLINE": "1", "TRANSFORMERS_OFFLINE": "1", "MODEL": tmp, "ENGINE": "custom", "SCHEDULER": "continuous",
            "KV_CACHE": "paged", "KV_BLOCK_SIZE": "16", "ATTN_BACKEND": "triton", "CUDA_GRAPHS": "1", "FUSED_PROJ": "1",
            "WEIGHT_LAYOUT": "auto", "TUNING_CACHE": "", "MAX_MODEL_LEN": str(args.ctx), "MAX_NUM_SEQS": str(max(64, args.batch)),
            "MAX_BATCHED_TOKENS": "4096", "KV_CACHE_TOKENS": str(max(64, args.batch) * args.ctx + 4096), "KV_WATERMARK": "0.0",
        })
        os.chdir(tmp)
        sys.path.insert(0, REF)
        import config
        config.DEVICE_MAP = os.environ.get("REF_DEVICE_MAP") or None       # "auto" needs accelerate, which is not installed
        config.IS_CHAT_MODEL = False
        config.DO_SAMPLE = False
        config.QUIET_TRANSFORMERS = True
        from engine.custom_engine import CustomEngine
        import random
        rng = random.Random(0)
        engine = CustomEngine()
        if engine.device.type != "cuda":
            out = {"impl": "reference", "unavailable": f"the reference's loader left the model on {engine.device} "
                                                       "(device_map needs accelerate, which is not installed)"}
            raise SystemExit
        info = engine.engine_config()
        pre_ms = prefill_run(engine, rng, 2048, vocab)
        main_run = decode_run(engine, rng, args.batch, args.ctx, args.steps, args.warmup, vocab)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                points[f"decode_b{b}"] = round(decode_run(engine, rng, b, args.ctx, max(16, args.steps // 4),
                                                          args.warmup, vocab)["tok_s"], 1)
        h, H, KV, D, I, L = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                             cfg["intermediate_size"], args.layers)
        gemm = L * (h * (H + 2 * KV) * D + H * D * h + 3 * h * I)
        wbytes = 2 * (gemm + L * (2 * h + 2 * D) + vocab * h + h)
        T = 2048
        pre_flops = 2 * T * gemm + 2 * vocab * h + L * 4 * H * D * T * (T + 1) / 2
        step_bytes = wbytes + args.batch * (args.ctx - args.steps / 2 - 8) * 2 * L * KV * D * 2
        out = {
            "impl": "reference",
            "metric": "Qwen3-4B decode tok/s at batch 8, context 4096 (prefill tok/s at 2,048 tokens in 'prefill')",
            "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: random weights (seeded), uniform-random token ids as words of a word-level tokenizer",
            "config": {"model": "Qwen3-4B-size", "layers": L, "model_layers": 36, "hidden": h, "q_heads": H, "kv_heads": KV,
                       "head_dim": D, "intermediate": I, "vocab": vocab, "tied": True, "global_batch": args.batch,
                       "seq_len": args.ctx, "page_size": 16, "parallelism": "single GPU",
                       "cuda_graphs": bool(info.get("cuda_graphs")), "attn_backend": info.get("attn_backend"),
                       "fused_proj": bool(info.get("fused_proj")), "timing": "the engine's own per-token wall-clock timestamps",
                       "l2": "inputs larger than L2 (8 GB weights + cache)"},
            "e2e": {"value": round(main_run["tok_s"], 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": None, "d2h_bytes_per_step": 4 * args.batch},
            "prefill": {"value": round(T / (pre_ms * 1e-3), 1), "tokens": T, "ms": round(pre_ms, 3)},
            "points": points,
        }
        if args.peak_tflops:
            out["prefill"]["frac"] = round(pre_flops / (pre_ms * 1e-3) / (args.peak_tflops * 1e12), 4)
        if args.peak_gbs:
            ach = step_bytes / (main_run["ms"] * 1e-3) / 1e9
            out["roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": args.peak_gbs, "unit": "GB/s",
                               "frac": round(ach / args.peak_gbs, 4)}
    except SystemExit:
        pass
    except BaseException as e:                       # noqa: BLE001 - whatever the reference raises is the reason
        import traceback
        traceback.print_exc(file=sys.stderr)
        out = {"impl": "reference", "unavailable": f"the reference raised {type(e).__name__}: {' '.join(str(e).split())[:300]}"}
    finally:
        os.chdir(ROOT)
        shutil.rmtree(tmp, ignore_errors=True)
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
    print(json.dumps(out))
    sys.stdout.flush()
    os._exit(0)                                      # the reference's engine loop is a daemon thread that never ends


if __name__ == "__main__":
    sys.exit(main())
