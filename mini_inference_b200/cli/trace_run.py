"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same
model, step function, cache manager and kernels that generation uses.  The reference has no
program of this kind; its nearest relative is the forced-token loop of
tests/test_kv_features.py:62-89 (admit, ensure, forward one chunk, advance).

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input: one JSON object a line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, OUT/<step>.f32 receives the logits at the wanted
places (order of the entries, then of `want`) as little-endian float32 [wanted, vocab].
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    ap.add_argument("--max-live", type=int, default=8, help="state slots: most requests live at a time")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.page_size <= 0 or 64 % args.page_size:
        ap.error("--page-size must divide 64")

    import numpy as np
    import torch

    from ..engine.batch import StepEntry
    from ..engine.factory import load_model, make_runner

    os.makedirs(args.out, exist_ok=True)
    print(f"[trace_run] loading {args.model} ({args.dtype})", file=sys.stderr, flush=True)
    _, model, _ = load_model(args.model, args.dtype, args.device)
    num_pages = max(1, -(-args.max_tokens // args.page_size))
    runner = make_runner(model, args.page_size, num_pages, args.max_live,
                         max_seq_len=min(model.spec.max_position, num_pages * args.page_size))
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in live:
                seq = runner.cache.admit(rid)
                if seq is None:
                    raise RuntimeError(f"step {step}: more than {args.max_live} live requests")
                live[rid] = seq
            if e["tokens"]:
                entries.append(StepEntry(live[rid], e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.step(entries)
            if logits is not None:
                arr = logits.float().cpu().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                np.ascontiguousarray(arr).tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            elif args.device.startswith("cuda"):
                torch.cuda.synchronize()
        for rid in rec.get("end", []):
            seq = live.pop(rid, None)
            if seq is not None:
                runner.cache.free(seq)
        print(f"done {step}", flush=True)
    if hasattr(runner.ops, "check_errors"):
        runner.ops.check_errors()
    return 0


if __name__ == "__main__":
    sys.exit(main())
