"""bin/trace_run against the plain implementation: the same requests whole, with the last 32
tokens decoded one by one, in portions of changing size, and mixed with other requests so
that pages are used again.  On the CPU the program runs in-process with the plain kernel
references standing in for the CUDA kernels; on the GPU it runs as the executable."""
import io
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.conftest import ROOT
from tests.helpers import plain_logits, random_cuts, random_tokens


def traces(vocab, seed=3):
    """name -> (steps, expectations); expectations: step -> [(request, position), ...]."""
    rng = random.Random(seed)
    reqs = {f"q{i}": random_tokens(vocab, n, seed=50 + i) for i, n in enumerate([61, 40, 35, 52, 33, 47])}
    out = {}

    def single(cutter):
        steps, expect, step = [], {}, 0
        for rid, ids in reqs.items():
            at = 0
            for n in cutter(len(ids)):
                want = list(range(n))
                steps.append({"step": step, "entries": [{"id": rid, "tokens": ids[at:at + n], "want": want}],
                              "end": [rid] if at + n == len(ids) else []})
                expect[step] = [(rid, at + w) for w in want]
                at += n
                step += 1
        return steps, expect

    out["whole"] = single(lambda n: [n])
    out["decode"] = single(lambda n: [n - 32] + [1] * 32)
    out["portions"] = single(lambda n: random_cuts(n, rng))

    steps, expect, step = [], {}, 0
    pending, live = list(reqs), {}
    while pending or live:
        while pending and len(live) < 4:
            live[pending.pop(0)] = 0
        entries, exp, ended = [], [], []
        for rid, at in list(live.items()):
            if rng.random() < 0.25 and len(live) > 1:
                continue
            left = len(reqs[rid]) - at
            n = 1 if (at > 0 and rng.random() < 0.5) else min(left, rng.randint(2, 9))
            if left - n == 1:
                n = left
            want = [w for w in range(n) if rng.random() < 0.7]
            entries.append({"id": rid, "tokens": reqs[rid][at:at + n], "want": want})
            exp += [(rid, at + w) for w in want]
            live[rid] = at + n
            if at + n == len(reqs[rid]):
                ended.append(rid)
                del live[rid]
        steps.append({"step": step, "entries": entries, "end": ended})
        if exp:
            expect[step] = exp
        step += 1
    out["mixed"] = (steps, expect)
    return reqs, out


def check_outputs(out_dir, model_dir, reqs, expect, vocab, tol):
    want = {rid: plain_logits(model_dir, ids) for rid, ids in reqs.items()}
    files = {f for f in os.listdir(out_dir) if f.endswith(".f32")}
    assert files == {f"{s}.f32" for s in expect}
    worst = 0.0
    for step, rows in expect.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out_dir, f"{step}.f32"), dtype="<f4").reshape(len(rows), vocab))
        ref = torch.stack([want[rid][pos] for rid, pos in rows])
        worst = max(worst, ((got - ref).abs().max() / ref.abs().max()).item())
    assert worst < tol, worst


MAX_TOKENS = 4 * 64          # four live requests of at most 64 tokens: pages are used again


@pytest.mark.parametrize("name", ["A", "B", "W"])
@pytest.mark.parametrize("way", ["whole", "decode", "portions", "mixed"])
def test_trace_run_cpu(tiny_dirs, tmp_path, monkeypatch, capsys, name, way):
    from mini_inference_b200 import ops
    from mini_inference_b200.cli import trace_run
    from tests.ref_ops import TorchRefOps
    d, cfg, _ = tiny_dirs[name]
    reqs, tr = traces(cfg["vocab_size"])
    steps, expect = tr[way]
    monkeypatch.setattr(ops, "get_ops", lambda device: TorchRefOps())
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    rc = trace_run.main(["--model", d, "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", str(MAX_TOKENS),
                         "--device", "cpu"])
    assert rc == 0
    assert capsys.readouterr().out.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
    check_outputs(str(tmp_path), d, reqs, expect, cfg["vocab_size"], 2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 4e-2)])
@pytest.mark.parametrize("name", ["A", "B", "W", "F"])
def test_trace_run_gpu(tiny_dirs, tmp_path, name, dtype, tol):
    d, cfg, _ = tiny_dirs[name]
    reqs, tr = traces(cfg["vocab_size"])
    for way, (steps, expect) in tr.items():
        out = tmp_path / way
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                            "--max-tokens", str(MAX_TOKENS)],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert r.stdout.split("\n")[:-1] == [f"done {s['step']}" for s in steps]
        check_outputs(str(out), d, reqs, expect, cfg["vocab_size"], tol)
