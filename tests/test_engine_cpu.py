"""The engine's batching and cache logic on the CPU: the step function runs with the plain
PyTorch kernel references (tests/ref_ops.py) in place of the CUDA kernels and must agree with
the plain whole-sequence implementation however the tokens are cut."""
import random

import pytest
import torch

from mini_inference_b200.engine.batch import StepEntry
from tests.helpers import make_engine, plain_logits, random_cuts, random_tokens, rel_err, run_cuts
from tests.ref_ops import TorchRefOps

TOL = 2e-5


@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_whole_decode_and_portions(tiny_dirs, name):
    d, cfg, page = tiny_dirs[name]
    ids = random_tokens(cfg["vocab_size"], 45, seed=5)
    want = plain_logits(d, ids)
    runner = make_engine(d, page, 64, ops=TorchRefOps())
    whole = run_cuts(runner, "w", ids, [len(ids)])
    assert rel_err(whole, want) < TOL
    dec = run_cuts(runner, "d", ids, [len(ids) - 32] + [1] * 32)
    assert rel_err(dec, want) < TOL
    por = run_cuts(runner, "p", ids, random_cuts(len(ids), random.Random(1)))
    assert rel_err(por, want) < TOL
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == 64


@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_mixed_batches_reuse_pages(tiny_dirs, name):
    d, cfg, page = tiny_dirs[name]
    rng = random.Random(7)
    lens = [23, 9, 31, 17, 40, 12, 27]
    reqs = {f"r{i}": random_tokens(cfg["vocab_size"], n, seed=100 + i) for i, n in enumerate(lens)}
    want = {k: plain_logits(d, v) for k, v in reqs.items()}
    pool_tokens = 4 * 48
    runner = make_engine(d, page, pool_tokens // page, ops=TorchRefOps())
    pending = list(reqs)
    live, got = {}, {k: [] for k in reqs}
    while pending or live:
        while pending and len(live) < 4:
            k = pending.pop(0)
            live[k] = [runner.cache.admit(k), 0]
        entries, owners = [], []
        for k, (seq, at) in live.items():
            if rng.random() < 0.2 and len(live) > 1:
                continue                                   # left out of this step
            left = len(reqs[k]) - at
            n = 1 if (at > 0 and rng.random() < 0.5) else min(left, rng.randint(2, 8))
            if left - n == 1:
                n = left
            entries.append(StepEntry(seq, reqs[k][at:at + n], range(n)))
            owners.append((k, n))
        if not entries:
            continue
        logits = runner.step(entries).float()
        row = 0
        for k, n in owners:
            got[k].append(logits[row:row + n])
            row += n
            live[k][1] += n
        for k in [k for k, (seq, at) in live.items() if at == len(reqs[k])]:
            runner.cache.free(live.pop(k)[0])
        runner.cache.check_invariants()
    for k in reqs:
        assert rel_err(torch.cat(got[k]), want[k]) < TOL, k
    assert runner.cache.free_pages() == pool_tokens // page
