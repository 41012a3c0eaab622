"""Shared test helpers: build an engine over a model folder, replay token lists through the
step function in different cuts, and compare with the plain implementation."""
import random

import torch

from mini_inference_b200.engine.batch import StepEntry
from mini_inference_b200.engine.factory import load_model, make_runner
from tests.plain import qwen3_plain as plain


def make_engine(model_dir, page_size, num_pages, dtype="float32", device="cpu", ops=None, max_seqs=4,
                max_seq_len=None):
    cfg, model, _ = load_model(model_dir, dtype, device)
    return make_runner(model, page_size, num_pages, max_seqs, max_seq_len=max_seq_len, ops=ops)


def plain_logits(model_dir, token_ids):
    cfg, w = plain.load_model_dir(model_dir, torch.float32)
    return plain.forward_logits(cfg, w, token_ids)


def run_cuts(runner, seq_id, token_ids, cuts):
    """Feed token_ids in portions of the given sizes (all logits wanted); returns [n, vocab]."""
    seq = runner.cache.admit(seq_id)
    out, at = [], 0
    for n in cuts:
        out.append(runner.step([StepEntry(seq, token_ids[at:at + n], range(n))]).float().cpu())
        at += n
    assert at == len(token_ids)
    runner.cache.free(seq)
    return torch.cat(out)


def random_cuts(n, rng, smallest=2, largest=9):
    cuts = []
    while n > 0:
        c = min(n, rng.randint(smallest, largest))
        if n - c == 1:
            c += 1
        cuts.append(c)
        n -= c
    return cuts


def random_tokens(vocab, n, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def rel_err(a, b):
    return ((a - b).abs().max() / b.abs().max().clamp_min(1e-30)).item()


def check_cuts(runner, model_dir, vocab, tol, n=45, seed=5):
    """whole prompt; most in one step + last 32 one by one; portions of changing size."""
    ids = random_tokens(vocab, n, seed=seed)
    want = plain_logits(model_dir, ids)
    pool = runner.cache.free_pages()
    whole = run_cuts(runner, "w", ids, [len(ids)])
    assert rel_err(whole, want) < tol, ("whole", rel_err(whole, want))
    dec = run_cuts(runner, "d", ids, [len(ids) - 32] + [1] * 32)
    assert rel_err(dec, want) < tol, ("decode", rel_err(dec, want))
    por = run_cuts(runner, "p", ids, random_cuts(len(ids), random.Random(1)))
    assert rel_err(por, want) < tol, ("portions", rel_err(por, want))
    first = run_cuts(runner, "f", ids[:3], [1, 1, 1])
    assert rel_err(first, want[:3]) < tol, ("first tokens", rel_err(first, want[:3]))
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == pool


def check_mixed(make, model_dir, vocab, page, tol, lens=(23, 9, 31, 17, 40, 12, 27, 36, 20, 33, 14, 38), seed=7):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool so small that pages are
    used again: it holds four of the longest requests and not a page more, so every page that a finished request gives
    back is handed out again (the pool is first in, first out).  The re-use is counted, not assumed."""
    rng = random.Random(seed)
    reqs = {f"r{i}": random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(lens)}
    want = {k: plain_logits(model_dir, v) for k, v in reqs.items()}
    pages = 4 * -(-max(lens) // page)
    runner = make(pages)
    takes = {}                                             # page id -> how often it was handed out
    for g in runner.cache.kv_groups:
        inner = g.pool.take
        def counted(inner=inner, gi=id(g)):
            pg = inner()
            takes[(gi, pg)] = takes.get((gi, pg), 0) + 1
            return pg
        g.pool.take = counted
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
        logits = runner.step(entries).float().cpu()
        row = 0
        for k, n in owners:
            got[k].append(logits[row:row + n])
            row += n
            live[k][1] += n
        for k in [k for k, (seq, at) in live.items() if at == len(reqs[k])]:
            runner.cache.free(live.pop(k)[0])
        runner.cache.check_invariants()
    for k in reqs:
        e = rel_err(torch.cat(got[k]), want[k])
        assert e < tol, (k, e)
    assert runner.cache.free_pages() == pages
    total, again = sum(takes.values()), sum(n - 1 for n in takes.values())
    assert again * 3 >= total, f"only {again} of {total} page takes were of a page used before"
