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
