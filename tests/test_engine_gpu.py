"""The engine on the GPU with its own kernels, in float32 and in bfloat16, against the plain
implementation: whole prompts, decoding token by token, portions, mixed batches with page
re-use, long decoding."""
import pytest
import torch

from tests.helpers import check_cuts, check_mixed, make_engine, plain_logits, random_tokens, rel_err, run_cuts

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOLS = {"float32": 2e-5, "bfloat16": 4e-2}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_whole_decode_and_portions(tiny_dirs, name, dtype):
    d, cfg, page = tiny_dirs[name]
    check_cuts(make_engine(d, page, 64, dtype=dtype, device=DEV), d, cfg["vocab_size"], TOLS[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "W"])
def test_mixed_batches_reuse_pages(tiny_dirs, name, dtype):
    d, cfg, page = tiny_dirs[name]
    check_mixed(lambda pages: make_engine(d, page, pages, dtype=dtype, device=DEV), d, cfg["vocab_size"], page,
                TOLS[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "W"])
def test_long_decoding(tiny_dirs, name, dtype):
    """A short prompt and 300 tokens one by one: several splits, many pages, window edges."""
    d, cfg, page = tiny_dirs[name]
    ids = random_tokens(cfg["vocab_size"], 310, seed=11)
    want = plain_logits(d, ids)
    runner = make_engine(d, page, 128, dtype=dtype, device=DEV)
    runner.ops.force_splits = 3
    try:
        got = run_cuts(runner, "long", ids, [10] + [1] * 300)
    finally:
        runner.ops.force_splits = None
    assert rel_err(got, want) < TOLS[dtype]
