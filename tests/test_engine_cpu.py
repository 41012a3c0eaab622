"""The engine's batching and cache logic on the CPU: the step function runs with the plain
PyTorch kernel references (tests/ref_ops.py) in place of the CUDA kernels and must agree with
the plain whole-sequence implementation however the tokens are cut."""
import pytest

from tests.helpers import check_cuts, check_mixed, make_engine
from tests.ref_ops import TorchRefOps

TOL = 2e-5


@pytest.mark.parametrize("name", ["A", "B", "W", "V"])
def test_whole_decode_and_portions(tiny_dirs, name):
    d, cfg, page = tiny_dirs[name]
    check_cuts(make_engine(d, page, 64, ops=TorchRefOps()), d, cfg["vocab_size"], TOL)


@pytest.mark.parametrize("name", ["A", "B", "W", "V"])
def test_mixed_batches_reuse_pages(tiny_dirs, name):
    d, cfg, page = tiny_dirs[name]
    check_mixed(lambda pages: make_engine(d, page, pages, ops=TorchRefOps()), d, cfg["vocab_size"], page, TOL)
