"""The plain implementation against the reference's own runner, once, on tiny random models:
tests/golden/*.npz hold the logits the reference produced (made by tests/golden/make_golden.py
from the same seeded weights)."""
import os

import numpy as np
import pytest
import torch

from tests.helpers import plain_logits

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_reference_runner(tiny_dirs, name):
    path = os.path.join(HERE, "golden", f"qwen3_tiny_{name}.npz")
    gold = np.load(path)
    d, cfg, _ = tiny_dirs[name]
    got = plain_logits(d, gold["token_ids"].tolist())
    for key in ("whole", "chunked"):
        ref = torch.from_numpy(gold[key])
        assert ((got - ref).abs().max() / ref.abs().max()).item() < 1e-5, key
