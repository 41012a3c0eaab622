"""Makes tests/golden/*.npz: logits of the REFERENCE's own runner on tiny random Qwen3 models.

The reference (davidjoyme/mini-inference) does not own the model: its ModelRunner drives the
sub-modules of a `transformers` model (engine/core/model_runner.py:86-88).  This script writes
this repo's seeded random-weights folders for the tiny configurations, loads each with
`transformers` exactly as the reference's loader would (float32, CPU), runs the reference's
ModelRunner + paged KVCache over a fixed token list (whole, and in 4-token portions) and stores
the logits.  tests/test_golden.py then checks the plain implementation under tests/plain/
against these files; nothing here is imported by the package or by the other tests.

Run once, on the CPU, with the reference checkout and `transformers` available:
    python tests/golden/make_golden.py /path/to/mini-inference
"""
import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from mini_inference_b200.weights import write_random_model  # noqa: E402
from tests.conftest import TINY  # noqa: E402
from tests.helpers import random_tokens  # noqa: E402


def main(reference_dir):
    os.environ["HF_HUB_OFFLINE"] = "1"
    sys.path.insert(0, reference_dir)
    import config
    config.DEVICE_MAP = None
    from engine.core.kv_cache import KVCache
    from engine.core.model_runner import ModelRunner
    from engine.core.request import Request, SamplingParams
    from transformers import AutoModelForCausalLM

    for name in ("A", "B"):                       # the reference refuses windowed layers (engine/models.py:17-22)
        cfg, kw, page = TINY[name]
        with tempfile.TemporaryDirectory() as d:
            write_random_model(cfg, d, norm_init="uniform", store_dtype="bfloat16", **kw)
            model = AutoModelForCausalLM.from_pretrained(d, dtype=torch.float32).eval()
        ids = random_tokens(cfg["vocab_size"], 23, seed=77)
        L, KV, D = cfg["num_hidden_layers"], cfg["num_key_value_heads"], cfg["head_dim"]
        cache = KVCache("paged", L, KV, D, 64, torch.float32, "cpu", block_size=page)
        runner = ModelRunner(model, cache)
        req = Request(prompt_ids=list(ids), params=SamplingParams(max_new_tokens=1))
        cache.admit(req, 256)
        cache.ensure(req, len(ids))
        whole = runner.forward([(req, 0, len(ids))], all_logits=True)
        cache.free(req)
        req = Request(prompt_ids=list(ids), params=SamplingParams(max_new_tokens=1))
        cache.admit(req, 256)
        parts = []
        for s in range(0, len(ids), 4):
            e = min(s + 4, len(ids))
            cache.ensure(req, e)
            parts.append(runner.forward([(req, s, e)], all_logits=True))
            req.num_computed = e
        chunked = torch.cat(parts)
        out = os.path.join(HERE, f"qwen3_tiny_{name}.npz")
        np.savez_compressed(out, token_ids=np.asarray(ids, dtype=np.int32), whole=whole.numpy().astype(np.float32),
                            chunked=chunked.numpy().astype(np.float32))
        print(name, "whole vs chunked", (whole - chunked).abs().max().item(), "->", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py PATH_TO_A_CHECKOUT_OF_davidjoyme/mini-inference")
    main(sys.argv[1])
