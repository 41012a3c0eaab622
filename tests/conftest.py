import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Two tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
    "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 512,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 96, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 32, "intermediate_size": 224,
    "vocab_size": 512, "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 1024,
}
# A third one with a window on some layers (two cache groups), odd sizes, one kv head.
TINY_W = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 80, "num_hidden_layers": 3,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48, "intermediate_size": 176,
    "vocab_size": 301, "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 512, "use_sliding_window": True, "sliding_window": 11,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention"],
}
# A fourth one whose head size (64) and page size (16) reach the tensor-core attention kernels.
TINY_F = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 200,
    "vocab_size": 333, "rope_theta": 300000.0, "rms_norm_eps": 2e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 2048,
}
# A fifth one: windowed layers whose head size (64), page size (16) and group of 3 reach the tensor-core attention
# kernels through the cache manager, with a window (40) that ends inside a 64-key tile and pages that are given back.
TINY_V = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 192, "num_hidden_layers": 2,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 264,
    "vocab_size": 411, "rope_theta": 20000.0, "rms_norm_eps": 4e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 2048, "use_sliding_window": True, "sliding_window": 40,
    "layer_types": ["sliding_attention", "full_attention"],
}
TINY = {"V": (TINY_V, dict(seed=5, std=0.07), 16), "F": (TINY_F, dict(seed=4, std=0.06), 16), "A": (TINY_A, dict(seed=0, std=0.02), 8), "B": (TINY_B, dict(seed=1, std=0.05), 4),
        "W": (TINY_W, dict(seed=2, std=0.08), 4)}


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """name -> (model folder, config dict, page size); folders live in a temporary place."""
    from mini_inference_b200.weights import write_random_model
    out = {}
    for name, (cfg, kw, page) in TINY.items():
        d = str(tmp_path_factory.mktemp(f"tiny{name}"))
        write_random_model(cfg, d, norm_init="uniform", store_dtype="bfloat16", **kw)
        out[name] = (d, cfg, page)
    return out
