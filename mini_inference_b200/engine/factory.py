"""From a model folder to a loaded model, its cache and its runner."""
from __future__ import annotations

import torch

from ..cache.manager import CacheManager
from ..config.registry import load_config
from ..parts.model import DecoderModel
from ..weights.store import load_into
from .runner import ModelRunner

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0"):
    """The model class is chosen by config.json (config/registry.py)."""
    dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
    cfg, spec = load_config(model_dir)
    model = DecoderModel(spec)
    info = load_into(model, model_dir, dtype, device)
    return cfg, model, info


def make_runner(model: DecoderModel, page_size: int, num_pages: int, max_seqs: int,
                max_seq_len: int = None, watermark: float = 0.0, ops=None) -> ModelRunner:
    max_seq_len = max_seq_len or min(model.spec.max_position, num_pages * page_size)
    cache = CacheManager(model.cache_needs(), page_size, num_pages, max_seqs, max_seq_len,
                         dtype=model.dtype, device=model.device, watermark=watermark)
    return ModelRunner(model, cache, ops)
