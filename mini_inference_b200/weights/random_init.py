"""Random-weights mode: write a model folder (config.json, model.safetensors) from a
configuration and a seed.  The reference builds random models only in its tests
(tests/test_models.py:55-62); here it is a mode of the loader, used by tests and benchmarks.

Each tensor is drawn on the CPU in float32 from a generator seeded by (seed, tensor index),
then stored in the requested dtype, so the same seed gives the same folder everywhere and a
float32 run and a bfloat16 run of one folder hold the same values."""
from __future__ import annotations

import json
import os

import torch

from ..config.registry import resolve
from ..parts.model import DecoderModel
from .safetensors_io import write_safetensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


def _draw(ws, seed: int, index: int, std: float, norm_init: str, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed * 1_000_003 + index)
    if ws.kind == "table":
        return torch.zeros(ws.shape, dtype=torch.int32)
    if ws.init == "norm":
        if norm_init == "ones":
            return torch.ones(ws.shape)
        return torch.rand(ws.shape, generator=g, device=device) + 0.5            # U(0.5, 1.5)
    if ws.init == "zeros":
        return torch.zeros(ws.shape)
    return torch.randn(ws.shape, generator=g, device=device) * std


def write_random_model(config: dict, out_dir: str, seed: int = 0, std: float = 0.02,
                       norm_init: str = "uniform", store_dtype: str = "bfloat16", device="cpu") -> str:
    """config: the config.json dict of a registered architecture.  device: where the values are drawn; the
    default (the CPU) gives the same folder on every machine, a GPU writes a many-gigabyte folder in seconds
    (its values differ from the CPU's for the same seed)."""
    arch = resolve(config)
    cfg = arch.config_class.from_dict(config)
    model = DecoderModel(arch.build_spec(cfg))
    dtype = _STORE[store_dtype]
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg.to_dict() if hasattr(cfg, "to_dict") else config, f, indent=1)
    items, seen = [], set()
    for index, (name, ws) in enumerate(model.weight_table()):
        if name in seen:
            continue
        seen.add(name)
        store = torch.int32 if ws.kind == "table" else dtype
        items.append((name, tuple(ws.shape), store,
                      lambda ws=ws, index=index, store=store: _draw(ws, seed, index, std, norm_init, device).to(store).cpu()))
    write_safetensors(os.path.join(out_dir, "model.safetensors"), items)
    return out_dir


def init_random_on_device(model, dtype: torch.dtype, device, seed: int = 0, std: float = 0.02,
                          norm_init: str = "ones", draw_dtype: torch.dtype = None) -> dict:
    """Random weights drawn directly on the device, tensor by tensor (benchmarks of large
    configurations: no folder is written, nothing passes through host memory)."""
    g = torch.Generator(device=device).manual_seed(seed)
    tensors, nbytes = {}, 0
    for name, ws in model.weight_table():
        if name in tensors:
            continue
        if ws.kind == "table":
            t = torch.zeros(ws.shape, dtype=torch.int32, device=device)
        elif ws.init == "norm":
            t = torch.ones(ws.shape, dtype=dtype, device=device) if norm_init == "ones" else \
                (torch.rand(ws.shape, generator=g, device=device) + 0.5).to(draw_dtype or dtype).to(dtype)
        else:
            t = torch.empty(ws.shape, dtype=draw_dtype or dtype, device=device).normal_(0.0, std, generator=g).to(dtype)
        tensors[name] = t
        nbytes += t.numel() * t.element_size()
    model.load(tensors, dtype, device)
    return {"tensors": len(tensors), "weight_bytes": nbytes}
