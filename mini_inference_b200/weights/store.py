"""Weights by tensor name, from a model folder into the model.

The reference hands loading to the library pipeline (engine/model_loader.py:28-33) and
fuses q/k/v and gate/up afterwards (engine/core/fused_linear.py:189-208).  Here the model
says which tensors it needs (DecoderModel.weight_table), this module reads exactly those by
name and reports everything that does not fit in ONE error; the parts fuse what they own.

Runtime dtype of a tensor:
  float32 run    every floating tensor is float32.
  bfloat16 run   16-bit tensors stay/become bfloat16; a tensor STORED in 32 bits stays in
                 32 bits unless it is a GEMM operand ("matrix"), which the tensor-core
                 kernels need in bfloat16; integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .safetensors_io import open_model_tensors


class WeightError(ValueError):
    """Missing tensors, unexpected tensors and wrong shapes of one checkpoint, all at once."""
    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = ["checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, got in self.wrong_dtype:
            lines.append(f"  wrong dtype: {name} is {got}, expected a floating type")
        super().__init__("\n".join(lines))


def runtime_dtype(stored: torch.dtype, kind: str, compute: torch.dtype) -> torch.dtype:
    if kind == "table":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64) and kind != "matrix":
        return torch.float32
    return torch.bfloat16


def check_names(table, files: Dict[str, object], ignorable=()):
    """Compare the model's tensor table with the checkpoint's header only (no data read)."""
    wanted = {name: ws for name, ws in table}
    missing = [n for n, ws in table if n not in files and not ws.optional]
    unexpected = sorted(n for n in files if n not in wanted and n not in ignorable)
    wrong_shape, wrong_dtype = [], []
    for name, ws in table:
        if name in files:
            dtype, shape = files[name].info(name)
            if tuple(shape) != tuple(ws.shape):
                wrong_shape.append((name, shape, ws.shape))
            if ws.kind != "table" and not dtype.is_floating_point:
                wrong_dtype.append((name, dtype))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype)


def load_into(model, model_dir: str, dtype: torch.dtype, device) -> dict:
    """Read the tensors of model.weight_table() from model_dir and hand them to the model."""
    files = open_model_tensors(model_dir)
    table = model.weight_table()
    try:
        check_names(table, files, model.ignorable_names())
        tensors, nbytes = {}, 0
        for name, ws in table:
            if name in tensors or name not in files:
                continue
            t = files[name].get(name)
            t = t.to(device=device, dtype=runtime_dtype(t.dtype, ws.kind, dtype))
            tensors[name] = t
            nbytes += t.numel() * t.element_size()
    finally:
        for f in {id(f): f for f in files.values()}.values():
            f.close()
    model.load(tensors, dtype, device)
    return {"tensors": len(tensors), "weight_bytes": nbytes}
