"""Reader and writer of the safetensors container (one file or an index of shards).

Layout: 8 bytes little-endian header length, a JSON header {name: {dtype, shape,
data_offsets}}, then the raw little-endian tensor bytes.  Tensors are read lazily through a
memory map, one by one and by name, so a large checkpoint never sits in host memory twice.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        self.header = json.loads(self._f.read(hlen))
        self.header.pop("__metadata__", None)
        self._base = 8 + hlen
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> Iterable[str]:
        return self.header.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        h = self.header[name]
        if h["dtype"] not in _DTYPES:
            raise ValueError(f"{self.path}: tensor {name} has unsupported dtype {h['dtype']}")
        return _DTYPES[h["dtype"]], tuple(h["shape"])

    def get(self, name: str) -> torch.Tensor:
        dtype, shape = self.info(name)
        a, b = self.header[name]["data_offsets"]
        if a == b:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._map)[self._base + a:self._base + b]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)     # read-only buffer: it is cloned at once
            return torch.frombuffer(buf, dtype=dtype).reshape(shape).clone()

    def close(self):
        try:
            self._map.close()
        except BufferError:
            pass
        self._f.close()


def open_model_tensors(model_dir: str) -> Dict[str, SafetensorsFile]:
    """name -> file that holds it, for model.safetensors or a sharded index."""
    single = os.path.join(model_dir, "model.safetensors")
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        return {name: f for name in f.keys()}
    if os.path.isfile(index):
        with open(index) as fh:
            weight_map = json.load(fh)["weight_map"]
        files = {fn: SafetensorsFile(os.path.join(model_dir, fn)) for fn in sorted(set(weight_map.values()))}
        # a name the index sends to a shard that does not hold it counts as missing
        return {name: files[fn] for name, fn in weight_map.items() if name in files[fn].header}
    raise FileNotFoundError(f"{model_dir} has neither model.safetensors nor model.safetensors.index.json")


def write_safetensors(path: str, tensors, order=None) -> None:
    """tensors: dict name -> tensor, or an iterable of (name, shape, dtype, make) with make()
    producing the tensor when its turn comes (bounds host memory for large models)."""
    if isinstance(tensors, dict):
        items = [(k, tuple(v.shape), v.dtype, (lambda v=v: v)) for k, v in tensors.items()]
    else:
        items = list(tensors)
    header, offset = {}, 0
    for name, shape, dtype, _ in items:
        n = 1
        for s in shape:
            n *= s
        size = n * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + size]}
        offset += size
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, shape, dtype, make in items:
            t = make().contiguous()
            assert tuple(t.shape) == tuple(shape) and t.dtype == dtype, name
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
