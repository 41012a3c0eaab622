"""Engine settings.  The reference keeps them as module globals that environment variables
override (config.py:13-161); here they are one dataclass whose fields keep the reference's
names in lower case and read the same environment variables as defaults."""
from __future__ import annotations

import os
from dataclasses import dataclass, field, fields
from typing import Optional


def _env(name, cast, default):
    raw = os.environ.get(name)
    if raw is None or raw == "":
        return default
    if cast is bool:
        return raw == "1" or raw.lower() in ("true", "on")
    return cast(raw)


@dataclass
class EngineArgs:
    dtype: str = field(default_factory=lambda: _env("DTYPE", str, "bfloat16"))                      # config.py:28
    max_model_len: int = field(default_factory=lambda: _env("MAX_MODEL_LEN", int, 32768))           # config.py:18
    kv_block_size: int = field(default_factory=lambda: _env("KV_BLOCK_SIZE", int, 16))              # config.py:84
    kv_watermark: float = field(default_factory=lambda: _env("KV_WATERMARK", float, 0.01))          # config.py:87
    kv_cache_tokens: Optional[int] = field(default_factory=lambda: _env("KV_CACHE_TOKENS", int, None))   # config.py:102
    kv_cache_mb: Optional[float] = field(default_factory=lambda: _env("KV_CACHE_MB", float, None))  # config.py:104
    gpu_memory_utilization: float = field(default_factory=lambda: _env("GPU_MEMORY_UTILIZATION", float, 0.90))  # config.py:105
    activation_reserve_gb: float = 2.0                                                              # config.py:106
    max_num_seqs: int = field(default_factory=lambda: _env("MAX_NUM_SEQS", int, 64))                # config.py:110
    max_batched_tokens: int = field(default_factory=lambda: _env("MAX_BATCHED_TOKENS", int, 4096))  # config.py:111
    chunked_prefill: bool = field(default_factory=lambda: _env("CHUNKED_PREFILL", bool, False))     # config.py:117
    cuda_graphs: bool = field(default_factory=lambda: _env("CUDA_GRAPHS", bool, False))             # config.py:142
    # with CUDA graphs: launch the next decode step (its tokens stay on the device) before the current one's tokens
    # are read, so the host's bookkeeping overlaps the GPU; a request that stops on EOS has run one step in vain
    overlap_decode: bool = field(default_factory=lambda: _env("OVERLAP_DECODE", bool, True))
    max_new_tokens: int = 100                                                                       # config.py:120
    do_sample: bool = False                                                                         # config.py:121
    temperature: float = 0.7                                                                        # config.py:122
    seed: int = 0
    device: str = "cuda:0"
    nvtx: bool = field(default_factory=lambda: _env("NVTX", bool, False))                           # config.py:155

    def __post_init__(self):
        self.dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(self.dtype, self.dtype)
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError(f"dtype '{self.dtype}' is not supported (bfloat16, float32)")
        if self.kv_block_size <= 0 or self.max_num_seqs <= 0 or self.max_batched_tokens <= 0:
            raise ValueError("kv_block_size, max_num_seqs and max_batched_tokens must be positive")

    def asdict(self):
        return {f.name: getattr(self, f.name) for f in fields(self)}
