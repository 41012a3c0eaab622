"""Typed Qwen3-dense configuration, read from the architecture's own config.json keys.

The reference keeps no typed configuration: it reads the loaded model's config object
with getattr fall-backs (engine/core/model_runner.py:76-80, engine/models.py:9-36).  The
same keys, fall-backs and refusals are made explicit here; every size the model uses comes
from this object.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Optional, Tuple


class ConfigError(ValueError):
    pass


_REQUIRED = ("hidden_size", "num_hidden_layers", "num_attention_heads", "intermediate_size", "vocab_size")


@dataclass(frozen=True)
class Qwen3Config:
    architecture: str
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    layer_windows: Tuple[Optional[int], ...]      # per layer: None = all keys, W = last W keys
    eos_token_ids: Tuple[int, ...] = ()

    # ---------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if raw.get(k) is None]
        if missing:
            raise ConfigError(f"config.json lacks {', '.join(missing)}")
        archs = raw.get("architectures") or ["Qwen3ForCausalLM"]
        H = int(raw["num_attention_heads"])
        hidden = int(raw["hidden_size"])
        # engine/core/model_runner.py:78-79: kv heads default to the query heads,
        # head_dim to hidden/heads; head_dim is otherwise free of both.
        KV = int(raw.get("num_key_value_heads") or H)
        D = int(raw.get("head_dim") or hidden // H)
        if H % KV:
            raise ConfigError(f"num_attention_heads {H} is not a multiple of num_key_value_heads {KV}")
        if D % 2:
            raise ConfigError(f"head_dim {D} is odd; rotate-half position encoding needs an even size")

        rope = raw.get("rope_parameters") or raw.get("rope_scaling") or {}
        theta = raw.get("rope_theta", rope.get("rope_theta"))
        if theta is None:
            raise ConfigError("config.json gives no rope_theta (neither at top level nor in rope_parameters)")
        kind = rope.get("rope_type", rope.get("type", "default"))
        if kind not in (None, "default"):
            raise ConfigError(f"rope_type '{kind}' is not supported (only the default rotary encoding)")
        if raw.get("attention_bias"):
            raise ConfigError("attention_bias=true is not supported (Qwen3 dense has no projection biases)")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act '{act}' is not supported (Qwen3 dense uses silu)")

        L = int(raw["num_hidden_layers"])
        windows = _layer_windows(raw, L)

        eos = raw.get("eos_token_id")
        eos = tuple(eos) if isinstance(eos, (list, tuple)) else (() if eos is None else (int(eos),))
        return cls(
            architecture=archs[0], hidden_size=hidden, num_hidden_layers=L,
            num_attention_heads=H, num_key_value_heads=KV, head_dim=D,
            intermediate_size=int(raw["intermediate_size"]), vocab_size=int(raw["vocab_size"]),
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)), rope_theta=float(theta),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=int(raw.get("max_position_embeddings", 32768)),
            layer_windows=windows, eos_token_ids=eos)

    @classmethod
    def from_dir(cls, model_dir: str) -> "Qwen3Config":
        return cls.from_dict(read_config_json(model_dir))

    # ---------------------------------------------------------------- writing
    def to_dict(self) -> dict:
        """The config.json form (what a model folder holds)."""
        d = {
            "architectures": [self.architecture], "model_type": "qwen3",
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "rope_parameters": {"rope_theta": self.rope_theta, "rope_type": "default"},
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_act": "silu", "attention_bias": False,
        }
        if any(w is not None for w in self.layer_windows):
            d["use_sliding_window"] = True
            d["sliding_window"] = next(w for w in self.layer_windows if w is not None)
            d["layer_types"] = ["sliding_attention" if w is not None else "full_attention"
                                for w in self.layer_windows]
        else:
            d["use_sliding_window"] = False
            d["sliding_window"] = None
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    def describe(self) -> dict:
        """The facts the reference's describe() returns (engine/models.py:35-36)."""
        return {"architecture": self.architecture, "qk_norm": "per_head", "moe": False,
                "heads": self.num_attention_heads, "kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim}

    def asdict(self) -> dict:
        return asdict(self)


def _layer_windows(raw: dict, L: int) -> Tuple[Optional[int], ...]:
    """Per-layer window from layer_types / sliding_window / use_sliding_window /
    max_window_layers.  The reference refuses any windowed layer because its cache cannot
    drop keys (engine/models.py:17-22); here a windowed layer gets a cache group of its own."""
    W = raw.get("sliding_window")
    types = raw.get("layer_types")
    if types:
        if len(types) != L:
            raise ConfigError(f"layer_types has {len(types)} entries for {L} layers")
        for t in types:
            if t not in ("full_attention", "sliding_attention"):
                raise ConfigError(f"layer type '{t}' is not supported (full_attention, sliding_attention)")
        if any(t == "sliding_attention" for t in types) and not W:
            raise ConfigError("layer_types names sliding_attention but sliding_window is not set")
        return tuple(int(W) if t == "sliding_attention" else None for t in types)
    if raw.get("use_sliding_window") and W:
        first = int(raw.get("max_window_layers", L))
        return tuple(int(W) if i >= first else None for i in range(L))
    return (None,) * L


def read_config_json(model_dir: str) -> dict:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir} has no config.json")
    with open(path) as f:
        return json.load(f)
