"""Architecture-neutral description of a decoder: which parts make each layer, with which
constants, and in which order the layers run.

A model family (models/qwen3.py) turns its typed configuration into a ModelSpec; the
generic decoder (parts/model.py) builds itself from the spec alone.  Nothing in a spec
names a model family, and no part receives more than its own PartSpec.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


def _freeze(value):
    if isinstance(value, Mapping):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    if isinstance(value, (list, tuple)):
        return tuple(_freeze(v) for v in value)
    return value


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name from its registry, with its sizes and constants."""
    kind: str
    params: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def of(kind: str, **params) -> "PartSpec":
        return PartSpec(kind, _freeze(params))

    def get(self, key, default=None):
        return dict(self.params).get(key, default)

    def as_dict(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (block) and the parts it arranges, by ROLE.  Which roles exist
    is the block's business: the pre-norm block takes "mixer", "feed_forward", "norm1", "norm2"
    and "position"; a block with one shared norm, or with four, names its own.  weight_names
    maps each part's tensor names, prefixed by its role ("mixer.q_proj", "norm1.weight", ...),
    to the checkpoint's names, so that no part knows a checkpoint's naming."""
    block: str
    parts: Tuple[Tuple[str, PartSpec], ...]
    weight_names: Tuple[Tuple[str, str], ...]

    @staticmethod
    def of(block: str, weight_names, **parts: PartSpec) -> "LayerSpec":
        names = weight_names.items() if isinstance(weight_names, Mapping) else weight_names
        return LayerSpec(block, tuple(parts.items()), tuple(sorted(names)))

    def part(self, role: str) -> PartSpec:
        return dict(self.parts)[role]

    def checkpoint_name(self, part_tensor: str) -> str:
        return dict(self.weight_names)[part_tensor]


@dataclass(frozen=True)
class ExecStep:
    """One entry of the execution order.  layer indexes ModelSpec.layers (a layer may be named
    by several steps: shared weights, separate caches).  cache_from names an EARLIER step whose
    cache this step's mixer reads instead of owning one."""
    layer: int
    cache_from: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[ExecStep, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_name: str
    lm_head_name: Optional[str]          # None: the head is the embedding matrix (tied)
    max_position: int
    eos_token_ids: Tuple[int, ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = field(default=())

    def __post_init__(self):
        for i, step in enumerate(self.order):
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {step.layer}; the model has {len(self.layers)}")
            if step.cache_from is not None:
                if not 0 <= step.cache_from < i:
                    raise ValueError(f"order[{i}] reads the cache of step {step.cache_from}, which does not run before it")
                if self.order[step.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}] reads the cache of step {step.cache_from}, which owns none")
