"""Interfaces and registries of the parts a decoder layer is assembled from.

A part (mixer, feed-forward, norm, position encoding, block arrangement) is a class
registered under a name.  It is built from its own PartSpec (sizes and constants), names
the tensors it needs in its own terms, and computes through the kernel namespace handed to
it in the StepContext.  It never sees the model's configuration or its neighbours' specs.

Interfaces
  every part   __init__(spec)            sizes/constants from spec only
               weight_specs()            -> [WeightSpec] (part-local names)
               load(tensors, dtype, device)   takes its tensors (part-local names), may fuse them
  Norm         forward(x, delta, ctx, rows=None) -> y
                   delta is added to x first (in place when rows is None); rows selects
                   the rows to normalise (then x is left untouched)
  Position     rotary_inv_freq() -> float32 [D/2] tensor or None
               on_embedding(x, ctx) -> x       (absolute encodings add here; default: identity)
                   may own tensors like any part (weight names under "position.<name>" of the first layer using it)
  FeedForward  forward(h, ctx) -> [T, hidden]
  Mixer        cache_need() -> KVCacheNeed | StateNeed | None
               forward(h, ctx, cache, position, owns_cache) -> [T, hidden]
                   cache is the LayerCache of the execution step (or of the step it reads)
  Block        __init__(spec, mixer, feed_forward, norm1, norm2, position)
               forward(x, delta, ctx, cache, owns_cache) -> (x, delta)
                   x is the residual stream, delta an addition not yet applied to it

Optional fast-path protocol (a block may use what its parts offer; none has to):
  Mixer        forward_open(h, ctx, cache, position, owns_cache) -> (rows, out_weight)
                   forward() without its last product: forward == linear(rows, out_weight); open_weight names that tensor
  FeedForward  forward_open(h, ctx) -> (rows, out_weight)      the same
  Norm         accepts_deferred = True   when forward hands `delta` to ctx.ops.add_rmsnorm untouched: the block may then
                   give it the result of ctx.ops.linear(..., defer=True) (possibly partial sums the kernel adds up)
               rms_params() -> (weight, eps)   when forward is the plain RMS norm
  FeedForward  gated_weights() -> (gate_up [2I, hidden], down [hidden, I])
                   when forward == linear(silu(g) * u, down) with [g | u] = linear(h, gate_up)
  Mixer, FeedForward   first_weight -> the tensor that forward() reads first
  Norm         takes_next_weight = True   when forward accepts next_weight=<tensor> and passes it to ctx.ops.add_rmsnorm: the
                   block names the first weight of the part that follows the norm, and the kernel may request it into L2
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

from ..config.spec import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    name: str                       # part-local name, e.g. "q_proj"
    shape: Tuple[int, ...]
    kind: str = "matrix"            # "matrix" (GEMM operand) | "vector" | "table" (integers)
    init: str = "normal"            # random-weights mode: "normal" | "norm" | "zeros"
    optional: bool = False


@dataclass(frozen=True)
class KVCacheNeed:
    """Keys and values in pages; window=None keeps every key, W keeps the last W."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state, one slot per live request, zeroed when claimed."""
    shape: Tuple[int, ...]
    dtype: str = "float32"          # "float32" or "compute"


class LayerCache:
    """What one execution step's mixer gets from the cache manager: for pages, the step's key
    and value pools [pages, kv_heads, page_size, head_dim] and the index of the cache group
    whose block tables (ctx.batch.groups[group]) address them; for state, the slot tensor."""
    def __init__(self, group: int, k=None, v=None, state=None):
        self.group, self.k, self.v, self.state = group, k, v, state


class StepContext:
    """What a part sees of the step being run."""
    def __init__(self, ops, batch, dtype, device):
        self.ops, self.batch, self.dtype, self.device = ops, batch, dtype, device
        self.defer_ok = False        # set by the model when every reader of a block's outputs accepts deferred sums
        self.hints_ok = False        # the kernel namespace's add_rmsnorm takes next_weight=


class Part:
    def __init__(self, spec: PartSpec):
        self.spec = spec

    def weight_specs(self):
        return []

    def load(self, tensors, dtype, device):
        pass


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def _register(family: str, name: str):
    def deco(cls):
        _REGISTRIES[family][name] = cls
        return cls
    return deco


def register_mixer(name): return _register("mixer", name)
def register_feed_forward(name): return _register("feed_forward", name)
def register_norm(name): return _register("norm", name)
def register_position(name): return _register("position", name)
def register_block(name): return _register("block", name)


def lookup(family: str, name: str):
    table = _REGISTRIES[family]
    if name not in table:
        raise KeyError(f"no {family} part named '{name}' is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[name]


def build_part(family: str, spec: PartSpec, *args):
    return lookup(family, spec.kind)(spec, *args)
