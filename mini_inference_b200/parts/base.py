"""Interfaces and registries of the parts a decoder layer is assembled from.

A part (mixer, feed-forward, norm, position encoding, block arrangement) is a class
registered under a name in the registry of its family.  It is built from its own PartSpec
(sizes and constants), names the tensors it needs in its own terms, and computes through the
kernel namespace handed to it in the StepContext.  It never sees the model's configuration
or its neighbours' specs.

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
  Block        roles = {role: family}    the parts it arranges; the model builds one part per role from
                                         LayerSpec.parts and hands them over as a dict
               __init__(spec, parts)
               mixer                     the part whose cache_need() the cache manager serves
               forward(x, delta, ctx, cache, owns_cache) -> (x, delta)
                   x is the residual stream, delta an addition not yet applied to it

Per-step arrays of a part's own (any part may offer this; the step builder calls it once per step and key):
  step_arrays_key = "name"               parts that share a key share the arrays (all attention layers: one work list)
  step_arrays(facts) -> {name: int32 numpy array}
                   facts: StepFacts (lens, pos0, kv_len, q_start, slots of the entries; tile size of the kernels).
                   The arrays travel to the device in the step's one metadata buffer; the part finds them as
                   ctx.batch.extras[key][name] (device) and ctx.batch.extras_host[key][name] (numpy).  For a given
                   list of entry lengths the arrays must always have the same sizes (decode steps are replayed
                   as graphs over fixed buffers).

Optional fast-path protocol.  Every name below is declared on Part with a default that means "not offered";
a block reads the attributes, it never probes with hasattr:
  offers_open = True       Mixer: forward_open(h, ctx, cache, position, owns_cache) -> (rows, out_weight)
                           FeedForward: forward_open(h, ctx) -> (rows, out_weight)
                               forward() without its last product: forward == linear(rows, out_weight)
  open_weight              the tensor forward_open returns as out_weight (after load)
  first_weight             the tensor that forward() streams first (after load)
  gated_weight             FeedForward: a [2 I, hidden] tensor that forward() hands to ctx.ops.gated_linear (its product is
                               read by the activation only, so the start-up timing of kernels times the pair)
  first_product_probe(ops, rows)
                           -> run(weight), or None.  run does what forward() does with its first weight (the product and
                               whatever this part lets the kernel namespace fuse with it) for `rows` rows of made-up input;
                               the start-up timing of many-row kernels then times that instead of the bare product
  accepts_deferred = True  Norm: forward hands `delta` to ctx.ops.add_rmsnorm untouched, so the block may give it the
                               result of ctx.ops.linear(..., defer=True) (possibly partial sums the kernel adds up)
  takes_next_weight = True Norm: forward accepts next_weight=<tensor> and passes it to ctx.ops.add_rmsnorm: the block
                               names the first weight of the part that follows, and the kernel may request it into L2
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
    whose block tables (ctx.batch.group_view(group, ...)) address them; for state, the slot tensor."""
    def __init__(self, group: int, k=None, v=None, state=None):
        self.group, self.k, self.v, self.state = group, k, v, state


class StepContext:
    """What a part sees of the step being run."""
    def __init__(self, ops, batch, dtype, device):
        self.ops, self.batch, self.dtype, self.device = ops, batch, dtype, device
        self.defer_ok = False        # set by the model when every reader of a block's outputs accepts deferred sums
        self.hints_ok = False        # the kernel namespace's add_rmsnorm takes next_weight=


class Part:
    # the optional protocol, declared (see the module text); a subclass overrides what it offers
    offers_open = False
    open_weight = None
    first_weight = None
    gated_weight = None
    accepts_deferred = False
    takes_next_weight = False
    step_arrays_key: Optional[str] = None

    def first_product_probe(self, ops, rows):
        return None

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def weight_specs(self):
        return []

    def load(self, tensors, dtype, device):
        pass

    def step_arrays(self, facts):
        return {}

    def step_flops(self, rows: int, pairs: int) -> int:
        """Floating-point operations beyond the part's matrix products, for `rows` tokens that see `pairs`
        (query, key) pairs (an attention mixer: scores and weighted sum)."""
        return 0


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
    if family not in _REGISTRIES:
        raise KeyError(f"no family of parts named '{family}' (known: {', '.join(sorted(_REGISTRIES))})")
    table = _REGISTRIES[family]
    if name not in table:
        raise KeyError(f"no {family} part named '{name}' is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[name]


def build_part(family: str, spec: PartSpec, *args):
    return lookup(family, spec.kind)(spec, *args)
