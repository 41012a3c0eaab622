from . import attention, block, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .base import (KVCacheNeed, LayerCache, Part, StateNeed, StepContext, WeightSpec, build_part, lookup,
                   register_block, register_feed_forward, register_mixer, register_norm, register_position)
from .model import DecoderModel

__all__ = ["KVCacheNeed", "LayerCache", "Part", "StateNeed", "StepContext", "WeightSpec", "build_part",
           "lookup", "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "DecoderModel"]
