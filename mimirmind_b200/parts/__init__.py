"""The parts layers are made of.  Importing this package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401
from .base import (Block, CacheArray, FeedForward, KVCacheSpec, LayerCache, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StateSpec, StepContext, WeightView)

__all__ = ["Block", "CacheArray", "FeedForward", "KVCacheSpec", "LayerCache", "Mixer", "Norm", "Part", "PositionEncoding",
           "Runtime", "StateSpec", "StepContext", "WeightView"]
