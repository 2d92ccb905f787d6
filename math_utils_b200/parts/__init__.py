"""The parts a model is put together from, and their registry."""
from . import attention, block, embedding, feedforward, norm, position  # noqa: F401  (they register themselves)
from .base import (Arrangement, Embedding, FeedForward, Head, KVCacheSpec, Mixer, Norm, Part,
                   PositionEncoding, StateCacheSpec, TensorSpec, build_part, known_parts, register_part)
from .linear import Linear

__all__ = ["Arrangement", "Embedding", "FeedForward", "Head", "KVCacheSpec", "Linear", "Mixer", "Norm",
           "Part", "PositionEncoding", "StateCacheSpec", "TensorSpec", "build_part", "known_parts",
           "register_part"]
