"""The parts a model is put together from, and their registry."""
from . import (attention, block, delta_rule, embedding, feedforward, latent_attention, mapped_attention, moe, norm, parallel,
               position, sink_attention, state_space)  # noqa: F401  (they register themselves)
from .base import (Arrangement, CompositeCacheSpec, Embedding, FeedForward, Head, KVCacheSpec, Mixer, Norm, Part,
                   PositionEncoding, RowCacheSpec, StateCacheSpec, TensorSpec, build_part, known_parts, register_part)
from .linear import Linear

__all__ = ["Arrangement", "CompositeCacheSpec", "Embedding", "FeedForward", "Head", "KVCacheSpec", "Linear", "Mixer", "Norm",
           "Part", "PositionEncoding", "RowCacheSpec", "StateCacheSpec", "TensorSpec", "build_part", "known_parts",
           "register_part"]
