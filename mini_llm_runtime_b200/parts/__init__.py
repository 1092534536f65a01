from . import attention, block, embedding, latent_attention, mlp, moe, norm, offsets, parallel, recurrent, rope, shift  # noqa: F401  (registers the parts)
from .base import (Block, Embedding, FeedForward, Head, KVCacheNeed, Mixer, Norm, Part, PendingDelta,
                   PositionEncoding, StreamOffsets, Shift, StateNeed, TensorSpec, build_part, known_parts, part_factory,
                   register_part, unregister_part)

__all__ = [
    "Block", "Embedding", "FeedForward", "Head", "KVCacheNeed", "Mixer", "Norm", "Part", "PendingDelta",
    "PositionEncoding", "StreamOffsets", "Shift", "StateNeed", "TensorSpec", "build_part", "known_parts", "part_factory",
    "register_part", "unregister_part",
]
