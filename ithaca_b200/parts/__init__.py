from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Runtime, register_block,
                   register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                   register_position)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registers the kinds)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Runtime", "register_block",
           "register_embedding", "register_feed_forward", "register_head", "register_mixer", "register_norm",
           "register_position"]
