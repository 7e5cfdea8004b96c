from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Runtime, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position)
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registers the kinds)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Runtime", "register_block",
           "register_feed_forward", "register_mixer", "register_norm", "register_position"]
