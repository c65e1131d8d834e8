"""Parts that layers are put together from; importing registers the built-in kinds."""

from . import attention, block, feed_forward, norm, position  # noqa: F401  (registration)
from .base import (Block, BuildEnv, FeedForward, LayerCache, Mixer, Norm, Part,
                   PositionEncoding)
from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, build_part, part_class,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position)

__all__ = ["BLOCKS", "Block", "BuildEnv", "FEED_FORWARDS", "FeedForward", "LayerCache",
           "MIXERS", "Mixer", "NORMS", "Norm", "POSITIONS", "Part", "PositionEncoding",
           "build_part", "part_class", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position"]
