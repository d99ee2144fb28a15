"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401
from .base import (Block, FeedForward, Mixer, Norm, Part, Position, build_block, build_part, build_position,
                   register_part, registered)

__all__ = ["Block", "FeedForward", "Mixer", "Norm", "Part", "Position", "build_block", "build_part",
           "build_position", "register_part", "registered"]
