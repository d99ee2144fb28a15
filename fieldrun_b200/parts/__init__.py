"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401
from .base import (Block, DeferredUpdate, WeightedRows, FeedForward, Mixer, Norm, Part, Position, as_tensor, build_block, build_part,
                   build_position, register_part, registered)

__all__ = ["Block", "DeferredUpdate", "WeightedRows", "as_tensor", "FeedForward", "Mixer", "Norm", "Part", "Position", "build_block", "build_part",
           "build_position", "register_part", "registered"]
