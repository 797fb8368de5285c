"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""
from .base import (Block, FeedForward, Mixer, Norm, PagedKVNeed, Part, PositionEncoding, StateNeed,
                   TensorDecl, build_part, part_class, register_part, whole_output)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)

__all__ = [
    "Block", "FeedForward", "Mixer", "Norm", "PagedKVNeed", "Part", "PositionEncoding", "StateNeed",
    "TensorDecl", "build_part", "part_class", "register_part", "whole_output",
]
