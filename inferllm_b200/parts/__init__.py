from . import attention, block, embedding, feedforward, norm, position  # noqa: F401 (registration)
from .base import (Block, FeedForward, FixedState, Mixer, Norm, PagedKV, Part, PositionEncoding,
                   ResidualStream, Runtime, TensorDecl, build_part, lookup, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)

__all__ = ["Block", "FeedForward", "FixedState", "Mixer", "Norm", "PagedKV", "Part",
           "PositionEncoding", "ResidualStream", "Runtime", "TensorDecl", "build_part", "lookup",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position"]
