"""Parts that layers are put together from.  Importing the package registers the built-in kinds."""
from .base import (Block, FeedForward, Mixer, Norm, PagedKVNeed, Part, PositionEncoding, StateNeed,
                   TensorDecl, build_part, part_class, register_part, whole_output)
from . import (attention, block, delta_rule, embedding, latent_attention, linear_attention, mlp, modulated_attention,  # noqa: F401
               norm, rope, routed, side_by_side, state_space, streams)                          # (registration)

__all__ = [
    "Block", "FeedForward", "Mixer", "Norm", "PagedKVNeed", "Part", "PositionEncoding", "StateNeed",
    "TensorDecl", "build_part", "part_class", "register_part", "whole_output",
]
