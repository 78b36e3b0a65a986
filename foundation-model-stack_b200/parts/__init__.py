"""Layer parts and their registries.  Importing this package registers the built-in kinds."""
from .base import Part, TensorDecl
from .registry import (build_block, build_feed_forward, build_mixer, build_norm, build_position, register_block,
                       register_feed_forward, register_mixer, register_norm, register_position, registered)
from . import norm, position, attention, feedforward  # noqa: F401  (registration)
from .block import Block, PreNormBlock
from .linear import Linear
from .position import PositionEncoding

__all__ = ["Part", "TensorDecl", "Block", "PreNormBlock", "Linear", "PositionEncoding", "build_block", "build_feed_forward",
           "build_mixer", "build_norm", "build_position", "register_block", "register_feed_forward", "register_mixer",
           "register_norm", "register_position", "registered"]
