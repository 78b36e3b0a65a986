"""Layer parts and their registries.  Importing this package registers the built-in kinds."""
from .base import Part, TensorDecl
from .registry import (build_feed_forward, build_mixer, build_norm, build_position, register_feed_forward,
                       register_mixer, register_norm, register_position, registered)
from . import norm, position, attention, feedforward  # noqa: F401  (registration)
from .block import Block
from .linear import Linear

__all__ = ["Part", "TensorDecl", "Block", "Linear", "build_feed_forward", "build_mixer", "build_norm",
           "build_position", "register_feed_forward", "register_mixer", "register_norm", "register_position",
           "registered"]
