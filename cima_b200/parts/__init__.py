from .registry import (build_block, build_feed_forward, build_mixer, build_norm, build_position,
                       register_block, register_feed_forward, register_mixer, register_norm,
                       register_position, registered)
from .runtime import Runtime
from .linear import GatedLinearPair, Linear
from . import norm, position, attention, feed_forward, block   # registers the built-in kinds

__all__ = ["build_block", "build_feed_forward", "build_mixer", "build_norm", "build_position",
           "register_block", "register_feed_forward", "register_mixer", "register_norm", "register_position",
           "registered", "Runtime", "GatedLinearPair", "Linear"]
