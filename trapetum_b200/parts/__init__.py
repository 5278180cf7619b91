"""Parts of a layer and the registries that build them (see :mod:`.base`)."""
from .base import (Block, FeedForward, KVNeed, Mixer, Norm, Part, PositionEncoding, Runtime, StateNeed,
                   build_part, known_parts, register_part)
from .stream import ResidualStream
from . import norm, rope, attention, feed_forward, block, ends  # noqa: F401  (register the built-in kinds)

__all__ = ["Block", "FeedForward", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "StateNeed",
           "ResidualStream", "build_part", "known_parts", "register_part"]
