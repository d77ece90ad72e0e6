from . import attention, block, embedding, feedforward, norm, rope  # noqa: F401  (registers the parts)
from .block import Block
from .base import (FeedForward, KVNeed, LayerCache, Mixer, Part, Runtime, StateNeed, StepContext, build_part,
                   part_class, register_part)

__all__ = ["Block", "FeedForward", "KVNeed", "LayerCache", "Mixer", "Part", "Runtime", "StateNeed", "StepContext",
           "build_part", "part_class", "register_part"]
