from .base import (FeedForward, Mixer, Norm, PagedKVNeed, Part, PartError, Runtime, StateNeed,
                   build_part, part_class, register_part)
from . import attention, block, embedding, ffn, norm, rotary  # noqa: F401  (register the built-in kinds)

__all__ = ["FeedForward", "Mixer", "Norm", "PagedKVNeed", "Part", "PartError", "Runtime", "StateNeed",
           "build_part", "part_class", "register_part"]
