from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (register the built-in parts)
from .base import (BuildEnv, CacheNeed, FixedState, PagedKV, Part, ResidualStream, WeightDecl, build_part,
                   register_part, unregister_part)
from .decoder import DecoderModel, EntryCache

__all__ = ["BuildEnv", "CacheNeed", "DecoderModel", "EntryCache", "FixedState", "PagedKV", "Part",
           "ResidualStream", "WeightDecl", "build_part", "register_part", "unregister_part"]
