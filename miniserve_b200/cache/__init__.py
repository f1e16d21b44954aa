from .blocks import BlockAllocator, BlockTable, OutOfBlocks
from .manager import CacheGroup, CacheManager, KVEntryView, RequestCache, StateEntryView

__all__ = ["BlockAllocator", "BlockTable", "CacheGroup", "CacheManager", "KVEntryView", "OutOfBlocks",
           "RequestCache", "StateEntryView"]
