from .allocator import CacheError, FreeList, GroupPages, SlotBook
from .storage import PAGE_SIZE, CacheGroup, LayerCache, SequenceCache

__all__ = ["CacheError", "FreeList", "GroupPages", "SlotBook", "PAGE_SIZE", "CacheGroup",
           "LayerCache", "SequenceCache"]
