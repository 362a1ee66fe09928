from .allocator import FreeList, SlotBook, CacheFull, ContextOverflow
from .cache import SequenceCache, CacheLayerView, CacheGroup, PAGE_SIZE

__all__ = ["FreeList", "SlotBook", "CacheFull", "ContextOverflow", "SequenceCache", "CacheLayerView",
           "CacheGroup", "PAGE_SIZE"]
