from .slots import CacheError, CacheFull, PagePool, SlotAllocator
from .kv import PAGE, CacheGroup, CacheNeed, KVCache, StateStore, pages_for

__all__ = ["CacheError", "CacheFull", "PagePool", "SlotAllocator", "PAGE", "CacheGroup",
           "CacheNeed", "KVCache", "StateStore", "pages_for"]
