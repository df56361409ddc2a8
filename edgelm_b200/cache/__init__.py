from .cache import PAGE, CacheEntry, KVGroup, SequenceCache, StateGroup, pages_for
from .slots import CacheError, FreeList

__all__ = ["PAGE", "CacheEntry", "KVGroup", "SequenceCache", "StateGroup", "pages_for", "CacheError", "FreeList"]
