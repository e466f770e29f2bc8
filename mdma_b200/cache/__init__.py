from .kv import CacheGroup, KVNeed, KVView, SequenceCache, StateNeed
from .slots import CacheFull, FreeList

__all__ = ["CacheFull", "CacheGroup", "FreeList", "KVNeed", "KVView", "SequenceCache", "StateNeed"]
