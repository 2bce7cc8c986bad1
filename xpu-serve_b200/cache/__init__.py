"""Per-sequence storage: slots, paged keys and values by layer group, fixed-size state."""
from .cache import PAGE_SIZE, Cache, CallView, KVGroup, StateGroup
from .pools import CacheError, CacheFull, IndexPool

__all__ = ["PAGE_SIZE", "Cache", "CallView", "KVGroup", "StateGroup", "CacheError", "CacheFull", "IndexPool"]
