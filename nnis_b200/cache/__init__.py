from .manager import (PAGE_SIZE, CacheManager, CacheSnapshot, KVRequest, KVView, StateRequest,
                      StateView)
from .slots import CacheFull, FreeList, SlotError

__all__ = ["PAGE_SIZE", "CacheManager", "CacheSnapshot", "KVRequest", "KVView", "StateRequest",
           "StateView", "CacheFull", "FreeList", "SlotError"]
