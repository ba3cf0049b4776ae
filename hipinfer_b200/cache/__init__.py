from .manager import (CacheError, CacheGroupSpec, CacheManager, OutOfPages, OutOfStateSlots, PagePool, RequestCache,
                      SlotPool, register_retention)

from .storage import CacheStorage, LayerCache

__all__ = ["CacheStorage", "LayerCache", "CacheError", "CacheGroupSpec", "CacheManager", "OutOfPages", "OutOfStateSlots", "PagePool",
           "RequestCache", "SlotPool", "register_retention"]
