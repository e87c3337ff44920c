from .manager import Appended, CacheManager, FixedStateNeed, PagedGroup, PagedKVNeed, RequestCache
from .pool import OutOfPages, PagePool
from .state_slots import OutOfStateSlots, StateSlots

__all__ = ["Appended", "CacheManager", "FixedStateNeed", "PagedGroup", "PagedKVNeed",
           "RequestCache", "OutOfPages", "PagePool", "OutOfStateSlots", "StateSlots"]
