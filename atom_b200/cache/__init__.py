from .manager import NO_PAGE, CacheGroup, CacheManager, RequestCache
from .page_pool import OutOfPages, PagePool
from .state_slots import OutOfSlots, StateSlots

__all__ = ["NO_PAGE", "CacheGroup", "CacheManager", "OutOfPages", "OutOfSlots", "PagePool", "RequestCache", "StateSlots"]
