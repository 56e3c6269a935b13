from .manager import NO_PAGE, CacheFullError, CacheManager, RequestCache
from .page_pool import PagePool, PoolError, SlotPool
from .spec import FixedStateSpec, PagedKVSpec

__all__ = ["NO_PAGE", "CacheFullError", "CacheManager", "RequestCache", "PagePool",
           "PoolError", "SlotPool", "FixedStateSpec", "PagedKVSpec"]
