from .manager import NO_PAGE, CacheManager, PagedStorage, RequestCache, StateStorage
from .pool import OutOfPages, PoolError, UnitPool

__all__ = ["CacheManager", "RequestCache", "PagedStorage", "StateStorage", "UnitPool", "OutOfPages", "PoolError",
           "NO_PAGE"]
