from .manager import CacheManager, KVGroup, KVNeedKey, RequestCache
from .pages import OutOfPages, PagePool
from .storage import CacheStorage, KVCacheView, StateView

__all__ = ["CacheManager", "CacheStorage", "KVCacheView", "KVGroup", "KVNeedKey", "OutOfPages", "PagePool",
           "RequestCache", "StateView"]
