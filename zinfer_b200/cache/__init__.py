from .manager import CacheManager, KVGroup, KVNeedKey, RequestCache
from .pages import OutOfPages, PagePool
from .sizing import bytes_per_page, bytes_per_token, pages_for
from .storage import CacheStorage, KVCacheView, StateView

__all__ = ["CacheManager", "CacheStorage", "KVCacheView", "KVGroup", "KVNeedKey", "OutOfPages", "PagePool",
           "RequestCache", "StateView", "bytes_per_page", "bytes_per_token", "pages_for"]
