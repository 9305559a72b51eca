from .manager import CacheFullError, CacheGroup, CacheManager, LayerCache, PagePool, RequestCache

__all__ = ["CacheFullError", "CacheGroup", "CacheManager", "LayerCache", "PagePool", "RequestCache"]
