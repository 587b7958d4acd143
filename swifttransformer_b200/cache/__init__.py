from .manager import CacheManager, PagedCacheView, PagedGroup, StateView
from .pages import PageError, PagePool

__all__ = ["CacheManager", "PageError", "PagePool", "PagedCacheView", "PagedGroup", "StateView"]
