"""Cache: page pools, the cache manager, and the views it hands to mixers."""

from .manager import FREED, CacheManager, CacheView, PagedView
from .pages import OutOfPages, PagePool

__all__ = ["FREED", "CacheManager", "CacheView", "PagedView", "OutOfPages", "PagePool"]
