from .manager import CacheManager, CacheGroup, PagePool, OutOfPages, CacheError, group_layers
from .storage import CacheStorage

__all__ = ["CacheManager", "CacheGroup", "PagePool", "OutOfPages", "CacheError", "group_layers", "CacheStorage"]
