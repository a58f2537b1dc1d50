from .manager import CacheManager
from .pages import CacheError, PagePool, SlotPool

__all__ = ["CacheManager", "CacheError", "PagePool", "SlotPool"]
