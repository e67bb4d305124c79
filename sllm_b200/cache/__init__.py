from .manager import CacheGroup, CacheManager, RequestCache
from .pools import OutOfPages, PagePool, SlotPool

__all__ = ["CacheGroup", "CacheManager", "RequestCache", "OutOfPages", "PagePool", "SlotPool"]
