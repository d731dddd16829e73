from .manager import CacheManager, PagedGroupSpec, StateGroupSpec
from .pages import OutOfPages, PagePool, SlotPool
from .storage import CacheStorage, PagedStorage

__all__ = ["CacheManager", "CacheStorage", "OutOfPages", "PagePool", "PagedGroupSpec",
           "PagedStorage", "SlotPool", "StateGroupSpec"]
