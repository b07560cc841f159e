from .manager import CacheManager, GroupSpec
from .page_pool import OutOfPages, PagePool, StateSlotAllocator
from .storage import CacheLayout, CacheStorage

__all__ = ["CacheManager", "GroupSpec", "OutOfPages", "PagePool", "StateSlotAllocator", "CacheLayout", "CacheStorage"]
