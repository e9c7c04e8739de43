from .allocator import PageAllocator, OutOfPages
from .manager import CacheManager, CacheGroup, pages_for

__all__ = ["PageAllocator", "OutOfPages", "CacheManager", "CacheGroup", "pages_for"]
