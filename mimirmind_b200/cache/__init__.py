from .manager import CacheError, CacheManager, GroupSpec
from .pages import INVALID_PAGE, PageAllocator, PageAllocatorError

__all__ = ["CacheError", "CacheManager", "GroupSpec", "INVALID_PAGE", "PageAllocator", "PageAllocatorError"]
