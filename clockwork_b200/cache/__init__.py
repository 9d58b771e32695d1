from .allocator import OutOfPages, PageAllocator
from .manager import NO_PAGE, CacheManager, PageGroup, RequestCache, StateSlots
from .prefix import PrefixCache, PrefixCacheStats, PrefixMatch, PrefixTree

__all__ = [
    "OutOfPages", "PageAllocator", "NO_PAGE", "CacheManager", "PageGroup", "RequestCache",
    "StateSlots", "PrefixCache", "PrefixCacheStats", "PrefixMatch", "PrefixTree",
]
