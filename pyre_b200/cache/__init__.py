from .allocator import OutOfPages, PageAllocator
from .manager import CacheManager, CacheStats, PagedGroup, StateSlots, pages_for, pages_per_group

__all__ = ["CacheManager", "CacheStats", "OutOfPages", "PageAllocator", "PagedGroup", "StateSlots", "pages_for", "pages_per_group"]
