"""Pages, block tables and state slots."""

from .manager import CacheManager, OutOfPages, OutOfSlots, PageAllocator, PagedCache, StateCache

__all__ = ["CacheManager", "OutOfPages", "OutOfSlots", "PageAllocator", "PagedCache", "StateCache"]
