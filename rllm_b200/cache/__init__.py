from .allocator import BlockAllocator, OutOfPages, SlotAllocator
from .manager import CacheManager, PagedKVView, StateView

__all__ = ["BlockAllocator", "OutOfPages", "SlotAllocator", "CacheManager", "PagedKVView", "StateView"]
