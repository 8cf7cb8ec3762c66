from .allocator import BlockAllocator, OutOfPages, SlotAllocator
from .manager import CacheManager, PagedKVView, RequestTooLong, StateView

__all__ = ["BlockAllocator", "OutOfPages", "SlotAllocator", "CacheManager", "RequestTooLong", "PagedKVView", "StateView"]
