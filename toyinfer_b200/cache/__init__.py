"""The cache: slots, pages, fixed-size states."""
from .allocators import CacheError, PagePool, SlotAllocator
from .manager import PAGE, CacheManager, KVView, StateView, bytes_per_token, pages_for

__all__ = ["CacheError", "PagePool", "SlotAllocator", "PAGE", "CacheManager", "KVView", "StateView", "bytes_per_token", "pages_for"]
