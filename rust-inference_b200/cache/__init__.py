"""The cache: slots, paged keys and values per group of layers, per-sequence state."""
from .allocator import CacheError, HostCache, PageTable, SlotAllocator
from .kv_cache import PAGE_SIZE, Cache, LayerCache

__all__ = ["CacheError", "HostCache", "PageTable", "SlotAllocator", "PAGE_SIZE", "Cache", "LayerCache"]
