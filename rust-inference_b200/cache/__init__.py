"""The cache: slots, paged keys and values per group of layers, per-sequence state."""
from .allocator import CacheError, PageTable, SlotAllocator
from .kv_cache import PAGE_SIZE, Cache, LayerCache

__all__ = ["CacheError", "PageTable", "SlotAllocator", "PAGE_SIZE", "Cache", "LayerCache"]
