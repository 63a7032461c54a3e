"""The cache: slots, pages, keys and values per layer group, and per-sequence state."""
from .allocators import CacheFull, CacheStateError, PageAllocator, SlotAllocator
from .sequence_cache import PAGE_SIZE, KVGroup, LayerCache, SequenceCache, pages_for

__all__ = ["CacheFull", "CacheStateError", "KVGroup", "LayerCache", "PAGE_SIZE", "PageAllocator",
           "SequenceCache", "SlotAllocator", "pages_for"]
