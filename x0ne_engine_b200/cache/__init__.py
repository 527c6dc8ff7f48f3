"""The cache: slots, paged keys and values per group of layers, fixed-size per-sequence state."""
from .paged import PAGE_SIZE, KVGroup, SequenceCache, pages_for
from .slots import CacheFull, FreeList

__all__ = ["PAGE_SIZE", "KVGroup", "SequenceCache", "pages_for", "CacheFull", "FreeList"]
