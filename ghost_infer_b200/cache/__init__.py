from .pages import PAGE_TOKENS, CacheFullError, PagePool, SlotAllocator, pages_for
from .sequence_cache import CacheRequest, LayerMemory, SequenceCache, StateRequest

__all__ = ["PAGE_TOKENS", "CacheFullError", "PagePool", "SlotAllocator", "pages_for",
           "CacheRequest", "LayerMemory", "SequenceCache", "StateRequest"]
