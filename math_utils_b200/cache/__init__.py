"""Slots, paged keys and values, and fixed-size per-sequence state."""
from .sequence_cache import (PAGE_TOKENS, CacheError, CacheFull, KVEntryView, KVGroup, PagePool,
                             SequenceCache, SlotAllocator, StateEntryView, StateGroup)

__all__ = ["PAGE_TOKENS", "CacheError", "CacheFull", "KVEntryView", "KVGroup", "PagePool",
           "SequenceCache", "SlotAllocator", "StateEntryView", "StateGroup"]
