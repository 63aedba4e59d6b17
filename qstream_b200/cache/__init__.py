"""The cache: slots, paged keys and values per layer group, per-sequence state."""
from .pages import PagePool, SlotTable
from .kv import (PAGE_TOKENS, CacheView, KvGroup, KvNeed, SequenceCache, StateNeed, StateStore)

__all__ = ["PagePool", "SlotTable", "PAGE_TOKENS", "CacheView", "KvGroup", "KvNeed", "SequenceCache",
           "StateNeed", "StateStore"]
