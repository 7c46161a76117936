from .pages import PAGE_TOKENS, CacheFull, CacheMisuse, PagePool, SequencePages, SlotTable, pages_for
from .store import CacheSpec, KVSpec, LayerCache, SequenceCache, StateSpec

__all__ = ["PAGE_TOKENS", "CacheFull", "CacheMisuse", "PagePool", "SequencePages", "SlotTable", "pages_for",
           "CacheSpec", "KVSpec", "LayerCache", "SequenceCache", "StateSpec"]
