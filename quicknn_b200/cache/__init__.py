"""Paged cache with a slot per sequence, grouped storage and fixed-size state."""
from .kv import PAGE, CacheGroup, KVCache, LineView
from .pages import CacheFull, PagePool, SlotTable

__all__ = ["PAGE", "CacheGroup", "KVCache", "LineView", "CacheFull", "PagePool", "SlotTable"]
