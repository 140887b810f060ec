"""Slots, pages and per-sequence state."""

from .allocator import IdPool
from .kv_cache import CacheNeed, CacheView, KVNeed, SequenceCache, StateNeed

__all__ = ["IdPool", "CacheNeed", "CacheView", "KVNeed", "SequenceCache", "StateNeed"]
