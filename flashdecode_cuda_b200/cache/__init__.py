"""Slots, paged key/value storage per layer group, and per-sequence state."""

from .allocator import IdAllocator, PoolExhausted
from .paged import ACTIVE, FREE, KVGroup, KVGroupSpec, PagedCache, SlotRecord, StateSpec

__all__ = ["IdAllocator", "PoolExhausted", "KVGroupSpec", "StateSpec", "KVGroup", "PagedCache",
           "SlotRecord", "ACTIVE", "FREE"]
