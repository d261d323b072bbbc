"""The cache: pages with block tables per group of layers, and per-request state slots."""
from .groups import NO_PAGE, CacheGroup, CacheNeed, PagedKV, StateSlot
from .manager import CacheManager, KVView, StateView
from .pages import OutOfPages, PagePool
from .slots import OutOfSlots, SlotAllocator

__all__ = ["NO_PAGE", "CacheGroup", "CacheNeed", "PagedKV", "StateSlot", "CacheManager", "KVView", "StateView",
           "OutOfPages", "PagePool", "OutOfSlots", "SlotAllocator"]
