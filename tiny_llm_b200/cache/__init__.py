from .manager import CacheEntryRef, CacheManager, KVGroup, KVNeed, StateNeed, StateSlots
from .pages import PageError, PagePool

__all__ = ["CacheManager", "CacheEntryRef", "KVGroup", "KVNeed", "StateNeed", "StateSlots", "PageError", "PagePool"]
