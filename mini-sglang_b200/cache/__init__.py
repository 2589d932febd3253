from .manager import CacheManager, KVGroup, OutOfSlots, PagedKVNeed, StateNeed
from .pages import OutOfPages, PagePool
from .radix import PrefixTree

__all__ = ["CacheManager", "KVGroup", "OutOfSlots", "PagedKVNeed", "StateNeed", "OutOfPages", "PagePool", "PrefixTree"]
