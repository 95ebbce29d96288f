from .manager import FULL, WINDOW, CacheError, CacheGroup, CacheManager, GroupSpec, PagePool, StateSlots

__all__ = ["FULL", "WINDOW", "CacheError", "CacheGroup", "CacheManager", "GroupSpec", "PagePool", "StateSlots"]
