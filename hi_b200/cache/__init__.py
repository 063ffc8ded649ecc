from .pages import FREED, CacheManager, OutOfPages, OutOfSlots, PagePool

__all__ = ["FREED", "CacheManager", "OutOfPages", "OutOfSlots", "PagePool"]
