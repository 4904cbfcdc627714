from .manager import FREED, AppendPlan, CacheManager, EntryCache, RequestCache
from .needs import FixedState, PagedKV
from .pages import OutOfPages, PagePool

__all__ = ["FREED", "AppendPlan", "CacheManager", "EntryCache", "RequestCache", "FixedState",
           "PagedKV", "OutOfPages", "PagePool"]
