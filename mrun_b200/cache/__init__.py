from .manager import FREED, AppendPlan, CacheManager, EntryCache, RequestCache, token_bytes
from .needs import FixedState, PagedKV
from .pages import OutOfPages, PagePool

__all__ = ["FREED", "AppendPlan", "CacheManager", "EntryCache", "RequestCache", "FixedState",
           "PagedKV", "OutOfPages", "PagePool", "token_bytes"]
