from .manager import FREED, AppendPlan, CacheManager, EntryCache, RequestCache, token_bytes
from .needs import FixedState, PagedKV, PagedLatent, PagedMaps
from .pages import OutOfPages, PagePool

__all__ = ["FREED", "AppendPlan", "CacheManager", "EntryCache", "RequestCache", "FixedState",
           "PagedKV", "PagedLatent", "OutOfPages", "PagePool", "token_bytes"]
