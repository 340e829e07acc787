from .pages import PagePool, SlotPool, CacheAccountingError
from .manager import CacheManager, GroupSpec, RequestCache, NO_PAGE
from .native import NativeCacheManager


def make_cache_manager(groups, page_size, pages_per_group, max_live_requests, native: bool = True):
    """The cache manager of the C++ host runtime, or its Python twin (same interface, same decisions)."""
    cls = NativeCacheManager if native else CacheManager
    return cls(groups, page_size, pages_per_group, max_live_requests)
