from .spec import GroupSpec, CacheAccountingError, NO_PAGE
from .native import NativeCacheManager

CacheManager = NativeCacheManager


def make_cache_manager(groups, page_size, pages_per_group, max_live_requests):
    """The cache manager of the C++ host runtime (csrc/host/host_runtime.cpp)."""
    return NativeCacheManager(groups, page_size, pages_per_group, max_live_requests)
