from .pages import PagePool, SlotPool, CacheAccountingError
from .manager import CacheManager, GroupSpec, RequestCache, NO_PAGE
