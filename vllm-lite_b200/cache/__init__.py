"""Paged key/value cache, per-request state slots and their device storage."""
from .manager import CacheLayout, CacheManager, OutOfPages, RequestCache  # noqa: F401
from .pool import Pool, PoolError  # noqa: F401
from .spec import FixedState, PagedKV  # noqa: F401


def make_cache_manager(layout, page_size, num_pages, max_requests, native=True):
    """The cache manager with its bookkeeping in C++ (default) or the pure-Python reference."""
    if native:
        from .native import NativeCacheManager
        return NativeCacheManager(layout, page_size, num_pages, max_requests)
    return CacheManager(layout, page_size, num_pages, max_requests)
