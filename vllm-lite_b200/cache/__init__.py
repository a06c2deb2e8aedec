"""Paged key/value cache, per-request state slots and their device storage."""
from .manager import CacheLayout, CacheManager, OutOfPages, RequestCache  # noqa: F401
from .pool import Pool, PoolError  # noqa: F401
from .spec import FixedState, PagedKV  # noqa: F401
