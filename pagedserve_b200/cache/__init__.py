"""Paged KV cache: page allocator, layer groups, block tables, per-request state slots."""

from pagedserve_b200.cache.manager import (  # noqa: F401
    CacheError,
    CacheFull,
    CacheGroup,
    CacheManager,
    KVNeed,
    PageAllocator,
    StateNeed,
)
