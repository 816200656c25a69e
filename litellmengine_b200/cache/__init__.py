"""The cache manager: paged keys and values per group of stages, block tables, state slots."""
from .pages import (CacheError, CacheGroup, CacheManager, OutOfPages, PagedNeed, PagePool,
                    StateNeed)

__all__ = ["CacheError", "CacheGroup", "CacheManager", "OutOfPages", "PagedNeed", "PagePool",
           "StateNeed"]
