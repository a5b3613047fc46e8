"""The cache manager: native page-id pool, paged slabs, block tables, seats, state slots."""

from .block_pool import BlockPool
from .manager import CacheExhausted, CacheManager, KvGroup, pages_needed, pages_that_fit

__all__ = ["BlockPool", "CacheExhausted", "CacheManager", "KvGroup", "pages_needed", "pages_that_fit"]
