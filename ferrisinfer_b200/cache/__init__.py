"""The cache manager: page pools, block tables, state slots."""

from .manager import NO_PAGE, CacheManager, PageGroup, PrefixIndex, RequestCache, register_cache_need
from .pages import PagePool
