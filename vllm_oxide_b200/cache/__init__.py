from .paged_cache import CacheGroup, PagedCache

__all__ = ["CacheGroup", "PagedCache"]
