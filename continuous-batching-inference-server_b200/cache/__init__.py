from .pool import CacheGroup, CachePool, LayerCache, cache_groups_of

__all__ = ["CacheGroup", "CachePool", "LayerCache", "cache_groups_of"]
