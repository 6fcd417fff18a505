"""The cache: the manager (host bookkeeping) and the storage (device tensors)."""

from ayaka_b200.cache.manager import CacheManager, PagePool
from ayaka_b200.cache.storage import CachePlan, CacheStorage, plan_cache

__all__ = ["CacheManager", "CachePlan", "CacheStorage", "PagePool", "plan_cache"]
