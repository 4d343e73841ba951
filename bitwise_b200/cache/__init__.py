from .manager import FREED, CacheError, CacheManager, GroupSpec, PagePool, RequestCache, groups_from_needs
from .storage import FINGERPRINT_SEED, CacheStorage, build_cache

__all__ = ["FREED", "CacheError", "CacheManager", "GroupSpec", "PagePool", "RequestCache",
           "groups_from_needs", "FINGERPRINT_SEED", "CacheStorage", "build_cache"]
