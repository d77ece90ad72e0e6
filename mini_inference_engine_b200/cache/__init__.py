from .manager import RELEASED, CacheManager, GroupSpec, RequestCache
from .pages import PageError, PagePool

__all__ = ["RELEASED", "CacheManager", "GroupSpec", "RequestCache", "PageError", "PagePool"]
