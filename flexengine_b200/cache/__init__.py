from .manager import RELEASED, CacheManager, PagedGroup, RequestCache, StateGroup
from .page_pool import CacheExhausted, PagePool

__all__ = ["RELEASED", "CacheManager", "PagedGroup", "RequestCache", "StateGroup", "CacheExhausted", "PagePool"]
