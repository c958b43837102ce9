from .manager import CacheGroup, CacheManager, RequestCache
from .page_pool import OutOfPages, PagePool, chain_hash
from .state_slots import StateSlots

__all__ = ["CacheGroup", "CacheManager", "RequestCache", "OutOfPages", "PagePool", "chain_hash", "StateSlots"]
