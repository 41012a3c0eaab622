from .manager import CacheManager, SeqCache
from .page_pool import PagePool
from .state_slots import StateSlots

__all__ = ["CacheManager", "SeqCache", "PagePool", "StateSlots"]
