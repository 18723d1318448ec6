from .book import PAGE, CacheBook, FreeList, GroupBook, KvLayout, pages_for
from .storage import Cache, LayerCache, StateSpec

__all__ = ["PAGE", "CacheBook", "FreeList", "GroupBook", "KvLayout", "pages_for", "Cache", "LayerCache", "StateSpec"]
