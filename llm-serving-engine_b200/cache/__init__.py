from .allocator import OutOfPages, PageAllocator
from .manager import RELEASED, CacheManager, KVGroupSpec, StateGroupSpec
from .pools import CachePools, CacheView, group_cache_layers, pages_for_memory

__all__ = [
    "OutOfPages", "PageAllocator", "RELEASED", "CacheManager", "KVGroupSpec", "StateGroupSpec",
    "CachePools", "CacheView", "group_cache_layers", "pages_for_memory",
]
