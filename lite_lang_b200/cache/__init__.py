from .manager import CacheError, CacheManager, PageAllocator, PagedGroupSpec, StateGroupSpec

__all__ = ["CacheError", "CacheManager", "PageAllocator", "PagedGroupSpec", "StateGroupSpec"]
