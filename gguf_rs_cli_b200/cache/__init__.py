from .cache import Cache, CacheLayout, KVGroup, KVSpec
from .pool import PAGE, PAGE_SHIFT, CacheError, CacheFull, FreeList, pages_for

__all__ = ["Cache", "CacheLayout", "KVGroup", "KVSpec", "PAGE", "PAGE_SHIFT", "CacheError", "CacheFull",
           "FreeList", "pages_for"]
