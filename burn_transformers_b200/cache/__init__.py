from .bank import CacheBank, KvGroup, pages_for
from .slots import FreeList
from .spec import PAGE_SIZE, CacheConfig, CacheNeed, KvSpec, StateSpec

__all__ = ["CacheBank", "KvGroup", "pages_for", "FreeList", "PAGE_SIZE", "CacheConfig", "CacheNeed", "KvSpec",
           "StateSpec"]
