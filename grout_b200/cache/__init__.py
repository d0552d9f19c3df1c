from .cache import CacheLayout, SequenceCache
from .slots import FreeList, PagePool, SlotList
from .spec import CacheFull, KVSpec, PAGE_TOKENS, StateSpec, StoreSizes
from .stores import KVLayerView, KVStore, StateLayerView, StateStore, pages_for

__all__ = ["CacheLayout", "SequenceCache", "FreeList", "PagePool", "SlotList", "CacheFull",
           "KVSpec", "PAGE_TOKENS", "StateSpec", "StoreSizes", "KVLayerView", "KVStore", "StateLayerView",
           "StateStore", "pages_for"]
