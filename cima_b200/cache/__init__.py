from .pages import CacheFull, FreeList
from .kv import CapacityError, KVCache, KVGroup, KVRequest, LayerKV, StateRequest

__all__ = ["CacheFull", "FreeList", "CapacityError", "KVCache", "KVGroup", "KVRequest", "LayerKV", "StateRequest"]
