"""Slots, paged keys and values, and fixed-size per-sequence state."""
from .slots import CacheFull, CacheMisuse, IndexPool
from .views import BundleView, KVLayerView, StateLayerView
from .manager import CacheManager, KVGroup, StateGroup, SequenceState

__all__ = ["CacheFull", "CacheMisuse", "IndexPool", "BundleView", "KVLayerView", "StateLayerView", "CacheManager",
           "KVGroup", "StateGroup", "SequenceState"]
