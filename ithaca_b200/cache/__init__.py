from .cache import PAGE_SIZE, KVRequest, LayerCache, SequenceCache, StateRequest, plan_groups
from .pages import CacheError, CacheFull, KVGroupLayout, PagePool, SlotTable, StateGroupLayout

__all__ = ["PAGE_SIZE", "KVRequest", "LayerCache", "SequenceCache", "StateRequest", "plan_groups", "CacheError",
           "CacheFull", "KVGroupLayout", "PagePool", "SlotTable", "StateGroupLayout"]
