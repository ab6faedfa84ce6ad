from .pools import CacheError, CacheFull, IndexPool, PageLedger
from .sequence_cache import KVView, SequenceCache, StateView, StepPlan

__all__ = ["CacheError", "CacheFull", "IndexPool", "PageLedger", "KVView", "SequenceCache",
           "StateView", "StepPlan"]
