from .allocator import CacheFull, IndexAllocator
from .layout import CacheGroup, KVNeed, StateNeed, plan_groups
from .store import PAGE_TOKENS, SequenceCache, pages_for

__all__ = ["CacheFull", "CacheGroup", "IndexAllocator", "KVNeed", "PAGE_TOKENS", "SequenceCache",
           "StateNeed", "pages_for", "plan_groups"]
