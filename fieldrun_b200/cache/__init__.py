from .pools import CacheFull, IndexPool
from .sequence_cache import PAGE_TOKENS, CacheNeed, LineView, SequenceCache, pages_for

__all__ = ["CacheFull", "CacheNeed", "IndexPool", "LineView", "PAGE_TOKENS", "SequenceCache", "pages_for"]
