from .book import CacheBook, CacheError, CacheFull, GroupGeometry
from .store import CacheView, SequenceCache

__all__ = ["CacheBook", "CacheError", "CacheFull", "CacheView", "GroupGeometry", "SequenceCache"]
