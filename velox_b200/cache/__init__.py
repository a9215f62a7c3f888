from .allocator import NULL_PAGE, OutOfPagesError, PageAllocator
from .manager import CacheGroup, CacheManager, SequenceCache

__all__ = [
    "CacheGroup",
    "CacheManager",
    "NULL_PAGE",
    "OutOfPagesError",
    "PageAllocator",
    "SequenceCache",
]
