from .cache import PAGE, Cache, CacheFull, CacheView, SeqRecord
from .pool import IndexPool, PoolError, PoolExhausted

__all__ = ["PAGE", "Cache", "CacheFull", "CacheView", "SeqRecord", "IndexPool", "PoolError", "PoolExhausted"]
