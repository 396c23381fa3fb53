from .cache import (PAGE, Cache, CacheFull, CacheView, PagedKV, SeqRecord, StateRecords, Storage,
                    register_storage)
from .pool import IndexPool, PoolError, PoolExhausted

__all__ = ["PAGE", "Cache", "CacheFull", "CacheView", "PagedKV", "SeqRecord", "StateRecords", "Storage",
           "register_storage", "IndexPool", "PoolError", "PoolExhausted"]
