from .paged import PAGE, Cache, StorageGroup
from .pool import CacheError, CacheFull, IdPool
