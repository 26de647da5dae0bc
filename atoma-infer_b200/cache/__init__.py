from .manager import (
    FULL_KEYS, WINDOW_KEYS, CacheError, CacheGroup, CacheManager, CacheNeed, OutOfPages,
)
