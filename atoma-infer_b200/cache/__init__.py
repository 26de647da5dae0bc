from .spec import FULL_KEYS, WINDOW_KEYS, CachedTensor, CacheGroup, CacheNeed, LayerCache
from .manager import CacheError, CacheManager, OutOfPages
from .kv_cache import KVCache, page_bytes, pages_for_memory, state_bytes_total
