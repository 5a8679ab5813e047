"""Cache classes with the reference's interfaces (models/cache/)."""
from .kvcomp_cache import KVCompCache
from .kvcomp_encode import KVCompCtx
from ..utils.config import KVCompCacheConfig, KVCompCacheConfigStatic

__all__ = ["KVCompCache", "KVCompCtx", "KVCompCacheConfig", "KVCompCacheConfigStatic"]
