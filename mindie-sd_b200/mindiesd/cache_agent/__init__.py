from .cache import CacheConfig
from .cache_agent import CacheAgent

__all__ = ["CacheConfig", "CacheAgent"]
