"""`CacheAgent` (mindiesd/cache_agent/cache_agent.py:26-87 of MindIE-SD): validates a `CacheConfig`
and routes `apply(function, ...)` through the configured cache, or straight to the function when
the configuration leaves nothing to cache."""
from ..utils.exception import ConfigError, ParametersInvalid, logger
from .attention_cache import AttentionCache, BlockMaskCache
from .cache import CacheConfig

CACHE_METHOD = {
    "attention_cache": AttentionCache,
    "block_mask_cache": BlockMaskCache,
}
# Methods of the reference that lie outside the attention path and are not built here.
_UNBUILT_METHODS = ("dit_block_cache",)


class CacheAgent:
    def __init__(self, config: CacheConfig):
        self._config = config
        self._check_config()
        self._cache_method = CACHE_METHOD[config.method](config)

    def apply(self, function, *args, **kwargs):
        if not callable(function):
            raise ParametersInvalid("Input function must be callable.")
        cfg = self._config
        inactive = (cfg.step_start >= cfg.steps_count or cfg.step_end == cfg.step_start or
                    cfg.block_start >= cfg.blocks_count or cfg.block_end == cfg.block_start or
                    cfg.step_interval == 1)
        if inactive and cfg.method == "attention_cache":
            return function(*args, **kwargs)
        return self._cache_method.apply(function, *args, **kwargs)

    def _check_config(self):
        cfg = self._config
        if cfg.method in _UNBUILT_METHODS:
            raise ConfigError(f"Method '{cfg.method}' is not part of this build (it caches whole DiT blocks, "
                              f"not attention); supported methods: {list(CACHE_METHOD)}.")
        if cfg.method not in CACHE_METHOD:
            raise ConfigError(f"Method '{cfg.method}' is not supported, "
                              f"the list of support methods is {list(CACHE_METHOD)}.")
        for name in ("blocks_count", "steps_count", "step_interval"):
            if getattr(cfg, name) <= 0:
                raise ConfigError(f"The '{name}' in config must > 0, but got {getattr(cfg, name)}.")
        for name in ("step_start", "block_start"):
            if getattr(cfg, name) < 0:
                raise ConfigError(f"The '{name}' in config must >= 0, but got {getattr(cfg, name)}.")
        if cfg.step_end < cfg.step_start:
            raise ConfigError(f"The 'step_end' must >= 'step_start', but got {cfg.step_end} and {cfg.step_start}.")
        if cfg.block_end < cfg.block_start:
            raise ConfigError(f"The 'block_end' must >= 'block_start', but got {cfg.block_end} and {cfg.block_start}.")
        if cfg.step_interval == 1:
            logger.debug("'step_interval' is 1, do not apply cache function.")
