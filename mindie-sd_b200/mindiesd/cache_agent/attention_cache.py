"""`AttentionCache` (mindiesd/cache_agent/attention_cache.py:17-35 of MindIE-SD): between
`step_start` and `step_end` the attention of a block is computed only on every `step_interval`-th
step and the kept output is returned on the steps in between."""
from ..utils.exception import logger
from .cache import CacheBase, CacheConfig


class AttentionCache(CacheBase):
    def __init__(self, config: CacheConfig):
        super().__init__(config)
        self._cache = [None] * config.blocks_count

    def apply_imp(self, func, *args, **kwargs):
        cfg, step, block = self._config, self._cur_step, self._cur_block
        reuse = cfg.step_start < step <= cfg.step_end and (step - cfg.step_start) % cfg.step_interval != 0
        if reuse:
            logger.debug("[AttentionCache] step: %d block: %d reuse cache.", step, block)
            return self._cache[block]
        out = func(*args, **kwargs)
        if cfg.step_start <= step < cfg.step_end:
            self._cache[block] = out
            logger.debug("[AttentionCache] step: %d block: %d update cache.", step, block)
        return out

    def _release(self):
        self._cache = [None] * self._config.blocks_count


class BlockMaskCache(CacheBase):
    """The same schedule applied to the RainFusion block mask instead of the attention output: on the
    steps in between, `bsa_sparse_attention_v3` is called with the kept mask as `cached_mask`, which
    skips the mask builder (the use the reference describes at sparse_flash_attn_rf_v3.py:212).
    `func(cached_mask=...)` must return (out, mask)."""

    def __init__(self, config: CacheConfig):
        super().__init__(config)
        self._masks = [None] * config.blocks_count

    def apply_imp(self, func, *args, **kwargs):
        cfg, step, block = self._config, self._cur_step, self._cur_block
        reuse = cfg.step_start < step <= cfg.step_end and (step - cfg.step_start) % cfg.step_interval != 0
        kept = self._masks[block] if reuse else None
        out, mask = func(*args, cached_mask=kept, **kwargs)
        if kept is None and cfg.step_start <= step < cfg.step_end:
            self._masks[block] = mask
        return out

    def _release(self):
        self._masks = [None] * self._config.blocks_count
