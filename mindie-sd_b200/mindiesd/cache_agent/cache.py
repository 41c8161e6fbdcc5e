"""Step/block bookkeeping shared by the caches (mindiesd/cache_agent/cache.py:17-57 of MindIE-SD).

A denoising run makes `steps_count` steps and every step calls each of the `blocks_count` DiT blocks
once, in order; `apply` is called once per (step, block) and the counters advance by themselves.
"""
from abc import ABC, abstractmethod
from dataclasses import dataclass


@dataclass
class CacheConfig:
    method: str
    blocks_count: int
    steps_count: int
    step_start: int = 0
    step_interval: int = 1
    step_end: int = 10000
    block_start: int = 0
    block_end: int = 10000


class CacheBase(ABC):
    def __init__(self, config: CacheConfig):
        super().__init__()
        self._config = config
        self._cur_step = 0
        self._cur_block = 0

    def apply(self, func, *args, **kwargs):
        result = self.apply_imp(func, *args, **kwargs)
        self._counter()
        return result

    @abstractmethod
    def apply_imp(self, func, *args, **kwargs):
        ...

    @abstractmethod
    def _release(self):
        ...

    def _counter(self):
        self._cur_block += 1
        if self._cur_block == self._config.blocks_count:  # a step is over
            self._cur_block = 0
            self._cur_step += 1
            if self._cur_step == self._config.steps_count:  # a run is over: drop what was kept
                self._cur_step = 0
                self._release()
