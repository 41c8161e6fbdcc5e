"""`AttentionParam`: the shape key of one attention call (mindiesd/layers/flash_attn/common.py:20-61
of MindIE-SD).  The reference uses it to cache the operator its runtime search picked; here there
is one kernel, so it only carries the validated shape.  `lru_cache_by_attn_param` and `attn_cache` (:20-42 there)
are kept for callers that memoise their own per-shape decisions with them."""
import functools
from collections import OrderedDict
from dataclasses import dataclass

import torch

# One process-wide table, most recently used last; keys are AttentionParam.to_hash().
attn_cache = OrderedDict()


def lru_cache_by_attn_param(maxsize=None):
    """Decorator for functions whose first argument is an AttentionParam: the result is remembered per shape in
    `attn_cache`; with `maxsize` the least recently used shapes are dropped once the table grows beyond it."""
    def decorate(fn):
        @functools.wraps(fn)
        def remembered(attn_param, *args, **kwargs):
            key = attn_param.to_hash()
            try:
                value = attn_cache[key]
            except KeyError:
                value = attn_cache[key] = fn(attn_param, *args, **kwargs)
                while maxsize is not None and len(attn_cache) > maxsize:
                    attn_cache.popitem(last=False)
            else:
                attn_cache.move_to_end(key)
            return value
        return remembered
    return decorate


@dataclass(frozen=True)
class AttentionParam:
    batch_size: int
    head_num: int
    head_dim: int
    q_seqlen: int
    kv_seqlen: int
    dtype: torch.dtype
    head_first: bool = False

    def to_str(self) -> str:
        return (f"batch_size={self.batch_size}, head_num={self.head_num}, head_dim={self.head_dim}, "
                f"q_seqlen={self.q_seqlen}, kv_seqlen={self.kv_seqlen}, dtype={self.dtype}, "
                f"head_first={self.head_first}")

    def to_hash(self) -> int:
        return hash(self.to_str())
