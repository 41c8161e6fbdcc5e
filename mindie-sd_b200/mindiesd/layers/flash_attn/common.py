"""`AttentionParam`: the shape key of one attention call (mindiesd/layers/flash_attn/common.py:20-61
of MindIE-SD).  The reference uses it to cache the operator its runtime search picked; here there
is one kernel, so it only carries the validated shape."""
from dataclasses import dataclass

import torch


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
