"""Single-process restatement of the Ulysses re-shard (docs/zh/features/parallelism.md:207-233 of
MindIE-SD): what each rank holds before and after the two all-to-alls.  Test infrastructure only."""
from __future__ import annotations

import torch


def seq_to_head(shards):
    """shards[r]: [B, S/P, N, D] (rank r's sequence shard, all heads).  Returns out[p]:
    [B, S, N/P, D] (rank p's head group over the full sequence)."""
    p = len(shards)
    return [torch.cat([s.tensor_split(p, dim=2)[r] for s in shards], dim=1) for r in range(p)]


def head_to_seq(shards):
    """Inverse: shards[p]: [B, S, N/P, D] -> out[r]: [B, S/P, N, D]."""
    p = len(shards)
    return [torch.cat([s.tensor_split(p, dim=1)[r] for s in shards], dim=2) for r in range(p)]
