"""Seeded inputs shared by the fixture generator and the tests (numpy RandomState: a frozen
stream, so the committed fixtures stay reproducible)."""
import numpy as np
import torch


def randn(seed, *shape, dtype=torch.float32):
    x = torch.from_numpy(np.random.RandomState(seed).standard_normal(size=shape).astype(np.float32))
    return x.to(dtype)


def structured_qk(seed, heads, grid, dim, txt_len=0, dtype=torch.bfloat16):
    """q, k [1, heads, txt_len + t*h*w, dim]: noise plus a smooth per-head spatial/temporal term, so
    that pooled block scores are well separated."""
    t, h, w = grid
    s = t * h * w
    tt, hh, ww = np.meshgrid(np.arange(t) / t, np.arange(h) / h, np.arange(w) / w, indexing="ij")
    feats = np.stack([np.cos(2 * np.pi * tt), np.sin(2 * np.pi * hh) * np.cos(np.pi * ww), 2 * tt - 1], -1)
    feats = torch.from_numpy(feats.reshape(s, 3).astype(np.float32))
    u = randn(seed + 7, heads, 3, dim) * (1.5 / dim ** 0.5)
    bias = torch.einsum("sr,nrd->nsd", feats, u)
    out = []
    for i in range(2):
        x = 0.5 * randn(seed + i, 1, heads, txt_len + s, dim)
        x[:, :, txt_len:] += bias
        out.append(x.to(dtype))
    return out


# (name, grid, txt_len, heads, dim, sparsity, layout, seed)
MASK_CASES = [
    ("aligned", (3, 40, 80), 0, 2, 64, 0.5, "BNSD", 11),
    ("nodiv_both", (3, 30, 52), 0, 2, 64, 0.5, "BNSD", 12),
    ("nodiv_h", (2, 21, 32), 0, 2, 64, 0.75, "BSND", 13),
    ("nodiv_w", (2, 24, 45), 0, 2, 64, 0.25, "BNSD", 14),
    ("text", (3, 40, 80), 256, 2, 64, 0.5, "BNSD", 15),
    ("text_ragged", (3, 30, 52), 200, 2, 128, 0.6, "BSND", 16),
    ("dense", (2, 24, 45), 0, 1, 128, 0.0, "BNSD", 17),
    ("wan480p", (21, 30, 52), 0, 1, 128, 0.75, "BNSD", 18),
    ("wan720p", (21, 45, 80), 0, 2, 128, 0.75, "BNSD", 19),
]

PERM_GRIDS = [(3, 40, 80), (3, 30, 52), (2, 21, 32), (2, 24, 45), (4, 8, 16), (3, 12, 11), (2, 9, 16)]

# (name, grid, heads, cdf threshold, row_sparse, seed): sequence = t*h*w tokens
ESTIMATE_CASES = [
    ("aligned", (2, 32, 32), 2, 0.85, 1.0, 51),      # 2048 tokens, 16 blocks
    ("ragged_block", (1, 29, 40), 2, 0.7, 1.0, 52),  # 1160 tokens: a multiple of 8, not of 128
    ("ragged_group", (1, 13, 89), 1, 0.9, 0.5, 53),  # 1157 tokens: not a multiple of 8; row cap active
    ("two_chunks", (3, 60, 52), 1, 0.6, 1.0, 54),    # 9360 tokens: more than one 8192-token key chunk of the golden
]
