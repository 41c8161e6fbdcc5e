"""FP8 (e4m3) attention-operand quantisation restated on CPU.  Test infrastructure only.

PARITY UNPINNED for the scale formula: the reference calls the closed operator
torch_npu.npu_dynamic_block_quant (mindiesd/layers/quant/block_quant.py:43-46) whose scale rule
is not in the source tree and which no reference test checks numerically.  This restatement
uses the usual dynamic rule scale = absmax / 448.  The accuracy bar of the FP8 attention is
defined against fp32 attention of the unquantised inputs (cosine similarity), not against this.
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0


def hadamard(n=128):
    """Sylvester Hadamard matrix H[i, j] = (-1)^popcount(i & j), scaled to be orthogonal."""
    i = torch.arange(n)
    bits = (i[:, None] & i[None, :])
    pop = sum((bits >> b) & 1 for b in range(n.bit_length()))
    return (1.0 - 2.0 * (pop % 2).double()) / n ** 0.5


def block_quant(x, row_block=128, rotate=False):
    """x [B, N, S, 128] -> (e4m3 [B, N, S, 128], fp32 scales [B, N, ceil(S/row_block)]).
    rotate: every token is first multiplied by the orthogonal Hadamard matrix."""
    if rotate:
        x = (x.double() @ hadamard(x.shape[-1])).float()
    b, n, s, d = x.shape
    nb = (s + row_block - 1) // row_block
    xf = x.float()
    pad = nb * row_block - s
    if pad:
        xf = torch.nn.functional.pad(xf, (0, 0, 0, pad))
    blocks = xf.reshape(b, n, nb, row_block * d)
    amax = blocks.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (blocks * (1.0 / scale).unsqueeze(-1)).reshape(b, n, nb * row_block, d)[:, :, :s]
    return q.to(torch.float8_e4m3fn), scale


def channel_quant(x):
    """x [B, N, S, 128] -> (e4m3, fp32 scales [B, N, 128]) with one scale per channel."""
    amax = x.float().abs().amax(2)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = x.float() * (1.0 / scale).unsqueeze(2)
    return q.to(torch.float8_e4m3fn), scale


def cosine(a, b):
    a = a.double().reshape(-1)
    b = b.double().reshape(-1)
    return float((a @ b) / (a.norm() * b.norm() + 1e-30))
