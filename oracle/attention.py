"""Dense and block-sparse attention oracles (CPU, torch/numpy).  Test infrastructure only."""
from __future__ import annotations

import math

import numpy as np
import torch


def attention_math(query, key, value, attn_mask=None, scale=None, head_first=False):
    """Restates `attention_math`, mindiesd/layers/flash_attn/attention_func.py:32-55.

    q is scaled in the input dtype, q k^T is taken in the input dtype, the softmax runs in fp32,
    the probabilities are cast back to the input dtype before the product with v.  A boolean mask
    (True = keep), 2-D or 4-D, becomes an additive -inf bias.
    """
    if scale is None:
        scale = query.shape[-1] ** -0.5
    if not head_first:
        query, key, value = (x.transpose(1, 2) for x in (query, key, value))
    dtype = query.dtype
    sq, skv = query.size(-2), key.size(-2)
    scores = ((query * scale) @ key.transpose(-2, -1)).to(torch.float32)
    if attn_mask is not None:
        if attn_mask.dim() not in (2, 4) or attn_mask.size(-2) != sq or attn_mask.size(-1) != skv:
            raise ValueError("attn_mask must be [q, kv] or [b, n, q, kv]")
        bias = torch.zeros(sq, skv, dtype=dtype)
        bias.masked_fill_(attn_mask.logical_not(), float("-inf"))
        scores = scores + bias
    probs = torch.softmax(scores, dim=-1).to(dtype)
    out = probs @ value
    if not head_first:
        out = out.transpose(1, 2)
    return out


def attention_math_chunked(query, key, value, scale=None, head_first=False, rows=4096, q_rows=None):
    """`attention_math` evaluated per head and per chunk of query rows (identical arithmetic per
    row, bounded memory).  `q_rows` optionally restricts the evaluation to a slice of query rows;
    the result then has only those rows."""
    if not head_first:
        query, key, value = (x.transpose(1, 2) for x in (query, key, value))
    b, n, sq, d = query.shape
    if scale is None:
        scale = d ** -0.5
    sel = range(sq)[q_rows] if q_rows is not None else range(sq)
    lo, hi = sel.start, sel.stop
    out = torch.empty(b, n, hi - lo, d, dtype=query.dtype)
    for bi in range(b):
        for ni in range(n):
            k = key[bi, ni % key.shape[1] if key.shape[1] == n else ni // (n // key.shape[1])]
            v = value[bi, ni % value.shape[1] if value.shape[1] == n else ni // (n // value.shape[1])]
            for r0 in range(lo, hi, rows):
                r1 = min(hi, r0 + rows)
                q = query[bi, ni, r0:r1] * scale
                s = (q @ k.transpose(0, 1)).to(torch.float32)
                p = torch.softmax(s, dim=-1).to(query.dtype)
                out[bi, ni, r0 - lo:r1 - lo] = p @ v
    if not head_first:
        out = out.transpose(1, 2)
    return out


def block_sparse_attention(query, key, value, block_mask, block=128, scale=None, q_blocks=None):
    """Restates `block_sparse_attention_cpu`, tests/plugin/test_block_sparse_attention.py:32-65.

    BNSD inputs; block_mask int8 [B, N, q_blocks, kv_blocks], 1 = attend.  Each q block attends to
    the keys of its kept blocks only; fp32 arithmetic; a row that keeps nothing yields zeros.
    Returns fp32 [B, N, S, D].  `q_blocks` restricts the evaluation to those query blocks (the other
    rows of the result stay zero): the same arithmetic per block at a bounded cost.
    """
    b, nq, s, d = query.shape
    nkv = key.shape[1]
    skv = key.shape[2]
    group = nq // nkv
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    qf = query.float().numpy()
    kf = key.float().numpy()
    vf = value.float().numpy()
    m = np.asarray(block_mask)
    out = np.zeros((b, nq, s, d), dtype=np.float32)
    qblocks = math.ceil(s / block)
    kblocks = math.ceil(skv / block)
    for bi in range(b):
        for ni in range(nq):
            for qb in (range(qblocks) if q_blocks is None else q_blocks):
                keep = np.repeat(m[bi, ni, qb, :kblocks], block)[:skv].astype(bool)
                r0, r1 = qb * block, min((qb + 1) * block, s)
                if not keep.any():
                    continue
                kk = kf[bi, ni // group][keep]
                vv = vf[bi, ni // group][keep]
                p = (qf[bi, ni, r0:r1] @ kk.T) * np.float32(scale)
                p = p - p.max(axis=-1, keepdims=True)
                e = np.exp(p)
                out[bi, ni, r0:r1] = (e / (e.sum(axis=-1, keepdims=True) + 1e-12)) @ vv
    return torch.from_numpy(out)


def ref_compare(golden, actual, err):
    """Restates `ref_compare`, tests/plugin/test_block_sparse_attention.py:68-74."""
    golden = golden.to(torch.float32)
    bound = torch.clamp(torch.abs(golden), min=1)
    abs_error = torch.abs(actual.to(torch.float32) - golden)
    eb = torch.mean(abs_error / bound)
    ok = bool((abs_error <= err * bound).all()) and bool(eb <= err / 2)
    return eb.item(), ok, abs_error.max().item()
