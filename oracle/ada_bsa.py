"""Adaptive block-sparse attention (ada_bsa) restated on CPU with numpy.  Test infrastructure only.

The reference implements the estimator and the attention as closed NPU kernels
(csrc/ops/sparse_block_estimate, csrc/ops/ada_block_sparse_attention); what pins their results are
the numpy goldens of its plugin tests, which this file restates:
`sparse_estimate_cpu` (tests/plugin/test_sparseblockestimate.py:49-145, both branches) and
`ada_block_sparse_attention_cpu` (tests/plugin/test_adablocksparseattention.py:35-87, identical to
the block-sparse golden restated in oracle/attention.py when causal is off).

Precision of the estimator golden.  It divides the fp32 queries by the numpy scalar
`np.sqrt(dim) * stride`; from numpy 2 on that promotes everything downstream to float64, while the
sorted copy used for the running sum is cast to float32.  The final comparison `row >= guard` then
sets float64 scores against a float32-rounded guard, so the block that defines the guard survives
only when its score rounded down.  `select_blocks(..., golden_rounding=True)` reproduces that (it
is what the committed fixture, produced with numpy 2.3, contains); the default keeps the guard
block, which is what the comparison does when scores and guard have one precision (numpy 1.x, and
any fp32 implementation).
"""
from __future__ import annotations

import math

import numpy as np


def strided_scores(q, k, scale_value, stride=8):
    """Pooled logits of one head (test_sparseblockestimate.py:62-87).

    q, k: fp32 [S, D].  Tokens are grouped `stride` at a time (zero padded); group g of q is
    matched with group h of k along the anti-diagonal of the stride x stride cell:
    p[g, h] = scale_value * sum_i q[stride*g + stride-1-i] . k[stride*h + i].
    The golden writes the scale as 1 / (sqrt(D) * stride); the operator takes it as an argument.
    """
    s, d = q.shape
    groups = math.ceil(s / stride)
    pad = groups * stride - s
    if pad:
        z = np.zeros((pad, d), dtype=np.float32)
        q = np.concatenate([q, z], 0)
        k = np.concatenate([k, z], 0)
    qg = q.reshape(groups, stride, d)[:, ::-1, :].reshape(groups, stride * d)
    kg = k.reshape(groups, stride * d)
    return (qg.astype(np.float64) * scale_value) @ kg.T.astype(np.float64)


def block_scores(q, k, scale_value, block=128, stride=8):
    """Softmax mass of every (q block, k block) pair of one head (test_sparseblockestimate.py:88-124):
    row softmax of the pooled logits over all key groups, summed over the block/stride columns of a
    key block and then over the block/stride rows of a query block.  float64 [blocks, blocks]."""
    reduce_size = block // stride
    p = strided_scores(q, k, scale_value, stride)
    p = np.exp(p - p.max(-1, keepdims=True))
    p = p / p.sum(-1, keepdims=True)
    groups = p.shape[0]
    blocks = math.ceil(groups / reduce_size)
    pad = blocks * reduce_size - groups
    if pad:
        p = np.pad(p, ((0, pad), (0, pad)))
    return p.reshape(blocks, reduce_size, blocks, reduce_size).sum(axis=(1, 3))


def select_blocks(scores, threshold, row_sparse=1.0, keep_sink=True, keep_recent=True, golden_rounding=False):
    """The per-row decision of the golden (test_sparseblockestimate.py:129-143).

    The last block's mass is cleared, the row is sorted in descending order, and the smallest
    prefix whose running sum reaches `threshold` of the total is kept (at most row_sparse of the
    row); every block at least as heavy as the last kept one stays (ties included), and the first
    and last blocks always stay.  The golden has no switch for the last two; with a flag off the
    block competes with its own mass.  Returns (bool mask [rows, cols], kept count per row)."""
    rows, cols = scores.shape
    mask = np.zeros((rows, cols), dtype=bool)
    for i in range(rows):
        row = np.array(scores[i], dtype=np.float64)
        if keep_recent:
            row[-1] = 0
        order = (-np.sort(-row)).astype(np.float32)
        cnt = int((order.cumsum(dtype=np.float32) < np.float32(threshold) * order.sum(dtype=np.float32)).sum()) + 1
        if row_sparse > 0 and cnt > row_sparse * cols:
            cnt = int(row_sparse * cols)
        cnt = max(1, min(cnt, cols))
        guard = order[cnt - 1]
        keep = (row if golden_rounding else row.astype(np.float32)) >= guard
        if keep_sink:
            keep[0] = True
        if keep_recent:
            keep[-1] = True
        mask[i] = keep
    return mask, mask.sum(-1).astype(np.int32)


def block_scores_causal(q, k, scale_value, block=128, stride=8, rows_per_chunk=128):
    """The causal branch of the golden (test_sparseblockestimate.py:62-124 with causal=True): the
    queries are taken in chunks of rows_per_chunk * stride tokens (the golden's M = 128 query groups);
    the groups of a chunk take their softmax over the key groups that end before the chunk's last token
    (a trailing partial group of keys is dropped, :73-76) -- NOT token-level causality --, and the
    probabilities are summed per block as in the other branch.  Returns (float64 [blocks, blocks] with
    zeros beyond what a chunk sees, int [blocks]: how many key blocks each query block's chunk sees)."""
    s, d = q.shape
    reduce_size = block // stride
    blocks = math.ceil(s / block)
    out = np.zeros((blocks, blocks), dtype=np.float64)
    seen = np.zeros(blocks, dtype=np.int64)
    chunk_tokens = rows_per_chunk * stride
    for c0 in range(0, s, chunk_tokens):
        m = min(chunk_tokens, s - c0)
        qc = q[c0:c0 + m]
        if m % stride:
            qc = np.concatenate([qc, np.zeros((stride - m % stride, d), dtype=np.float32)], 0)
        groups_q = qc.shape[0] // stride
        qg = qc.reshape(groups_q, stride, d)[:, ::-1, :].reshape(groups_q, stride * d)
        kseq = (c0 + m) // stride * stride
        kg = k[:kseq].reshape(kseq // stride, stride * d)
        p = (qg.astype(np.float64) * scale_value) @ kg.T.astype(np.float64)
        p = np.exp(p - p.max(-1, keepdims=True))
        p = p / p.sum(-1, keepdims=True)
        pad_c = (-p.shape[1]) % reduce_size
        pad_r = (-p.shape[0]) % reduce_size
        p = np.pad(p, ((0, pad_r), (0, pad_c)))
        r = p.reshape(p.shape[0] // reduce_size, reduce_size, p.shape[1] // reduce_size, reduce_size).sum(axis=(1, 3))
        qb0 = c0 // block
        out[qb0:qb0 + r.shape[0], :r.shape[1]] = r[:blocks - qb0]
        seen[qb0:qb0 + r.shape[0]] = r.shape[1]
    return out, seen


def select_blocks_causal(scores, seen, threshold, row_sparse=1.0, golden_rounding=False):
    """The per-row decision of the golden's causal branch (test_sparseblockestimate.py:127-143): rows 0
    and 1 keep every block up to their own; row i ranks the blocks 0..i with its own block's mass cleared,
    keeps the prefix reaching `threshold` of the total (at most int(row_sparse * (i + 1)) blocks) with
    ties, and always the first block; its own block stays only if the guard is 0.  "Blocks 0..i" are cut
    to the seen[i] key blocks the row's chunk saw (the golden slices an array that holds only those), so for
    a sequence whose trailing partial key group was dropped the cleared "own" block is the last one seen."""
    rows = scores.shape[0]
    mask = np.zeros(scores.shape, dtype=bool)
    for i in range(rows):
        if i <= 1:
            mask[i, :i + 1] = True
            continue
        n = min(i + 1, int(seen[i]))
        row = np.array(scores[i, :n], dtype=np.float64)
        row[-1] = 0
        order = (-np.sort(-row)).astype(np.float32)
        cnt = int((order.cumsum(dtype=np.float32) < np.float32(threshold) * order.sum(dtype=np.float32)).sum()) + 1
        if row_sparse > 0 and cnt > row_sparse * len(row):
            cnt = int(row_sparse * len(row))
        cnt = max(1, min(cnt, len(row)))
        guard = order[cnt - 1]
        keep = (row if golden_rounding else row.astype(np.float32)) >= guard
        keep[0] = True
        mask[i, :n] = keep
    return mask, mask.sum(-1).astype(np.int32)


def sparse_block_estimate(query, key, scale_value, threshold, row_sparse=1.0, block=128, stride=8,
                          keep_sink=True, keep_recent=True, golden_rounding=False, causal=False):
    """`sparse_estimate_cpu` for BNSD fp32 arrays [B, N, S, D] (key may have fewer heads).
    Returns (bool mask [B, N, blocks, blocks], int32 counts [B, N, blocks], float64 scores)."""
    b, n, s, _ = query.shape
    group = n // key.shape[1]
    blocks = math.ceil(s / block)
    mask = np.zeros((b, n, blocks, blocks), dtype=bool)
    count = np.zeros((b, n, blocks), dtype=np.int32)
    score = np.zeros((b, n, blocks, blocks), dtype=np.float64)
    for bi in range(b):
        for ni in range(n):
            if causal:
                sc, seen = block_scores_causal(query[bi, ni], key[bi, ni // group], scale_value, block, stride)
                mask[bi, ni], count[bi, ni] = select_blocks_causal(sc, seen, threshold, row_sparse, golden_rounding)
            else:
                sc = block_scores(query[bi, ni], key[bi, ni // group], scale_value, block, stride)
                mask[bi, ni], count[bi, ni] = select_blocks(sc, threshold, row_sparse, keep_sink, keep_recent,
                                                             golden_rounding)
            score[bi, ni] = sc
    return mask, count, score
