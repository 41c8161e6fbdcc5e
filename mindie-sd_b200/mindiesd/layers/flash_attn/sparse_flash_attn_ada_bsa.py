"""Adaptive block-sparse attention: a cumulative-mass block estimate followed by attention over the
kept blocks (mindiesd/layers/flash_attn/sparse_flash_attn_ada_bsa.py:14-77 of MindIE-SD).  No token
permutation is involved: the mask is estimated from q and k as they are."""
from ...layers import _custom_ops as ops


def get_estimate_mask(query, key, value, scale=None, head_num=None, is_causal=False, input_layout="BNSD",
                      actual_seq_lengths=None, actual_seq_lengths_kv=None, keep_sink=True, keep_recent=True,
                      sparsity=0.0, cdf_threshold=1.0, sparse_size=128, stride=8):
    """Returns (int8 mask [B, N, blocks, blocks rounded up to 32], int32 kept count [B, N, blocks])."""
    return ops.sparse_block_estimate(
        query, key, actual_seq_lengths=None, actual_seq_lengths_kv=None, input_layout=input_layout, stride=stride,
        sparse_size=sparse_size, num_heads=head_num, num_key_value_heads=head_num, scale_value=scale / stride,
        threshold=cdf_threshold, causal=is_causal, keep_sink=keep_sink, keep_recent=keep_recent,
        row_sparse=1.0 - sparsity)


def ada_block_sparse_attention(query, key, value, smask, sct, scale=None, head_num=None, is_causal=False,
                               input_layout="BNSD", actual_seq_lengths=None, actual_seq_lengths_kv=None,
                               sparse_size=128):
    return ops.ada_block_sparse_attention(
        query, key, value, num_heads=head_num, num_key_value_heads=head_num, input_layout=input_layout,
        scale_value=scale, causal=is_causal, sparse_size=sparse_size, sparse_mask=smask, sparse_count_table=sct)
