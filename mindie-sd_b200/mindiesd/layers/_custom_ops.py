"""Keyword wrappers around torch.ops.mindiesd.* and their fake implementations.

The attention and estimator wrappers keep the names, argument names and defaults of
mindiesd/layers/_custom_ops.py:19-72, 124-390 of MindIE-SD.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import register_ops
from ..utils.exception import ParametersInvalid


def laser_attention(query, key, value, atten_mask=None, alibi_mask=None, drop_mask=None, scale_value=1.0,
                    head_num=2, input_layout="BNSD", keep_prob=1.0, pre_tokens=2147483647, next_tokens=1,
                    is_high_precision=True) -> Tuple[torch.Tensor, torch.Tensor]:
    return torch.ops.mindiesd.la(
        query=query, key=key, value=value, atten_mask=atten_mask, alibi_mask=alibi_mask, drop_mask=drop_mask,
        scale_value=scale_value, head_num=head_num, input_layout=input_layout, keep_prob=keep_prob,
        pre_tokens=pre_tokens, next_tokens=next_tokens, is_highPrecision=is_high_precision)


@register_ops.register_mindie_fake_op("la")
def _la_fake(query, key, value, atten_mask=None, alibi_mask=None, drop_mask=None, scale_value=1.0, head_num=2,
             input_layout="BNSD", keep_prob=1.0, pre_tokens=2147483647, next_tokens=1, is_highPrecision=True):
    lse = query.new_empty([query.shape[0], query.shape[1], query.shape[2]], dtype=torch.float32)
    return lse, query.new_empty(query.shape, dtype=torch.float32)


def rain_fusion_attention(query, key, value, select_idx, select_num_idx, blockshape: List[int], attn_mask=None,
                          actual_seq_qlen: Optional[List[int]] = None, actual_seq_kvlen: Optional[List[int]] = None,
                          block_table=None, q_input_layout="TND", kv_input_layout="TND", head_num=1, mask_type=0,
                          scale=1.0, inner_precise=1, block_size=0) -> Tuple[torch.Tensor, torch.Tensor]:
    return torch.ops.mindiesd.rainfusionattention(
        query=query, key=key, value=value, select_idx=select_idx, select_num_idx=select_num_idx,
        blockshape=blockshape, attn_mask=attn_mask, actual_seq_qlen=actual_seq_qlen,
        actual_seq_kvlen=actual_seq_kvlen, block_table=block_table, q_input_layout=q_input_layout,
        kv_input_layout=kv_input_layout, head_num=head_num, mask_type=mask_type, scale=scale,
        inner_precise=inner_precise, block_size=block_size)


@register_ops.register_mindie_fake_op("rainfusionattention")
def _rainfusion_fake(query, key, value, select_idx, select_num_idx, blockshape, attn_mask=None, actual_seq_qlen=None,
                     actual_seq_kvlen=None, block_table=None, q_input_layout="TND", kv_input_layout="TND",
                     head_num=1, mask_type=0, scale=1.0, inner_precise=1, block_size=0):
    lse = query.new_empty([query.shape[0], query.shape[1], query.shape[2]])
    return torch.empty_like(query), lse


def block_sparse_attention(query, key, value, block_sparse_mask=None, block_shape: Optional[List[int]] = None,
                           q_input_layout="BNSD", kv_input_layout="BNSD", num_key_value_heads=1, scale_value=1.0,
                           inner_precise=0, actual_seq_lengths: Optional[List[int]] = None,
                           actual_seq_lengths_kv: Optional[List[int]] = None,
                           softmax_lse_flag=0) -> Tuple[torch.Tensor, torch.Tensor]:
    kwargs = dict(query=query, key=key, value=value, block_sparse_mask=block_sparse_mask,
                  block_shape=block_shape if block_shape is not None else [128, 128],
                  q_input_layout=q_input_layout, kv_input_layout=kv_input_layout,
                  num_key_value_heads=num_key_value_heads, scale_value=scale_value, inner_precise=inner_precise,
                  softmax_lse_flag=softmax_lse_flag)
    if actual_seq_lengths is not None:
        kwargs["actual_seq_lengths"] = actual_seq_lengths
    if actual_seq_lengths_kv is not None:
        kwargs["actual_seq_lengths_kv"] = actual_seq_lengths_kv
    return torch.ops.mindiesd.block_sparse_attention(**kwargs)


@register_ops.register_mindie_fake_op("block_sparse_attention")
def _block_sparse_fake(query, key, value, block_sparse_mask=None, block_shape=None, q_input_layout="BNSD",
                       kv_input_layout="BNSD", num_key_value_heads=1, scale_value=1.0, inner_precise=0,
                       actual_seq_lengths=None, actual_seq_lengths_kv=None, softmax_lse_flag=0):
    if q_input_layout == "TND":
        shape = [query.shape[0], query.shape[1], 1]
    else:
        shape = [query.shape[0], query.shape[1], query.shape[2], 1]
    return torch.empty_like(query), query.new_empty(shape, dtype=torch.float32)


def sparse_block_estimate(query, key, actual_seq_lengths: Optional[List[int]] = None,
                          actual_seq_lengths_kv: Optional[List[int]] = None, input_layout="BNSD", stride=8,
                          sparse_size=128, num_heads=1, num_key_value_heads=1, scale_value=1.0, threshold=1.0,
                          causal=False, keep_sink=True, keep_recent=True,
                          row_sparse=1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    return torch.ops.mindiesd.sparse_block_estimate(
        query=query, key=key, actual_seq_lengths=actual_seq_lengths, actual_seq_lengths_kv=actual_seq_lengths_kv,
        input_layout=input_layout, stride=stride, sparse_size=sparse_size, num_heads=num_heads,
        num_key_value_heads=num_key_value_heads, scale_value=scale_value, threshold=threshold, causal=causal,
        keep_sink=keep_sink, keep_recent=keep_recent, row_sparse=row_sparse)


@register_ops.register_mindie_fake_op("sparse_block_estimate")
def _sparse_block_estimate_fake(query, key, actual_seq_lengths=None, actual_seq_lengths_kv=None, input_layout="BNSD",
                                stride=8, sparse_size=128, num_heads=1, num_key_value_heads=1, scale_value=1.0,
                                threshold=1.0, causal=False, keep_sink=True, keep_recent=True, row_sparse=1.0):
    if input_layout == "BNSD":
        b, nq, s, _ = query.shape
    elif input_layout == "BSND":
        b, s, nq, _ = query.shape
    elif input_layout == "BSH":
        b, s, _ = query.shape
        nq = num_heads
    else:
        raise ParametersInvalid(f"The input_layout only support 'BNSD', 'BSND' and 'BSH', but got {input_layout}")
    blocks = (s + sparse_size - 1) // sparse_size
    mask = query.new_empty([b, nq, blocks, (blocks + 31) // 32 * 32], dtype=torch.int8)
    return mask, query.new_empty([b, nq, blocks], dtype=torch.int32)


def ada_block_sparse_attention(query, key, value, sparse_mask, sparse_count_table, input_layout="BNSD",
                               sparse_size=128, num_heads=1, num_key_value_heads=1, scale_value=1.0, causal=False,
                               inner_precise=1, pre_tokens=214748647, next_tokens=214748647,
                               actual_seq_lengths: Optional[List[int]] = None,
                               actual_seq_lengths_kv: Optional[List[int]] = None) -> torch.Tensor:
    return torch.ops.mindiesd.ada_block_sparse_attention(
        query=query, key=key, value=value, sparse_mask=sparse_mask, sparse_count_table=sparse_count_table,
        input_layout=input_layout, sparse_size=sparse_size, num_heads=num_heads,
        num_key_value_heads=num_key_value_heads, scale_value=scale_value, causal=causal,
        inner_precise=inner_precise, pre_tokens=pre_tokens, next_tokens=next_tokens,
        actual_seq_lengths=actual_seq_lengths, actual_seq_lengths_kv=actual_seq_lengths_kv)


@register_ops.register_mindie_fake_op("ada_block_sparse_attention")
def _ada_block_sparse_attention_fake(query, key, value, sparse_mask, sparse_count_table, input_layout="BNSD",
                                     sparse_size=128, num_heads=1, num_key_value_heads=1, scale_value=1.0,
                                     causal=False, inner_precise=1, pre_tokens=214748647, next_tokens=214748647,
                                     actual_seq_lengths=None, actual_seq_lengths_kv=None):
    return torch.empty_like(query)


# ---- operators that replace torch_npu calls or eager torch code of the reference ---------------------

@register_ops.register_mindie_fake_op("attention_fwd")
def _attention_fwd_fake(query, key, value, scale, head_first, causal=False):
    return torch.empty_like(query)


@register_ops.register_mindie_fake_op("rf_sparse_attention")
def _rf_sparse_attention_fake(query, key, value, block_mask, select_idx, select_num_idx, latent_shape, txt_len, scale,
                              input_layout, inputs_permuted=False, q_pairs=None):
    return query.new_empty(query.shape)


@register_ops.register_mindie_fake_op("rf_pair_blocks")
def _rf_pair_blocks_fake(block_mask):
    b, n, qb, _ = block_mask.shape
    return block_mask.new_empty((b, n, (qb + 1) // 2, 2), dtype=torch.int32)


@register_ops.register_mindie_fake_op("attention_varlen_fwd")
def _attention_varlen_fwd_fake(query, key, value, cu_seqlens_q, cu_seqlens_k, scale, causal=False):
    return query.new_empty(query.shape)


@register_ops.register_mindie_fake_op("rf_rearrange")
def _rf_rearrange_fake(x, latent_shape, txt_len, input_layout, inverse):
    return x.new_empty(x.shape)


@register_ops.register_mindie_fake_op("rf_block_mask")
def _rf_block_mask_fake(query, key, latent_shape, txt_len, sparsity, scale, block_size, input_layout,
                        protect_first_frame, temporal_band, return_lists):
    t, h, w = latent_shape
    blocks = (t * h * w + 127) // 128 + (txt_len + 127) // 128
    heads = query.shape[1] if input_layout == "BNSD" else query.shape[2]
    mask = query.new_empty([query.shape[0], heads, blocks, blocks], dtype=torch.int8)
    if return_lists:
        return (mask, query.new_empty([blocks, heads, blocks], dtype=torch.int64),
                query.new_empty([blocks, heads], dtype=torch.int64))
    return mask, query.new_empty([0], dtype=torch.int64), query.new_empty([0], dtype=torch.int64)


@register_ops.register_mindie_fake_op("rf_pool")
def _rf_pool_fake(x, latent_shape, txt_len, block_size, input_layout, permute):
    n, s = (x.shape[1], x.shape[2]) if input_layout == "BNSD" else (x.shape[2], x.shape[1])
    if permute:
        t, h, w = latent_shape
        blocks = (t * h * w + 127) // 128 + (txt_len + 127) // 128
    else:
        blocks = (s + 127) // 128
    return x.new_empty([x.shape[0], n, blocks, x.shape[3]], dtype=torch.float32)


@register_ops.register_mindie_fake_op("rf_mask_from_pooled")
def _rf_mask_from_pooled_fake(q_pooled, k_pooled, latent_shape, txt_len, sparsity, block_size, protect_first_frame,
                              temporal_band, return_lists):
    b, n, blocks, _ = q_pooled.shape
    mask = q_pooled.new_empty([b, n, blocks, blocks], dtype=torch.int8)
    if return_lists:
        return (mask, q_pooled.new_empty([blocks, n, blocks], dtype=torch.int64),
                q_pooled.new_empty([blocks, n], dtype=torch.int64))
    return mask, q_pooled.new_empty([0], dtype=torch.int64), q_pooled.new_empty([0], dtype=torch.int64)


@register_ops.register_mindie_fake_op("fa_block_quant")
def _fa_block_quant_fake(x, block_size, head_first, per_channel, rotate):
    b, d = x.shape[0], x.shape[3]
    n, s = (x.shape[1], x.shape[2]) if head_first else (x.shape[2], x.shape[1])
    nscale = d if per_channel else (s + block_size - 1) // block_size
    return x.new_empty([b, n, s, d], dtype=torch.float8_e4m3fn), x.new_empty([b, n, nscale], dtype=torch.float32)


@register_ops.register_mindie_fake_op("fa_rotate_quant")
def _fa_rotate_quant_fake(x, rot, block_size, head_first):
    b, n, s, d = (x.shape[0], x.shape[1], x.shape[2], x.shape[3]) if head_first else \
        (x.shape[0], x.shape[2], x.shape[1], x.shape[3])
    return (x.new_empty([b, n, s, d], dtype=torch.float8_e4m3fn),
            x.new_empty([b, n, (s + block_size - 1) // block_size], dtype=torch.float32))


@register_ops.register_mindie_fake_op("fp8_attention")
def _fp8_attention_fake(query, key, value, q_scale, k_scale, v_scale, scale, k_block, v_block, out_dtype):
    return query.new_empty(query.shape, dtype=out_dtype)
