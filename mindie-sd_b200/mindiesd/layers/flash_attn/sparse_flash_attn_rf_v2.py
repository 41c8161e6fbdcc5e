"""RainFusion v2 host logic on CUDA kernels.

Every public name of mindiesd/layers/flash_attn/sparse_flash_attn_rf_v2.py (MindIE-SD) is kept with
its signature: `avgpool` (:24-73), `get_mask_index` (:76-91), `get_blockwise_mask` (:94-134),
`rearrange_with_remaining` (:137-196), `inv_rearrange_with_remaining` (:199-289),
`do_tensor_rearrange_pooling` (:292-317), `do_tensor_inv_rearrange` (:321-337),
`do_tensor_pooling` (:340-348), `rain_fusion_attention` (:351-381).  Where the reference chains a
dozen eager torch operators, each function here is one kernel launch; `sparse_attention` does not
go through these helpers one by one but uses the fused mask builder.
"""
import math

import torch

from .. import _custom_ops as ops
from ...utils.exception import ParametersInvalid


def _check_layout(input_layout):
    if input_layout not in ("BNSD", "BSND"):
        raise ParametersInvalid(f"The input_layout must in ['BSND', 'BNSD'], but got {input_layout}.")


class PooledTensor(torch.Tensor):
    """A pooled q/k/v stack as `do_tensor_rearrange_pooling` returns it, carrying the exact fp32
    means next to the values rounded to the input dtype, so that `get_blockwise_mask` thresholds on
    the unrounded scores."""

    @staticmethod
    def wrap(rounded, exact):
        out = rounded.as_subclass(PooledTensor)
        out._exact = exact
        return out

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        # Any torch operation yields a plain tensor: the fp32 side-car only survives a direct hand-over.
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **(kwargs or {}))


def avgpool(input_tensor, pool_size=128, input_layout="BNSD"):
    """Mean over every `pool_size` consecutive tokens; the tail block over its real length.
    Returns the input layout and dtype with the token axis replaced by the block axis."""
    _check_layout(input_layout)
    pooled = torch.ops.mindiesd.rf_pool(input_tensor, [0, 0, 0], 0, pool_size, input_layout, False)
    pooled = pooled.to(input_tensor.dtype)
    return pooled if input_layout == "BNSD" else pooled.transpose(1, 2)


def get_mask_index(mask):
    """[b, n, s, s] boolean mask -> int64 [b, n, s, s]: per row the ascending indices of the True
    entries, then -1."""
    s = mask.shape[-1]
    cols = torch.arange(s, device=mask.device).expand(mask.shape)
    keyed = torch.where(mask.bool(), cols, s)
    ordered, _ = torch.sort(keyed, dim=-1)
    return torch.where(ordered < s, ordered, -1).to(torch.int64)


def get_blockwise_mask(qkv_pool, txt_len, sparsity, scale, pool_size, latent_shape_q, latent_shape_k,
                       input_layout, return_binary=False, protect_first_frame=True):
    """Block mask (int8 [B, N, qb, kb]) or compacted lists (select_idx [qb, N, kb], select_num_idx
    [qb, N], batch 0) from the pooled q/k/v stack of `do_tensor_rearrange_pooling`."""
    _check_layout(input_layout)
    exact = getattr(qkv_pool, "_exact", None)
    if exact is not None:
        q_pool, k_pool = exact
    else:
        q_pool, k_pool, _ = torch.chunk(qkv_pool, 3, dim=0)
        if input_layout == "BSND":
            q_pool, k_pool = q_pool.transpose(1, 2), k_pool.transpose(1, 2)
        q_pool, k_pool = q_pool.float().contiguous(), k_pool.float().contiguous()
    mask, sel, num = torch.ops.mindiesd.rf_mask_from_pooled(
        q_pool, k_pool, list(latent_shape_q), int(txt_len), float(sparsity), int(pool_size),
        bool(protect_first_frame), -1, not return_binary)
    if return_binary:
        return mask
    return sel, num


def rearrange_with_remaining(tensor, latent_shape_q, latent_shape_k, input_layout):
    """Tokens of a (t, h, w) grid -> 8x8 spatial windows per frame (remainder rows and columns
    appended per frame; the first frame untouched when h or w is not a multiple of 8)."""
    _check_layout(input_layout)
    return torch.ops.mindiesd.rf_rearrange(tensor, list(latent_shape_q), 0, input_layout, False)


def inv_rearrange_with_remaining(tensor, latent_shape_q, latent_shape_k, input_layout):
    _check_layout(input_layout)
    return torch.ops.mindiesd.rf_rearrange(tensor, list(latent_shape_q), 0, input_layout, True)


def do_tensor_rearrange_pooling(query, key, value, text_len, pool_size, latent_shape_q, latent_shape_k, input_layout):
    """Returns (q', k', v', pooled): the three tensors with image tokens window-permuted and text
    tokens moved to the back, and the pooled stack [3B, ...] in the input dtype and layout."""
    _check_layout(input_layout)
    grid = list(latent_shape_q)
    outs = [torch.ops.mindiesd.rf_rearrange(x, grid, int(text_len), input_layout, False) for x in (query, key, value)]
    exact = [torch.ops.mindiesd.rf_pool(x, grid, int(text_len), pool_size, input_layout, True)
             for x in (query, key, value)]
    rounded = torch.cat([p.to(query.dtype) for p in exact], dim=0)
    if input_layout == "BSND":
        rounded = rounded.transpose(1, 2)
    return outs[0], outs[1], outs[2], PooledTensor.wrap(rounded, (exact[0], exact[1]))


def do_tensor_inv_rearrange(tensor, text_len, latent_shape_q, latent_shape_k, input_layout):
    _check_layout(input_layout)
    return torch.ops.mindiesd.rf_rearrange(tensor, list(latent_shape_q), int(text_len), input_layout, True)


def do_tensor_pooling(tensor, text_len):
    """BSND tensor with `text_len` leading text tokens -> pooled [B, blocks, N, D], text and image
    pooled separately, text first."""
    parts = [avgpool(tensor[:, :text_len], 128, "BSND")] if text_len else []
    parts.append(avgpool(tensor[:, text_len:], 128, "BSND"))
    return torch.cat(parts, dim=1)


def rain_fusion_attention(query, key, value, scale=None, head_num=None, input_layout="TND", select_idx=None,
                          select_num_idx=None, blockshape=None, actual_seq_lengths=None, actual_seq_lengths_kv=None,
                          inner_precise=0):
    out, _ = ops.rain_fusion_attention(
        query, key, value, select_idx, select_num_idx, blockshape, attn_mask=None,
        actual_seq_qlen=actual_seq_lengths, actual_seq_kvlen=actual_seq_lengths_kv, block_table=None,
        q_input_layout=input_layout, kv_input_layout=input_layout, head_num=head_num, mask_type=0,
        scale=scale if scale is not None else query.shape[-1] ** -0.5, inner_precise=inner_precise, block_size=0)
    return out
