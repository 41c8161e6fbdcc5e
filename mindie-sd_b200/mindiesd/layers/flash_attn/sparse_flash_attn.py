"""`sparse_attention`: the sparse attention entry of the layer API
(mindiesd/layers/flash_attn/sparse_flash_attn.py:29-183 of MindIE-SD)."""
from typing import Optional

import torch

from .sparse_flash_attn_ada_bsa import ada_block_sparse_attention, get_estimate_mask
from .sparse_flash_attn_rf_v2 import rain_fusion_attention
from .sparse_flash_attn_rf_v3 import bsa_sparse_attention_v3, do_tensor_rearrange_only, permuted_block_sparse_attention
from ...utils.exception import ParametersInvalid
from ...utils.status import checked

MAX_TOKEN = 2147483647


def check_params(input_layout, sparse_type):
    if input_layout not in ["BSND", "BNSD"]:
        raise ParametersInvalid(f"The input_layout must in ['BSND', 'BNSD'], but got {input_layout}.")
    if sparse_type not in [None, "rf_v2", "rf_v3", "ada_bsa"]:
        raise ParametersInvalid(f"sparse_type must be None, 'rf_v2', 'rf_v3' or 'ada_bsa', but got {sparse_type}.")


def sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attn_mask: Optional[torch.Tensor] = None,
                     scale: Optional[float] = None, is_causal: Optional[bool] = False, head_num: int = 1,
                     input_layout: str = "BNSD", inner_precise: int = 0, sparse_type: Optional[str] = None,
                     txt_len: int = 0, block_size: int = 128, latent_shape_q: Optional[list] = None,
                     latent_shape_k: Optional[list] = None, keep_sink: Optional[bool] = True,
                     keep_recent: Optional[bool] = True, cdf_threshold: float = 1.0, sparsity: float = 0.0, **kwargs):
    check_params(input_layout, sparse_type)
    batch, head_dim = q.shape[0], q.shape[-1]
    scale = head_dim ** -0.5 if scale is None else scale

    if sparse_type == "rf_v2":
        grid = list(latent_shape_q)
        # Compacted block lists straight from the un-permuted q and k.
        _, select_idx, select_num_idx = torch.ops.mindiesd.rf_block_mask(
            q, k, grid, int(txt_len), float(sparsity), float(scale), int(block_size), input_layout, True, -1, True)
        if q.dtype in (torch.bfloat16, torch.float16) and k.shape == q.shape and block_size == 128:
            out = permuted_block_sparse_attention(q, k, v, grid, txt_len, scale, input_layout, select_idx=select_idx,
                                                  select_num_idx=select_num_idx,
                                                  fuse_loads=bool(kwargs.get("fuse_loads", False)))
            return checked(out, "sparse_attention")
        q_rf, k_rf, v_rf = do_tensor_rearrange_only(q, k, v, txt_len, latent_shape_q, latent_shape_k, input_layout)
        if input_layout == "BSND":
            q_seq, kv_seq = q_rf.shape[1], k_rf.shape[1]
            layout = "TND"
            q_rf, k_rf, v_rf = (x.reshape(-1, x.shape[2], head_dim) for x in (q_rf, k_rf, v_rf))
        else:
            q_seq, kv_seq = q_rf.shape[2], k_rf.shape[2]
            layout = input_layout
        out = rain_fusion_attention(q_rf, k_rf, v_rf, scale=scale, head_num=head_num, input_layout=layout,
                                    select_idx=select_idx, select_num_idx=select_num_idx,
                                    blockshape=[block_size, block_size], actual_seq_lengths=[q_seq] * batch,
                                    actual_seq_lengths_kv=[kv_seq] * batch, inner_precise=inner_precise)
        if layout == "TND":
            out = out.reshape(batch, q_seq, -1, head_dim)
        out = torch.ops.mindiesd.rf_rearrange(out, grid, int(txt_len), input_layout, True)
    elif sparse_type == "rf_v3":
        out, _ = bsa_sparse_attention_v3(q, k, v, latent_shape_q=latent_shape_q, latent_shape_k=latent_shape_k,
                                         txt_len=txt_len, pool_size=block_size, sparsity=sparsity,
                                         input_layout=input_layout, head_num=head_num, scale=scale,
                                         inner_precise=inner_precise, fuse_loads=bool(kwargs.get("fuse_loads", False)))
    elif sparse_type == "ada_bsa":
        smask, sct = get_estimate_mask(q, k, v, scale=scale, head_num=head_num, is_causal=is_causal,
                                       input_layout=input_layout, keep_sink=keep_sink, keep_recent=keep_recent,
                                       sparsity=sparsity, cdf_threshold=cdf_threshold, sparse_size=block_size)
        out = ada_block_sparse_attention(q, k, v, smask, sct, scale=scale, head_num=head_num, is_causal=is_causal,
                                         input_layout=input_layout, sparse_size=block_size)
    else:
        out = torch.ops.mindiesd.attention_fwd(q, k, v, float(scale), input_layout == "BNSD")
    return checked(out, "sparse_attention")
