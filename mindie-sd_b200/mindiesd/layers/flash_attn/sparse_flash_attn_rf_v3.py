"""RainFusion v3: block-sparse attention from an int8 block mask, with mask reuse across steps
(mindiesd/layers/flash_attn/sparse_flash_attn_rf_v3.py:22-295 of MindIE-SD)."""
import torch

from .. import _custom_ops as ops
from ...utils.exception import ParametersInvalid


def _bsa_inv_rearrange(out, tq, hq, wq, input_layout="BSND"):
    """Back from window order to (t, h, w) raster order (no text tokens)."""
    return torch.ops.mindiesd.rf_rearrange(out, [tq, hq, wq], 0, input_layout, True)


def do_tensor_rearrange_only(q, k, v, txt_len, latent_shape_q, latent_shape_k, input_layout):
    """Window permutation of q, k, v without pooling: what a step with a cached mask needs."""
    grid = list(latent_shape_q)
    return tuple(torch.ops.mindiesd.rf_rearrange(x, grid, int(txt_len), input_layout, False) for x in (q, k, v))


def permutation_fuses(latent_shape, txt_len, dtype) -> bool:
    """Whether the attention kernel can fetch the window order from un-permuted q, k, v (eight consecutive
    positions of the permuted order are then eight consecutive tokens of the original one): the grid width
    and the text length are multiples of 8 and the operands are two-byte floats."""
    return latent_shape[2] % 8 == 0 and int(txt_len) % 8 == 0 and dtype in (torch.bfloat16, torch.float16)


_PAIR_TABLES = {}  # (data_ptr, version, shape, device) of a reused block mask -> its pairing table


def pairing_table_of(mask):
    """The query-block pairing table of a block mask that is being REUSED (`cached_mask`): built the first time the
    mask comes back and kept while the same, unmodified tensor keeps coming back.  Building it costs about what it
    saves in one attention launch, so a mask used once never gets one."""
    key = (mask.data_ptr(), mask._version, tuple(mask.shape), mask.device)
    table = _PAIR_TABLES.get(key)
    if table is None:
        if len(_PAIR_TABLES) >= 8:
            _PAIR_TABLES.pop(next(iter(_PAIR_TABLES)))
        table = _PAIR_TABLES[key] = torch.ops.mindiesd.rf_pair_blocks(mask)
    return table


def permuted_block_sparse_attention(q, k, v, grid, txt_len, scale, input_layout, mask=None, select_idx=None,
                                    select_num_idx=None, fuse_loads=False, q_pairs=None):
    """Block-sparse attention in the window order of `grid` on q, k, v given in their ORIGINAL order; the
    result is in the original order too.  The kernel's epilogue writes every output row straight to its
    original position, so the inverse permutation of the reference's pipeline costs nothing.  q, k and v
    are permuted by one gather each -- or, with fuse_loads (and a grid `permutation_fuses` accepts), fetched
    in window order by the kernel's own loads, which saves the three gathers but makes every 128-token tile
    32 small copies instead of 2 large ones: at the 21x45x80 grid that is slower, hence off by default."""
    grid = list(grid)
    if fuse_loads and permutation_fuses(grid, txt_len, q.dtype) and k.shape == q.shape:
        return torch.ops.mindiesd.rf_sparse_attention(q, k, v, mask, select_idx, select_num_idx, grid, int(txt_len),
                                                      float(scale), input_layout, False)
    q_, k_, v_ = (torch.ops.mindiesd.rf_rearrange(x, grid, int(txt_len), input_layout, False) for x in (q, k, v))
    return torch.ops.mindiesd.rf_sparse_attention(q_, k_, v_, mask, select_idx, select_num_idx, grid, int(txt_len),
                                                  float(scale), input_layout, True, q_pairs)


def rain_fusion_attention_v3(query, key, value, block_sparse_mask, scale=None, head_num=None,
                             num_key_value_heads=None, input_layout="BNSD", actual_seq_lengths=None,
                             actual_seq_lengths_kv=None, sparse_size=128, inner_precise=4):
    """softmax(scale q k^T over the kept 128x128 blocks) v.  The operator takes BNSD; a BSND input
    is passed as a transposed view (the kernel reads through strides, so nothing is copied)."""
    if scale is None:
        scale = query.shape[-1] ** -0.5
    if num_key_value_heads is None:
        num_key_value_heads = head_num
    if input_layout not in ("BNSD", "BSND"):
        raise ParametersInvalid(f"The input_layout must in ['BSND', 'BNSD'], but got {input_layout}.")
    permuted = input_layout == "BSND"
    if permuted:
        query, key, value = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    out, _ = ops.block_sparse_attention(
        query, key, value, block_sparse_mask=block_sparse_mask, block_shape=[sparse_size, sparse_size],
        q_input_layout="BNSD", kv_input_layout="BNSD", num_key_value_heads=num_key_value_heads or 1,
        scale_value=scale, inner_precise=inner_precise, actual_seq_lengths=actual_seq_lengths,
        actual_seq_lengths_kv=actual_seq_lengths_kv, softmax_lse_flag=0)
    return out.transpose(1, 2) if permuted else out


def bsa_sparse_attention_v3(q, k, v, latent_shape_q, latent_shape_k=None, txt_len=0, pool_size=128, sparsity=0.5,
                            input_layout="BSND", head_num=None, num_key_value_heads=None, scale=None,
                            inner_precise=4, cached_mask=None, protect_first_frame=True, temporal_band=-1,
                            fuse_loads=False):
    """rearrange -> mask -> block-sparse attention -> inverse rearrange.  Returns (out, mask); pass
    the mask back as `cached_mask` on later steps to skip the mask builder.  `temporal_band` >= 0
    additionally keeps block pairs whose frames lie within that distance (not in the reference)."""
    if latent_shape_k is None:
        latent_shape_k = latent_shape_q
    if head_num is None:
        head_num = q.shape[1] if input_layout == "BNSD" else q.shape[2]
    if scale is None:
        scale = float(q.shape[-1]) ** -0.5
    grid = list(latent_shape_q)
    if cached_mask is None:
        # One fused launch pair on the un-permuted q and k: the permutation is index arithmetic.
        new_mask, _, _ = torch.ops.mindiesd.rf_block_mask(
            q, k, grid, int(txt_len), float(sparsity), float(scale), int(pool_size), input_layout,
            bool(protect_first_frame), int(temporal_band), False)
    else:
        new_mask = cached_mask
    if q.dtype in (torch.bfloat16, torch.float16) and k.shape == q.shape and pool_size == 128:
        # A mask that comes back from an earlier step brings its pairing table with it (query blocks that share a
        # thread block chosen by the overlap of their key lists: same output, fewer steps in the kernel).
        reused = cached_mask is not None and not fuse_loads and new_mask.is_cuda and new_mask.dtype == torch.int8 \
            and 16 <= new_mask.shape[2] <= 1024 and new_mask.shape[3] <= 1024 and new_mask.stride(3) == 1
        out = permuted_block_sparse_attention(q, k, v, grid, txt_len, scale, input_layout, mask=new_mask,
                                              fuse_loads=fuse_loads, q_pairs=pairing_table_of(new_mask) if reused else None)
        return out, new_mask
    q_, k_, v_ = do_tensor_rearrange_only(q, k, v, txt_len, latent_shape_q, latent_shape_k, input_layout)
    s_dim = 2 if input_layout == "BNSD" else 1
    lens = [q_.shape[s_dim]] * q_.shape[0]
    out = rain_fusion_attention_v3(q_, k_, v_, new_mask, scale=scale, head_num=head_num,
                                   num_key_value_heads=num_key_value_heads, input_layout=input_layout,
                                   actual_seq_lengths=lens, actual_seq_lengths_kv=lens, sparse_size=pool_size,
                                   inner_precise=inner_precise)
    out = torch.ops.mindiesd.rf_rearrange(out, grid, int(txt_len), input_layout, True)
    return out, new_mask
