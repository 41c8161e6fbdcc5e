"""RainFusion host logic restated on CPU with numpy/torch.  Test infrastructure only.

Restates mindiesd/layers/flash_attn/sparse_flash_attn_rf_v2.py: avgpool (:24-73),
get_mask_index (:76-91), get_blockwise_mask (:94-134), rearrange_with_remaining (:137-196),
inv_rearrange_with_remaining (:199-289), do_tensor_rearrange_pooling (:292-317),
do_tensor_inv_rearrange (:321-337).
"""
from __future__ import annotations

import math

import numpy as np
import torch


def window_permutation(t, h, w):
    """Index vector `src` with permuted[p] = original[src[p]] for the image tokens of a (t,h,w)
    grid (rf_v2.py:137-196).  Aligned grids (h, w multiples of 8): every frame becomes a raster
    of 8x8 windows.  Otherwise frame 0 is untouched and each later frame is laid out as windows
    of the (h - h%8) x (w - w%8) corner, then the h-remainder rows at full width, then the
    w-remainder columns of the windowed rows."""
    hw = h * w
    idx = np.arange(t * hw, dtype=np.int64).reshape(t, h, w)
    rh, rw = h % 8, w % 8
    hm, wm = h - rh, w - rw

    def windows(x):  # [f, hm, wm] -> [f, hm*wm]
        f = x.shape[0]
        return x.reshape(f, hm // 8, 8, wm // 8, 8).transpose(0, 1, 3, 2, 4).reshape(f, -1)

    if rh == 0 and rw == 0:
        return windows(idx).reshape(-1)
    first = idx[0].reshape(-1)
    rest = idx[1:]
    parts = [windows(rest[:, :hm, :wm])]
    if rh:
        parts.append(rest[:, hm:, :].reshape(t - 1, -1))
    if rw:
        parts.append(rest[:, :hm, wm:].reshape(t - 1, -1))
    return np.concatenate([first, np.concatenate(parts, axis=1).reshape(-1)])


def full_permutation(t, h, w, txt_len):
    """Source index of every position of the permuted order [image' | text] when the source order
    is [text | image] (rf_v2.py:297-311)."""
    img = window_permutation(t, h, w) + txt_len
    return np.concatenate([img, np.arange(txt_len, dtype=np.int64)])


def rearrange(x, latent_shape, txt_len=0, layout="BNSD"):
    """do_tensor_rearrange_only / the permutation half of do_tensor_rearrange_pooling."""
    src = torch.from_numpy(full_permutation(*latent_shape, txt_len))
    return x.index_select(2 if layout == "BNSD" else 1, src)


def inv_rearrange(x, latent_shape, txt_len=0, layout="BNSD"):
    """do_tensor_inv_rearrange (rf_v2.py:321-337) / _bsa_inv_rearrange (rf_v3.py:22-97)."""
    src = full_permutation(*latent_shape, txt_len)
    inv = np.empty_like(src)
    inv[src] = np.arange(src.size)
    return x.index_select(2 if layout == "BNSD" else 1, torch.from_numpy(inv))


def avgpool(x, pool_size=128, layout="BNSD"):
    """Block means along the token axis, the tail block over its real length (rf_v2.py:24-73).
    Computed in the input dtype's torch reduction, as the reference does."""
    dim = 2 if layout == "BNSD" else 1
    s = x.shape[dim]
    full = s // pool_size
    parts = []
    if full:
        body = x.narrow(dim, 0, full * pool_size)
        shape = list(x.shape)
        shape[dim:dim + 1] = [full, pool_size]
        parts.append(body.reshape(shape).mean(dim=dim + 1))
    if s % pool_size:
        parts.append(x.narrow(dim, full * pool_size, s % pool_size).mean(dim=dim, keepdim=True))
    return torch.cat(parts, dim=dim) if len(parts) > 1 else parts[0]


def pooled_means(q, k, latent_shape, txt_len=0, pool_size=128, layout="BNSD"):
    """Pooled q and k exactly as do_tensor_rearrange_pooling builds them (rf_v2.py:292-317): image
    tokens are permuted and pooled, text tokens pooled separately and appended."""
    dim = 2 if layout == "BNSD" else 1
    outs = []
    for x in (q, k):
        img = x.narrow(dim, txt_len, x.shape[dim] - txt_len)
        src = torch.from_numpy(window_permutation(*latent_shape))
        pooled = avgpool(img.index_select(dim, src), pool_size, layout)
        if txt_len:
            pooled = torch.cat([pooled, avgpool(x.narrow(dim, 0, txt_len), pool_size, layout)], dim=dim)
        outs.append(pooled)
    return outs


def keep_len_of(cols, sparsity):
    return math.ceil(cols * (1 - sparsity))


def blockwise_mask(q_pool, k_pool, txt_len, sparsity, scale, pool_size, latent_shape, layout="BNSD",
                   protect_first_frame=True, use_softmax=True):
    """get_blockwise_mask(..., return_binary=True) (rf_v2.py:94-129): block scores, softmax over
    the key blocks, threshold at the keep_len-th largest value of each row with `>=` (ties are
    kept), then text rows/columns and first-frame rows/columns forced on.  With
    use_softmax=False the threshold is taken on the raw scores in float64 (the softmax is a
    monotone map of each row, so the kept set is the same up to floating-point ties)."""
    if layout == "BSND":
        q_pool, k_pool = q_pool.transpose(1, 2), k_pool.transpose(1, 2)
    if use_softmax:
        scores = torch.softmax(torch.einsum("bnld,bnsd->bnls", q_pool, k_pool) * scale, dim=-1)
    else:
        scores = torch.einsum("bnld,bnsd->bnls", q_pool.double(), k_pool.double())
    cols = scores.shape[-1]
    keep = keep_len_of(cols, sparsity)
    thr = torch.topk(scores, k=keep, dim=-1).values[..., -1:]
    mask = scores >= thr
    tb = (txt_len + pool_size - 1) // pool_size
    if tb:
        mask[:, :, -tb:, :] = True
        mask[:, :, :, -tb:] = True
    if protect_first_frame:
        fb = (latent_shape[1] * latent_shape[2] + pool_size - 1) // pool_size
        if fb:
            mask[:, :, :fb, :] = True
            mask[:, :, :, :fb] = True
    return mask.to(torch.int8)


def temporal_band(latent_shape, txt_len, band, pool_size=128):
    """Extension that the reference does not have: bool [blocks, blocks], True where the frame
    ranges of a q block and a k block of the permuted image lie within `band` frames of each
    other.  Frames stay contiguous under the window permutation, so block i of the permuted
    image covers frames (i*128)//(h*w) .. (min((i+1)*128, t*h*w) - 1)//(h*w)."""
    t, h, w = latent_shape
    img = t * h * w
    ib = (img + pool_size - 1) // pool_size
    tb = (txt_len + pool_size - 1) // pool_size
    i = np.arange(ib)
    lo = (i * pool_size) // (h * w)
    hi = (np.minimum((i + 1) * pool_size, img) - 1) // (h * w)
    near = (lo[None, :] - band <= hi[:, None]) & (lo[:, None] - band <= hi[None, :])
    out = np.zeros((ib + tb, ib + tb), dtype=bool)
    out[:ib, :ib] = near
    return out


def mask_index(mask):
    """get_mask_index (rf_v2.py:76-91): per row the ascending ids of the kept blocks, -1 padded."""
    m = np.asarray(mask).astype(bool)
    out = np.full(m.shape, -1, dtype=np.int64)
    it = np.nonzero(m)
    counts = m.sum(-1)
    # rank of each kept entry within its row
    rank = (np.cumsum(m, axis=-1) - 1)[it]
    out[it[:-1] + (rank,)] = it[-1]
    return torch.from_numpy(out), torch.from_numpy(counts.astype(np.int64))


def select_lists(mask):
    """The (select_idx, select_num_idx) pair of get_blockwise_mask without return_binary
    (rf_v2.py:131-134): batch 0 only, laid out [q_blocks, heads, kv_blocks] and [q_blocks, heads]."""
    idx, num = mask_index(mask)
    return idx[0].transpose(0, 1).contiguous(), num[0].transpose(0, 1).contiguous()
