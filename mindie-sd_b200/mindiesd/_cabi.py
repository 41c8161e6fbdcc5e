"""ctypes binding of the C-ABI library (``include/mindiesd_b200.h``).

The library is the only implementation of the hot path: if it cannot be loaded, or a call returns
an error code, the caller gets an exception -- there is no other path to fall back to.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_LIB_NAME = "libmindiesd_b200.so"
_lib = None

BF16, FP16, FP32, E4M3 = 0, 1, 2, 3
SPARSE_NONE, SPARSE_MASK, SPARSE_LIST = 0, 1, 2

_ERRORS = {
    -1: "a required pointer is NULL",
    -2: "unsupported size",
    -3: "unsupported element type",
    -4: "stride or pointer not 16-byte aligned",
    -5: "scalar argument out of range",
    -6: "the CUDA driver refused the request",
    -7: "size exceeds a fixed capacity of the entry point",
}


class NativeLibraryError(RuntimeError):
    """The CUDA library is missing or one of its entry points reported an error."""


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32),
        ("seq_q", C.c_int32), ("seq_kv", C.c_int32), ("head_dim", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("v_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("in_dtype", C.c_int32), ("out_dtype", C.c_int32), ("scale", C.c_float),
        ("sparse_mode", C.c_int32), ("block_size", C.c_int32),
        ("block_mask", C.c_void_p), ("mask_stride", C.c_int64 * 3),
        ("select_idx", C.c_void_p), ("select_num", C.c_void_p),
        ("q_scale", C.c_void_p), ("k_scale", C.c_void_p), ("v_scale", C.c_void_p),
        ("k_scale_block", C.c_int32), ("v_scale_block", C.c_int32),
        ("lse_stride", C.c_int64 * 3),
        ("causal", C.c_int32), ("num_seqs", C.c_int32),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_kv", C.c_void_p),
        ("perm_t", C.c_int32), ("perm_h", C.c_int32), ("perm_w", C.c_int32), ("perm_txt", C.c_int32),
        ("perm_inputs_permuted", C.c_int32),
        ("wait_limit_us", C.c_uint32), ("test_withhold", C.c_int32),
        ("q_pairs", C.c_void_p), ("q_pair_count", C.c_int32),
    ]


class PairArgs(C.Structure):
    _fields_ = [
        ("mask", C.c_void_p), ("mask_stride", C.c_int64 * 3),
        ("batch", C.c_int32), ("heads", C.c_int32), ("q_blocks", C.c_int32), ("kv_blocks", C.c_int32),
        ("pairs", C.c_void_p),
    ]


class RearrangeArgs(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("dst", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("elem_bytes", C.c_int32),
        ("src_stride", C.c_int64 * 3), ("dst_stride", C.c_int64 * 3),
        ("t", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("txt_len", C.c_int32),
        ("inverse", C.c_int32),
    ]


class MaskArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("dtype", C.c_int32),
        ("t", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("txt_len", C.c_int32),
        ("block_size", C.c_int32), ("scale", C.c_float), ("sparsity", C.c_double),
        ("protect_first_frame", C.c_int32), ("temporal_band", C.c_int32),
        ("mask", C.c_void_p), ("select_idx", C.c_void_p), ("select_num", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
    ]


class PoolArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("pooled", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("x_stride", C.c_int64 * 3),
        ("dtype", C.c_int32),
        ("t", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("txt_len", C.c_int32),
        ("permute", C.c_int32), ("block_size", C.c_int32),
    ]


class PooledMaskArgs(C.Structure):
    _fields_ = [
        ("q_pooled", C.c_void_p), ("k_pooled", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("blocks", C.c_int32), ("head_dim", C.c_int32),
        ("t", C.c_int32), ("h", C.c_int32), ("w", C.c_int32), ("txt_len", C.c_int32),
        ("block_size", C.c_int32), ("protect_first_frame", C.c_int32), ("temporal_band", C.c_int32),
        ("sparsity", C.c_double),
        ("mask", C.c_void_p), ("select_idx", C.c_void_p), ("select_num", C.c_void_p),
    ]


class QuantArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("out", C.c_void_p), ("scales", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("x_stride", C.c_int64 * 3),
        ("dtype", C.c_int32), ("mode", C.c_int32), ("row_block", C.c_int32), ("rotate", C.c_int32),
    ]


class RotateQuantArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("rot", C.c_void_p), ("out", C.c_void_p), ("scales", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("x_stride", C.c_int64 * 3),
        ("dtype", C.c_int32), ("row_block", C.c_int32),
    ]


class EstimateArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("dtype", C.c_int32),
        ("batch", C.c_int32), ("heads", C.c_int32), ("kv_heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("stride", C.c_int32), ("sparse_size", C.c_int32),
        ("scale", C.c_float), ("threshold", C.c_float), ("row_sparse", C.c_double),
        ("causal", C.c_int32), ("keep_sink", C.c_int32), ("keep_recent", C.c_int32),
        ("mask", C.c_void_p), ("mask_cols", C.c_int32), ("count", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
        ("causal_key_tokens", C.c_int32),
    ]


MAX_RANKS = 8


class RopeArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("out", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("x_stride", C.c_int64 * 3), ("out_stride", C.c_int64 * 3),
        ("dtype", C.c_int32), ("table_dtype", C.c_int32), ("mode", C.c_int32),
    ]


class UlyssesMoveArgs(C.Structure):
    _fields_ = [
        ("tensor", C.c_void_p * 3), ("table", C.c_void_p * MAX_RANKS),
        ("tensor_row_stride", C.c_int64), ("tensor_head_stride", C.c_int64), ("table_row_stride", C.c_int64),
        ("n_src", C.c_int32), ("rows", C.c_int32), ("world", C.c_int32), ("group_heads", C.c_int32),
        ("head0", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("dtype", C.c_int32), ("inverse", C.c_int32),
        ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("rope_mode", C.c_int32), ("thread_blocks", C.c_int32),
    ]


ROPE_HALF, ROPE_INTERLEAVED = 1, 2


def library_path() -> Path:
    override = os.environ.get("MINDIESD_B200_LIB")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / "plugin" / _LIB_NAME


def lib():
    """Loads the library on first use; raises NativeLibraryError if it is absent."""
    global _lib
    if _lib is None:
        path = library_path()
        if not path.exists():
            raise NativeLibraryError(
                f"{path} not found: build it with `python mindie-sd_b200/csrc/build.py`; "
                "this package has no other implementation of its operators")
        try:
            handle = C.CDLL(str(path))
        except OSError as exc:  # pragma: no cover - depends on the machine
            raise NativeLibraryError(f"cannot load {path}: {exc}") from exc
        handle.mindiesd_abi_version.restype = C.c_int
        for name in ("mindiesd_attention_fwd", "mindiesd_rf_rearrange", "mindiesd_rf_block_mask",
                     "mindiesd_rf_pool", "mindiesd_rf_mask_from_pooled", "mindiesd_fa_block_quant",
                     "mindiesd_sparse_block_estimate", "mindiesd_fa_rotate_quant", "mindiesd_rope",
                     "mindiesd_ulysses_move"):
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.restype = C.c_int
                fn.argtypes = [C.c_void_p, C.c_void_p]
        if hasattr(handle, "mindiesd_rf_block_mask_scratch_bytes"):
            handle.mindiesd_rf_block_mask_scratch_bytes.restype = C.c_size_t
            handle.mindiesd_rf_block_mask_scratch_bytes.argtypes = [C.c_int32] * 4
        if hasattr(handle, "mindiesd_sparse_block_estimate_scratch_bytes"):
            handle.mindiesd_sparse_block_estimate_scratch_bytes.restype = C.c_size_t
            handle.mindiesd_sparse_block_estimate_scratch_bytes.argtypes = [C.c_int32] * 3
        handle.mindiesd_device_status.restype = C.c_int
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise NativeLibraryError(f"{what}: invalid argument ({_ERRORS.get(rc, rc)})")
    raise NativeLibraryError(f"{what}: CUDA error {rc}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float16:
        return FP16
    if dtype == torch.float32:
        return FP32
    if dtype == torch.float8_e4m3fn:
        return E4M3
    raise NativeLibraryError(f"unsupported element type {dtype}")


def current_stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def device_status() -> int:
    """Synchronises the current device and returns (and clears) its kernel status word."""
    return int(lib().mindiesd_device_status())


def strides_bns(x: torch.Tensor, head_first: bool):
    """Element strides (batch, head, token) of a 4-D tensor in BNSD (head_first) or BSND order."""
    if x.stride(3) != 1:
        raise NativeLibraryError("the channel dimension must be contiguous")
    sb, s1, s2, _ = x.stride()
    return (sb, s1, s2) if head_first else (sb, s2, s1)


# ---- convenience callers: torch tensors in, torch tensors out, nothing else between ---------------

def _dims(x, head_first):
    b, d = x.shape[0], x.shape[3]
    n, s = (x.shape[1], x.shape[2]) if head_first else (x.shape[2], x.shape[1])
    return b, n, s, d


def attention(q, k, v, head_first=True, scale=None, block_mask=None, select_idx=None, select_num=None,
              out_dtype=None, want_lse=False, q_scale=None, k_scale=None, v_scale=None, k_scale_block=0,
              v_scale_block=0, out=None, causal=False, cu_seqlens_q=None, cu_seqlens_kv=None, wait_limit_us=0,
              test_withhold=0, perm_grid=None, perm_txt=0, perm_inputs_permuted=False, q_pairs=None):
    """mindiesd_attention_fwd on the current stream.  Returns out, or (out, lse) when want_lse.
    cu_seqlens_q / cu_seqlens_kv (int32 device tensors [num_seqs + 1]) select the packed
    variable-length form: q, k, v are then [1, N, T, D] (head_first) or [1, T, N, D]."""
    b, n, sq, d = _dims(q, head_first)
    _, nkv, skv, _ = _dims(k, head_first)
    if out is None:
        odt = out_dtype or (q.dtype if q.dtype != torch.float8_e4m3fn else torch.bfloat16)
        out = torch.empty(q.shape, dtype=odt, device=q.device)
    a = AttnArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    lse = None
    if want_lse:
        lse = torch.empty(b, n, sq, dtype=torch.float32, device=q.device)
        a.lse = lse.data_ptr()
    a.batch, a.heads, a.kv_heads, a.seq_q, a.seq_kv, a.head_dim = b, n, nkv, sq, skv, d
    a.q_stride[:] = strides_bns(q, head_first)
    a.k_stride[:] = strides_bns(k, head_first)
    a.v_stride[:] = strides_bns(v, head_first)
    a.o_stride[:] = strides_bns(out, head_first)
    a.in_dtype, a.out_dtype = dtype_code(q.dtype), dtype_code(out.dtype)
    a.scale = float(scale if scale is not None else d ** -0.5)
    a.block_size = 128
    if block_mask is not None:
        a.sparse_mode = SPARSE_MASK
        a.block_mask = block_mask.data_ptr()
        a.mask_stride[:] = (block_mask.stride(0), block_mask.stride(1), block_mask.stride(2))
    elif select_idx is not None:
        a.sparse_mode = SPARSE_LIST
        a.select_idx, a.select_num = select_idx.data_ptr(), select_num.data_ptr()
    if q_scale is not None:
        a.q_scale, a.k_scale, a.v_scale = q_scale.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr()
        a.k_scale_block, a.v_scale_block = k_scale_block, v_scale_block
    a.causal = int(bool(causal))
    if cu_seqlens_q is not None:
        for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_kv", cu_seqlens_kv)):
            if t is None or t.dtype != torch.int32 or t.device != q.device or not t.is_contiguous():
                raise NativeLibraryError(f"{name} must be a contiguous int32 tensor on the device of q")
        a.num_seqs = cu_seqlens_q.numel() - 1
        a.cu_seqlens_q, a.cu_seqlens_kv = cu_seqlens_q.data_ptr(), cu_seqlens_kv.data_ptr()
    if perm_grid is not None:  # the RainFusion window permutation applied inside the kernel
        a.perm_t, a.perm_h, a.perm_w = (int(x) for x in perm_grid)
        a.perm_txt = int(perm_txt)
        a.perm_inputs_permuted = int(bool(perm_inputs_permuted))
    a.wait_limit_us, a.test_withhold = int(wait_limit_us), int(test_withhold)
    if q_pairs is not None:  # which two query blocks share a thread block (rf_pair_blocks)
        if q_pairs.dtype != torch.int32 or q_pairs.device != q.device or not q_pairs.is_contiguous():
            raise NativeLibraryError("q_pairs must be a contiguous int32 tensor on the device of q")
        a.q_pairs, a.q_pair_count = q_pairs.data_ptr(), q_pairs.shape[-2]
    check(lib().mindiesd_attention_fwd(C.byref(a), current_stream_ptr(q.device)), "mindiesd_attention_fwd")
    return (out, lse) if want_lse else out


def rf_pair_blocks(block_mask):
    """mindiesd_rf_pair_blocks: int32 [B, N, (q_blocks + 1) // 2, 2] pairing of the query blocks of an int8 block
    mask [B, N, q_blocks, kv_blocks] by the overlap of their key-block lists, for attention(q_pairs=...)."""
    b, n, qb, kb = block_mask.shape
    pairs = torch.empty(b, n, (qb + 1) // 2, 2, dtype=torch.int32, device=block_mask.device)
    a = PairArgs()
    a.mask, a.pairs = block_mask.data_ptr(), pairs.data_ptr()
    a.mask_stride[:] = (block_mask.stride(0), block_mask.stride(1), block_mask.stride(2))
    a.batch, a.heads, a.q_blocks, a.kv_blocks = b, n, qb, kb
    check(lib().mindiesd_rf_pair_blocks(C.byref(a), current_stream_ptr(block_mask.device)), "mindiesd_rf_pair_blocks")
    return pairs


def rf_rearrange(x, grid, txt_len=0, head_first=True, inverse=False):
    b, n, s, d = _dims(x, head_first)
    dst = torch.empty_like(x)
    a = RearrangeArgs()
    a.src, a.dst = x.data_ptr(), dst.data_ptr()
    a.batch, a.heads, a.seq, a.head_dim, a.elem_bytes = b, n, s, d, x.element_size()
    a.src_stride[:] = strides_bns(x, head_first)
    a.dst_stride[:] = strides_bns(dst, head_first)
    a.t, a.h, a.w = grid
    a.txt_len, a.inverse = txt_len, int(inverse)
    check(lib().mindiesd_rf_rearrange(C.byref(a), current_stream_ptr(x.device)), "mindiesd_rf_rearrange")
    return dst


def rf_block_mask(q, k, grid, txt_len=0, sparsity=0.0, head_first=True, protect_first_frame=True, temporal_band=-1,
                  want_lists=False, scratch=None):
    b, n, s, d = _dims(q, head_first)
    blocks = (grid[0] * grid[1] * grid[2] + 127) // 128 + (txt_len + 127) // 128
    mask = torch.empty(b, n, blocks, blocks, dtype=torch.int8, device=q.device)
    a = MaskArgs()
    a.q, a.k = q.data_ptr(), k.data_ptr()
    a.batch, a.heads, a.seq, a.head_dim = b, n, s, d
    a.q_stride[:] = strides_bns(q, head_first)
    a.k_stride[:] = strides_bns(k, head_first)
    a.dtype = dtype_code(q.dtype)
    a.t, a.h, a.w = grid
    a.txt_len, a.block_size, a.scale, a.sparsity = txt_len, 128, d ** -0.5, float(sparsity)
    a.protect_first_frame, a.temporal_band = int(protect_first_frame), temporal_band
    a.mask = mask.data_ptr()
    sel = num = None
    if want_lists:
        sel = torch.empty(blocks, n, blocks, dtype=torch.int64, device=q.device)
        num = torch.empty(blocks, n, dtype=torch.int64, device=q.device)
        a.select_idx, a.select_num = sel.data_ptr(), num.data_ptr()
    nbytes = lib().mindiesd_rf_block_mask_scratch_bytes(b, n, s, d)
    if scratch is None:
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
    a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    check(lib().mindiesd_rf_block_mask(C.byref(a), current_stream_ptr(q.device)), "mindiesd_rf_block_mask")
    return (mask, sel, num) if want_lists else mask


def rf_pool(x, grid=None, txt_len=0, head_first=True):
    b, n, s, d = _dims(x, head_first)
    a = PoolArgs()
    if grid is None:
        blocks = (s + 127) // 128
    else:
        blocks = (grid[0] * grid[1] * grid[2] + 127) // 128 + (txt_len + 127) // 128
        a.t, a.h, a.w = grid
        a.txt_len, a.permute = txt_len, 1
    pooled = torch.empty(b, n, blocks, d, dtype=torch.float32, device=x.device)
    a.x, a.pooled = x.data_ptr(), pooled.data_ptr()
    a.batch, a.heads, a.seq, a.head_dim = b, n, s, d
    a.x_stride[:] = strides_bns(x, head_first)
    a.dtype, a.block_size = dtype_code(x.dtype), 128
    check(lib().mindiesd_rf_pool(C.byref(a), current_stream_ptr(x.device)), "mindiesd_rf_pool")
    return pooled


def fa_block_quant(x, row_block=128, head_first=True, per_channel=False, rotate=False):
    b, n, s, d = _dims(x, head_first)
    out = torch.empty(b, n, s, d, dtype=torch.float8_e4m3fn, device=x.device)
    nscale = d if per_channel else (s + row_block - 1) // row_block
    scales = torch.empty(b, n, nscale, dtype=torch.float32, device=x.device)
    a = QuantArgs()
    a.x, a.out, a.scales = x.data_ptr(), out.data_ptr(), scales.data_ptr()
    a.batch, a.heads, a.seq, a.head_dim = b, n, s, d
    a.x_stride[:] = strides_bns(x, head_first)
    a.dtype, a.mode, a.row_block, a.rotate = dtype_code(x.dtype), int(per_channel), row_block, int(rotate)
    check(lib().mindiesd_fa_block_quant(C.byref(a), current_stream_ptr(x.device)), "mindiesd_fa_block_quant")
    return out, scales


def rf_block_mask_static(q, k, grid, txt_len=0, sparsity=0.0, head_first=True, protect_first_frame=True,
                         temporal_band=-1, want_lists=False):
    """mindiesd_rf_block_mask_static: the mask builder with its scratch inside the library, for hosts
    that may not allocate device memory.  Outputs are still the caller's; sizes beyond the library's
    fixed 4 MiB of scratch raise NativeLibraryError (capacity)."""
    fn = lib().mindiesd_rf_block_mask_static
    fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_void_p]
    b, n, s, d = _dims(q, head_first)
    blocks = (grid[0] * grid[1] * grid[2] + 127) // 128 + (txt_len + 127) // 128
    mask = torch.empty(b, n, blocks, blocks, dtype=torch.int8, device=q.device)
    a = MaskArgs()
    a.q, a.k = q.data_ptr(), k.data_ptr()
    a.batch, a.heads, a.seq, a.head_dim = b, n, s, d
    a.q_stride[:] = strides_bns(q, head_first)
    a.k_stride[:] = strides_bns(k, head_first)
    a.dtype = dtype_code(q.dtype)
    a.t, a.h, a.w = grid
    a.txt_len, a.block_size, a.scale, a.sparsity = txt_len, 128, d ** -0.5, float(sparsity)
    a.protect_first_frame, a.temporal_band = int(protect_first_frame), temporal_band
    a.mask = mask.data_ptr()
    sel = num = None
    if want_lists:
        sel = torch.empty(blocks, n, blocks, dtype=torch.int64, device=q.device)
        num = torch.empty(blocks, n, dtype=torch.int64, device=q.device)
        a.select_idx, a.select_num = sel.data_ptr(), num.data_ptr()
    check(fn(C.byref(a), current_stream_ptr(q.device)), "mindiesd_rf_block_mask_static")
    return (mask, sel, num) if want_lists else mask


def sparse_block_estimate(q, k, scale, threshold, row_sparse=1.0, head_first=True, keep_sink=True, keep_recent=True,
                          scratch=None, causal=False, causal_key_tokens=0):
    """mindiesd_sparse_block_estimate on tensors whose token count is a multiple of 8.
    Returns (int8 mask [B, N, blocks, blocks rounded up to 32], int32 count [B, N, blocks])."""
    b, n, s, d = _dims(q, head_first)
    nkv = k.shape[1] if head_first else k.shape[2]
    blocks = (s + 127) // 128
    cols = (blocks + 31) // 32 * 32
    mask = torch.empty(b, n, blocks, cols, dtype=torch.int8, device=q.device)
    count = torch.empty(b, n, blocks, dtype=torch.int32, device=q.device)
    if scratch is None:
        scratch = torch.empty(lib().mindiesd_sparse_block_estimate_scratch_bytes(b, n, s), dtype=torch.uint8,
                              device=q.device)
    a = EstimateArgs()
    a.q, a.k = q.data_ptr(), k.data_ptr()
    a.q_stride[:] = strides_bns(q, head_first)
    a.k_stride[:] = strides_bns(k, head_first)
    a.dtype = dtype_code(q.dtype)
    a.batch, a.heads, a.kv_heads, a.seq, a.head_dim = b, n, nkv, s, d
    a.stride, a.sparse_size = 8, 128
    a.scale, a.threshold, a.row_sparse = float(scale), float(threshold), float(row_sparse)
    a.causal, a.keep_sink, a.keep_recent = int(bool(causal)), int(keep_sink), int(keep_recent)
    a.causal_key_tokens = int(causal_key_tokens)
    a.mask, a.mask_cols, a.count = mask.data_ptr(), cols, count.data_ptr()
    a.scratch, a.scratch_bytes = scratch.data_ptr(), scratch.numel()
    check(lib().mindiesd_sparse_block_estimate(C.byref(a), current_stream_ptr(q.device)),
          "mindiesd_sparse_block_estimate")
    return mask, count


def fa_rotate_quant(x, rot, row_block=128, head_first=True):
    """mindiesd_fa_rotate_quant: (x @ rot) quantised to e4m3 in row_block-token blocks without
    materialising the product.  Returns (e4m3 [B, N, S, D], fp32 scales [B, N, blocks])."""
    b, n, s, d = _dims(x, head_first)
    rot = rot.to(device=x.device, dtype=x.dtype).contiguous()
    out = torch.empty(b, n, s, d, dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.empty(b, n, (s + row_block - 1) // row_block, dtype=torch.float32, device=x.device)
    a = RotateQuantArgs()
    a.x, a.rot, a.out, a.scales = x.data_ptr(), rot.data_ptr(), out.data_ptr(), scales.data_ptr()
    a.batch, a.heads, a.seq, a.head_dim = b, n, s, d
    a.x_stride[:] = strides_bns(x, head_first)
    a.dtype, a.row_block = dtype_code(x.dtype), row_block
    check(lib().mindiesd_fa_rotate_quant(C.byref(a), current_stream_ptr(x.device)), "mindiesd_fa_rotate_quant")
    return out, scales


def rope(x, cos, sin, mode, head_first=False, out=None):
    """mindiesd_rope: x [B, N, S, D] (head_first) or [B, S, N, D]; cos/sin contiguous [S, D] tables in fp32
    or the type of x; mode ROPE_HALF / ROPE_INTERLEAVED."""
    b, n, s, d = _dims(x, head_first)
    if out is None:
        out = torch.empty_like(x)
    a = RopeArgs()
    a.x, a.out, a.cos, a.sin = x.data_ptr(), out.data_ptr(), cos.data_ptr(), sin.data_ptr()
    a.batch, a.heads, a.seq, a.head_dim = b, n, s, d
    a.x_stride[:] = strides_bns(x, head_first)
    a.out_stride[:] = strides_bns(out, head_first)
    a.dtype, a.table_dtype, a.mode = dtype_code(x.dtype), dtype_code(cos.dtype), int(mode)
    check(lib().mindiesd_rope(C.byref(a), current_stream_ptr(x.device)), "mindiesd_rope")
    return out


def ulysses_move(tensors, table_ptrs, table_row_stride, rows, world, group_heads, head0, heads, inverse=False,
                 cos=None, sin=None, rope_mode=0, thread_blocks=0):
    """mindiesd_ulysses_move on the current stream.  tensors: this rank's [rows, N, 128] views (q, k, v; or
    the output when inverse), all with the strides of the first; table_ptrs: one device address per rank."""
    t0 = tensors[0]
    a = UlyssesMoveArgs()
    for i, t in enumerate(tensors):
        if t.stride(-1) != 1 or t.stride() != t0.stride() or t.dtype != t0.dtype:
            raise NativeLibraryError("ulysses_move: the tensors must share dtype and strides, channels contiguous")
        a.tensor[i] = t.data_ptr()
    for r, ptr in enumerate(table_ptrs):
        a.table[r] = int(ptr)
    a.tensor_row_stride, a.tensor_head_stride, a.table_row_stride = t0.stride(-3), t0.stride(-2), int(table_row_stride)
    a.n_src, a.rows, a.world, a.group_heads, a.head0, a.heads = len(tensors), rows, world, group_heads, head0, heads
    a.head_dim, a.dtype, a.inverse = t0.shape[-1], dtype_code(t0.dtype), int(inverse)
    if rope_mode:
        a.cos, a.sin, a.rope_mode = cos.data_ptr(), sin.data_ptr(), int(rope_mode)
    a.thread_blocks = int(thread_blocks)
    check(lib().mindiesd_ulysses_move(C.byref(a), current_stream_ptr(t0.device)), "mindiesd_ulysses_move")


def copy_2d(dst_ptr, dst_pitch, src_ptr, src_pitch, width_bytes, height, stream):
    """mindiesd_copy_2d on `stream` (a torch.cuda.Stream): rows of width_bytes, pitches in bytes."""
    fn = lib().mindiesd_copy_2d
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]
    check(fn(dst_ptr, dst_pitch, src_ptr, src_pitch, width_bytes, height, stream.cuda_stream), "mindiesd_copy_2d")


def peer_export(t: torch.Tensor):
    """(handle bytes, offset) that lets another process on this box map tensor `t` (mindiesd_peer_export)."""
    fn = lib().mindiesd_peer_export
    fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_uint64)]
    handle = (C.c_uint8 * 64)()
    offset = C.c_uint64(0)
    check(fn(t.data_ptr(), handle, C.byref(offset)), "mindiesd_peer_export")
    return bytes(handle), int(offset.value)


def peer_open(handle: bytes, offset: int) -> int:
    """Device address, valid on the current device, of the buffer another process exported."""
    fn = lib().mindiesd_peer_open
    fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_void_p)]
    buf = (C.c_uint8 * 64).from_buffer_copy(handle)
    ptr = C.c_void_p(0)
    check(fn(buf, offset, C.byref(ptr)), "mindiesd_peer_open")
    return int(ptr.value)
