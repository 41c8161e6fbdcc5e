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
    ]


class RearrangeArgs(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("dst", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
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
        ("block_size", C.c_int32), ("sparsity", C.c_float), ("scale", C.c_float),
        ("protect_first_frame", C.c_int32), ("temporal_band", C.c_int32),
        ("mask", C.c_void_p), ("select_idx", C.c_void_p), ("select_num", C.c_void_p),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
    ]


class QuantArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("out", C.c_void_p), ("scales", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("head_dim", C.c_int32),
        ("x_stride", C.c_int64 * 3),
        ("dtype", C.c_int32), ("mode", C.c_int32), ("row_block", C.c_int32),
    ]


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
                     "mindiesd_fa_block_quant"):
            fn = getattr(handle, name, None)
            if fn is not None:
                fn.restype = C.c_int
                fn.argtypes = [C.c_void_p, C.c_void_p]
        if hasattr(handle, "mindiesd_rf_block_mask_scratch_bytes"):
            handle.mindiesd_rf_block_mask_scratch_bytes.restype = C.c_size_t
            handle.mindiesd_rf_block_mask_scratch_bytes.argtypes = [C.c_int32] * 4
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
