"""`attention_forward_varlen`: flash-attn-varlen-style entry on packed [T, N, D] tensors
(mindiesd/layers/flash_attn/attention_forward_varlen.py:59-149 of MindIE-SD).

Same signature and the same rejections as the reference (every reserved argument must stay None,
dropout 0).  All sequences go to the kernel in ONE launch, as the reference hands them to one fused
call (:142-149): the kernel reads the cumulative lengths on the device and every thread block finds
the sequence its query tiles belong to, so nothing is copied or padded and the host never reads a
length.  `causal=True` is the reference's sparse_mode 3 (:133-138): the triangle is aligned to the
last query and the last key of each sequence.
"""
import math
from dataclasses import dataclass
from typing import Optional

import torch

from ...utils.exception import ParametersInvalid
from ...utils.status import checked


@dataclass
class AttentionInputs:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    max_seqlen_q: int = None
    max_seqlen_k: int = None
    dropout_p: float = 0.0
    window_size: int = None
    softcap: float = None
    alibi_slopes: torch.Tensor = None
    deterministic: bool = None
    return_attn_probs: bool = None
    block_table: torch.Tensor = None


def validate_varlen_attention_inputs(inputs: AttentionInputs):
    reserved = ("max_seqlen_q", "max_seqlen_k", "window_size", "softcap", "alibi_slopes", "deterministic",
                "return_attn_probs", "block_table")
    given = {name: getattr(inputs, name) for name in reserved if getattr(inputs, name) is not None}
    if given:
        raise ParametersInvalid("Unsupported parameters in varlen attention: " +
                                ", ".join(f"{k}={v}" for k, v in given.items()))
    if not math.isclose(inputs.dropout_p, 0.0, abs_tol=1e-6):
        raise ParametersInvalid(f"dropout_p should be set to 0.0 during evaluation, but got {inputs.dropout_p}")
    for name, tensor in (("q", inputs.q), ("k", inputs.k), ("v", inputs.v)):
        if tensor.dim() != 3:
            raise ParametersInvalid(f"Expected {name} to be 3D (T, N, D), but got {tensor.dim()}D tensor.")


def attention_forward_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: Optional[int] = None,
                             max_seqlen_k: Optional[int] = None, dropout_p: float = 0.0,
                             softmax_scale: Optional[float] = None, causal: bool = False,
                             window_size: Optional[int] = None, softcap: Optional[float] = None,
                             alibi_slopes: Optional[torch.Tensor] = None, deterministic: Optional[bool] = None,
                             return_attn_probs: Optional[bool] = None, block_table: Optional[torch.Tensor] = None):
    """q [Tq, N, D], k/v [Tk, Nkv, D]; cu_seqlens_* hold batch + 1 cumulative lengths.  Returns [Tq, N, D]."""
    validate_varlen_attention_inputs(AttentionInputs(
        q=q, k=k, v=v, max_seqlen_q=max_seqlen_q, max_seqlen_k=max_seqlen_k, dropout_p=dropout_p,
        window_size=window_size, softcap=softcap, alibi_slopes=alibi_slopes, deterministic=deterministic,
        return_attn_probs=return_attn_probs, block_table=block_table))
    head_dim = q.shape[-1]
    if softmax_scale is None:
        softmax_scale = head_dim ** -0.5
    cu_q = _as_device_int32(cu_seqlens_q, q.device)
    cu_k = _as_device_int32(cu_seqlens_k, q.device)
    if cu_q.dim() != 1 or cu_q.shape != cu_k.shape or cu_q.numel() < 2:
        raise ParametersInvalid("cu_seqlens_q / cu_seqlens_k must hold batch + 1 cumulative lengths ending at T.")
    if not isinstance(cu_seqlens_q, torch.Tensor) or not cu_seqlens_q.is_cuda:
        # Host-side lengths can be checked without touching the device.
        if int(cu_seqlens_q[-1]) != q.shape[0] or int(cu_seqlens_k[-1]) != k.shape[0]:
            raise ParametersInvalid("cu_seqlens_q / cu_seqlens_k must hold batch + 1 cumulative lengths ending at T.")
    return checked(torch.ops.mindiesd.attention_varlen_fwd(q, k, v, cu_q, cu_k, float(softmax_scale), bool(causal)),
                   "attention_forward_varlen")


def _as_device_int32(cu_seqlens, device):
    """The cumulative lengths as an int32 vector on `device`: a list, a list of 0-d tensors (the
    reference's annotation), a host tensor or a device tensor.  A device tensor is used as it is."""
    if isinstance(cu_seqlens, torch.Tensor):
        return cu_seqlens.to(device=device, dtype=torch.int32).contiguous()
    return torch.tensor([int(x) for x in cu_seqlens], dtype=torch.int32, device=device)
