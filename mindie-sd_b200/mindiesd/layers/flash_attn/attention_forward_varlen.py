"""`attention_forward_varlen`: flash-attn-varlen-style entry on packed [T, N, D] tensors
(mindiesd/layers/flash_attn/attention_forward_varlen.py:59-149 of MindIE-SD).

Same signature and the same rejections as the reference (every reserved argument must stay None,
dropout 0).  Each sequence is one launch of the dense kernel on a [1, len, N, D] view of the packed
tensor, so nothing is copied or padded.  `causal=True` is rejected: video-DiT self-attention is not
causal and the kernel has no causal mode.
"""
import math
from dataclasses import dataclass
from typing import Optional

import torch

from ...utils.exception import ParametersInvalid


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
    if causal:
        raise ParametersInvalid("causal=True is not supported by the B200 attention kernel.")
    head_dim = q.shape[-1]
    if softmax_scale is None:
        softmax_scale = head_dim ** -0.5
    bounds_q = [int(x) for x in cu_seqlens_q]
    bounds_k = [int(x) for x in cu_seqlens_k]
    if len(bounds_q) != len(bounds_k) or len(bounds_q) < 2 or bounds_q[-1] != q.shape[0] or bounds_k[-1] != k.shape[0]:
        raise ParametersInvalid("cu_seqlens_q / cu_seqlens_k must hold batch + 1 cumulative lengths ending at T.")
    out = torch.empty_like(q)
    for i in range(len(bounds_q) - 1):
        q0, q1, k0, k1 = bounds_q[i], bounds_q[i + 1], bounds_k[i], bounds_k[i + 1]
        if q1 <= q0:
            continue
        if k1 <= k0:
            out[q0:q1].zero_()
            continue
        out[q0:q1] = torch.ops.mindiesd.attention_fwd(q[q0:q1].unsqueeze(0), k[k0:k1].unsqueeze(0),
                                                      v[k0:k1].unsqueeze(0), float(softmax_scale), False)[0]
    return out
