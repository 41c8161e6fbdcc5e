"""The unfused attention formula (`attention_math`, mindiesd/layers/flash_attn/attention_func.py:32-55
of MindIE-SD): what `attention_forward(..., fused=False)` evaluates, on whatever device the tensors
live, with ordinary torch operators.  It is never reached from the default (fused) path."""
import torch

from ...utils.exception import ParametersInvalid


def attention_math(query, key, value, attn_mask, scale, head_first=False):
    if not head_first:
        query, key, value = query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2)
    dtype = query.dtype
    q_len, kv_len = query.size(-2), key.size(-2)
    scores = ((query * scale) @ key.transpose(-2, -1)).to(torch.float32)
    if attn_mask is not None:
        if attn_mask.dim() not in (2, 4) or attn_mask.size(-2) != q_len or attn_mask.size(-1) != kv_len:
            raise ParametersInvalid("The attn_mask must be a 2D tensor with shape [q_seqlen, kv_seqlen],"
                                    " or a 4D tensor with shape [batch_size, num_heads, q_seqlen, kv_seqlen]")
        bias = torch.zeros(q_len, kv_len, dtype=dtype, device=query.device)
        bias.masked_fill_(attn_mask.logical_not(), float("-inf"))
        scores = scores + bias
    out = torch.softmax(scores, dim=-1).to(dtype) @ value
    return out if head_first else out.transpose(1, 2)
