"""`attention_forward`: the dense attention entry of the layer API
(mindiesd/layers/flash_attn/attention_forward.py:24-129 of MindIE-SD).

Same signature, validation, defaults and error type.  The reference's `opt_mode` / `op_type` /
`layout` keyword arguments choose among several NPU operators; they are validated here exactly as
there and then all lead to the one sm_100a kernel, which reads BNSD and BSND through strides.
"""
import os

import torch

from .attention_func import attention_math
from .common import AttentionParam
from ...utils.exception import ParametersInvalid
from ...utils.status import checked

_SUPPORTED_FA_TYPES = {"prompt_flash_attn", "fused_attn_score", "ascend_laser_attention"}
_SUPPORTED_LAYOUTS = {"BNSD", "BSND", "BSH"}


def attention_forward(query, key, value, attn_mask=None, scale=None, fused=True, head_first=False, **kwargs):
    check_input_params((query, key, value, attn_mask, scale, fused))
    if head_first:
        param = AttentionParam(query.shape[0], query.shape[1], query.shape[-1], query.shape[2], key.shape[2],
                               query.dtype, head_first)
    else:
        param = AttentionParam(query.shape[0], query.shape[-2], query.shape[-1], query.shape[1], key.shape[1],
                               query.dtype, head_first)
    if scale is None:
        scale = param.head_dim ** -0.5
    if not fused:
        return attention_math(query, key, value, attn_mask, scale, head_first)

    opt_mode = kwargs.get("opt_mode", "runtime")
    if opt_mode == "manual":
        op_type = os.getenv("MINDIE_SD_FA_TYPE") or kwargs.get("op_type", "fused_attn_score")
        if op_type not in _SUPPORTED_FA_TYPES:
            raise ParametersInvalid(f"Unsupported FA type: '{op_type}'. Supported values: {_SUPPORTED_FA_TYPES}")
        layout = kwargs.get("layout", "BNSD")
        if layout not in _SUPPORTED_LAYOUTS:
            raise ParametersInvalid(f"Unsupported layout: '{layout}'. Supported values: {_SUPPORTED_LAYOUTS}")
    elif opt_mode not in ("runtime", "static"):
        raise ParametersInvalid(f"The input 'opt_mode':{opt_mode} is invalid. "
                                f"The list of supported options is ['runtime', 'static', 'manual']")
    if attn_mask is not None:
        raise ParametersInvalid("The fused attention kernel takes no attn_mask (video-DiT self-attention is unmasked); "
                                "use fused=False for a masked evaluation.")
    if query.dtype not in (torch.bfloat16, torch.float16):
        raise ParametersInvalid(f"The fused attention kernel supports bfloat16 and float16, but got {query.dtype}.")
    return checked(torch.ops.mindiesd.attention_fwd(query, key, value, float(scale), bool(head_first)), "attention_forward")


def check_input_params(input_params):
    query, key, value, attn_mask, scale, fused = input_params
    for name, x in (("query", query), ("key", key), ("value", value)):
        if not isinstance(x, torch.Tensor):
            raise ParametersInvalid(f"The data type of input {name} must be torch.Tensor, but got {type(x)}.")
    for name, x in (("query", query), ("key", key), ("value", value)):
        if x.dim() != 4:
            raise ParametersInvalid(f"The dimensional of input {name} must be 4, but got {x.dim()}.")
    if not isinstance(fused, bool):
        raise ParametersInvalid(f"The data type of input fused must be bool, but got {type(fused)}.")
    if attn_mask is not None and not isinstance(attn_mask, torch.Tensor):
        raise ParametersInvalid(f"The data type of input attn_mask must be torch.Tensor, but got {type(attn_mask)}.")
    if scale is not None and not isinstance(scale, float):
        raise ParametersInvalid(f"The data type of input scale must be float, but got {type(scale)}.")
