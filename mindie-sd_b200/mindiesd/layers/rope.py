"""`rotary_position_embedding` (mindiesd/layers/rope.py:54-115 of MindIE-SD).

Same signature, checks, modes and layouts.  `fused=True` runs the CUDA kernel (the reference calls
`torch_npu.npu_rotary_mul` there); `fused=False` is the reference's explicit torch formula on the
tensors' own device.  Both compute in the dtype of `cos` and return the dtype of `x`; the kernel
follows the unfused formula's roundings, so the two branches agree bit for bit.

Sequence-parallel callers do not need this call at all: `ulysses_attention(..., rope=(cos, sin, mode))`
applies the rotation to q and k inside the kernel that re-shards them.
"""
import torch

from ..utils.exception import ParametersInvalid

_MODES = {"rotated_half": 1, "rotated_interleaved": 2}


def check_input_params(x, cos, sin, rotated_mode, head_first, fused):
    for name, val in (("x", x), ("cos", cos), ("sin", sin)):
        if not isinstance(val, torch.Tensor):
            raise ParametersInvalid(f"The data type of input {name} must be torch.Tensor, but got {type(val)}.")
    if not isinstance(rotated_mode, str):
        raise ParametersInvalid(f"The data type of input rotated_mode must be str, but got {type(rotated_mode)}.")
    if not isinstance(head_first, bool):
        raise ParametersInvalid(f"The data type of input head_first must be bool, but got {type(head_first)}.")
    if not isinstance(fused, bool):
        raise ParametersInvalid(f"The data type of input fused must be bool, but got {type(fused)}.")
    if x.dim() != 4:
        raise ParametersInvalid(f"The dimensional of input x must be a 4, but got {x.dim()}.")
    for name, val in (("cos", cos), ("sin", sin)):
        if val.dim() not in (2, 4):
            raise ParametersInvalid(f"The dimensional of input {name} must be a 2 or 4, but got {val.dim()}.")
    if cos.dim() != sin.dim():
        raise ParametersInvalid(f"The dimensional of input cos must be equal to the dimensional of input sin, "
                                f"but {cos.dim()} != {sin.dim()}.")


def reshape_for_broadcast(x, cos, sin, head_first=False):
    shape = [1] * x.ndim
    shape[-1] = x.shape[-1]
    seq_axis = x.ndim - 2 if head_first else 1
    shape[seq_axis] = x.shape[seq_axis]
    return cos.view(*shape), sin.view(*shape)


def _unfused(x, cos, sin, mode):
    x_in = x.to(cos.dtype)
    if mode == 2:
        real, imag = x_in.reshape(*x_in.shape[:-1], -1, 2).unbind(-1)
        rotated = torch.stack([-imag, real], dim=-1).flatten(3)
    else:
        real, imag = x_in.reshape(*x_in.shape[:-1], 2, -1).unbind(-2)
        rotated = torch.cat([-imag, real], dim=-1)
    return (x_in * cos + rotated * sin).type_as(x)


def rotary_position_embedding(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotated_mode: str = "rotated_half",
                              head_first: bool = False, fused: bool = True) -> torch.Tensor:
    """x: [B, N, S, D] (head_first), [B, S, N, D], or [S, B, N, D] with tables [S, 1, 1, D].
    cos/sin: [S, D], [1, 1, S, D], [1, S, 1, D] or [S, 1, 1, D]."""
    check_input_params(x, cos, sin, rotated_mode, head_first, fused)
    if rotated_mode not in _MODES:
        raise ParametersInvalid(f"Unsupported rotated_mode: {rotated_mode}. The supported "
                                "rotated_mode must be 'rotated_half' or 'rotated_interleaved'")
    mode = _MODES[rotated_mode]
    d = x.shape[-1]
    if cos.dim() == 2:
        cos4, sin4 = reshape_for_broadcast(x, cos, sin, head_first=head_first)
    else:
        cos4, sin4 = cos, sin
    if not fused:
        return _unfused(x, cos4, sin4, mode)
    if not x.is_cuda:
        raise ParametersInvalid("The fused rotary embedding runs on a CUDA device; pass fused=False on the host.")
    # Which axis of x the tables run along: the one where they are not 1 (besides the channels).
    axes = [i for i in range(3) if cos4.shape[i] != 1]
    if cos4.shape[-1] != d or sin4.shape != cos4.shape or len(axes) > 1 or d % 2 or \
            cos.dtype not in (torch.float32, x.dtype) or sin.dtype != cos.dtype:
        return _unfused(x, cos4, sin4, mode)  # broadcast patterns the kernel does not take
    seq_axis = axes[0] if axes else (2 if head_first else 1)
    if cos4.shape[seq_axis] != x.shape[seq_axis]:
        raise ParametersInvalid(f"cos/sin cover {cos4.shape[seq_axis]} positions but x has {x.shape[seq_axis]}.")
    from .. import _cabi
    # View x as [B, N, S, D] for the kernel: move the table axis to position 2.
    order = [i for i in range(3) if i != seq_axis]
    xv = x.permute(order[0], order[1], seq_axis, 3)
    if xv.stride(3) != 1:
        xv = xv.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    ov = out.permute(order[0], order[1], seq_axis, 3)
    tab_c = cos4.reshape(-1, d).contiguous()
    tab_s = sin4.reshape(-1, d).contiguous()
    _cabi.rope(xv, tab_c, tab_s, mode, head_first=True, out=ov)
    return out
