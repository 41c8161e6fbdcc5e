"""Rotary position embedding oracle (CPU, torch).  Test infrastructure only."""
import torch


def rotary_position_embedding(x, cos, sin, rotated_mode="rotated_half", head_first=False):
    """Restates the unfused branch of `rotary_position_embedding`, mindiesd/layers/rope.py:91-115.

    x is cast to the dtype of cos, `x * cos + rotated(x) * sin` is evaluated in that dtype with
    torch's elementwise roundings, the result is cast back to the dtype of x.
    rotated_half:        rotated(x) = (-x[d/2:], x[:d/2])
    rotated_interleaved: rotated(x) = (-x1, x0, -x3, x2, ...)
    2-D tables [S, D] broadcast along the token axis of x (axis -2 when head_first, else axis 1).
    """
    if cos.dim() == 2:
        shape = [1] * x.ndim
        shape[-1] = x.shape[-1]
        axis = x.ndim - 2 if head_first else 1
        shape[axis] = x.shape[axis]
        cos, sin = cos.view(*shape), sin.view(*shape)
    xi = x.to(cos.dtype)
    if rotated_mode == "rotated_interleaved":
        even, odd = xi[..., 0::2], xi[..., 1::2]
        rot = torch.stack([-odd, even], dim=-1).flatten(-2)
    elif rotated_mode == "rotated_half":
        h = xi.shape[-1] // 2
        rot = torch.cat([-xi[..., h:], xi[..., :h]], dim=-1)
    else:
        raise ValueError(rotated_mode)
    return (xi * cos + rot * sin).to(x.dtype)
