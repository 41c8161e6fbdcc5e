"""`rotary_position_embedding`: argument checks and the unfused branch on CPU (as the reference's
tests/layers/test_rope.py checks them), and the CUDA kernel on a GPU -- bit-equal to the oracle, which
is pinned to vectors of the reference's own unfused branch (tests/golden/rope.npz)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import inputs
import make_golden
from oracle import rope as orope

G = Path(__file__).resolve().parent / "golden"


def test_argument_checks():
    from mindiesd import ParametersInvalid, rotary_position_embedding as rope
    x = torch.randn(2, 64, 8, 16, dtype=torch.float16)
    cos, sin = torch.randn(1, 64, 1, 16), torch.randn(1, 64, 1, 16)
    bad = [
        ([2, 64, 8, 16], cos, sin, "rotated_half", False, True),          # x is not a tensor
        (x[0], cos, sin, "rotated_half", False, True),                    # x is not 4-D
        (x, [1, 64, 1, 16], sin, "rotated_half", False, True),            # cos is not a tensor
        (x, cos, [1, 64, 1, 16], "rotated_half", False, True),            # sin is not a tensor
        (x, cos[0], sin, "rotated_half", False, True),                    # cos is 3-D
        (x, cos, sin[0], "rotated_half", False, True),                    # sin is 3-D
        (x, cos[0, :, 0], sin, "rotated_half", False, True),              # cos and sin differ in rank
        (x, cos, sin, 1, False, True),                                    # mode is not a string
        (x, cos, sin, "rotated", False, True),                            # unknown mode
        (x, cos, sin, "rotated_half", 1, True),                           # head_first is not a bool
        (x, cos, sin, "rotated_half", False, 1),                          # fused is not a bool
    ]
    for args in bad:
        with pytest.raises(ParametersInvalid):
            rope(*args)


def test_unfused_branch_equals_reference_vectors():
    from mindiesd import rotary_position_embedding as rope
    z = np.load(G / "rope.npz")
    for name, xs, head_first, ts, tdt, xdt, mode, seed in make_golden.ROPE_CASES:
        x = inputs.randn(seed, *xs, dtype=xdt)
        cos, sin = inputs.randn(seed + 100, *ts, dtype=tdt), inputs.randn(seed + 200, *ts, dtype=tdt)
        got = rope(x, cos, sin, mode, head_first, False)
        assert got.dtype == xdt and torch.equal(got.float(), torch.from_numpy(z[name])), name


@pytest.mark.gpu
def test_kernel_equals_reference_vectors_and_oracle():
    from mindiesd import _cabi, rotary_position_embedding as rope
    z = np.load(G / "rope.npz")
    for name, xs, head_first, ts, tdt, xdt, mode, seed in make_golden.ROPE_CASES:
        x = inputs.randn(seed, *xs, dtype=xdt)
        cos, sin = inputs.randn(seed + 100, *ts, dtype=tdt), inputs.randn(seed + 200, *ts, dtype=tdt)
        got = rope(x.cuda(), cos.cuda(), sin.cuda(), mode, head_first, True)
        assert got.dtype == xdt and got.shape == x.shape
        assert torch.equal(got.float().cpu(), torch.from_numpy(z[name])), name
    # a larger case against the oracle: Wan-like head dim, BSND, both modes, strided input (a head slice)
    for mode in ("rotated_half", "rotated_interleaved"):
        x = inputs.randn(70, 1, 3000, 6, 128, dtype=torch.bfloat16)
        cos, sin = inputs.randn(71, 3000, 128), inputs.randn(72, 3000, 128)
        xs = x[:, :, 1:5]
        got = rope(xs.cuda(), cos.cuda(), sin.cuda(), mode, False, True)
        assert torch.equal(got.cpu(), orope.rotary_position_embedding(xs, cos, sin, mode, False))
    assert _cabi.device_status() == 0
