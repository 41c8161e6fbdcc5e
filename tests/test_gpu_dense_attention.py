"""GPU parity of the dense attention kernel, called through the C ABI, against the CPU oracle
(`oracle.attention.attention_math`, the reference's unfused formula) and the committed vectors of
the reference itself.  Tolerance of the bf16 path: max-abs 2e-2, mean-abs 2e-3."""
from pathlib import Path

import numpy as np
import pytest
import torch

import inputs
from oracle import attention as oa

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _check(out, want, max_abs=MAX_ABS, mean_abs=MEAN_ABS):
    diff = (out.float().cpu() - want.float()).abs()
    assert not torch.isnan(out.float()).any()
    assert diff.max().item() <= max_abs, diff.max().item()
    assert diff.mean().item() <= mean_abs, diff.mean().item()


def _status_ok():
    from mindiesd import _cabi
    assert _cabi.device_status() == 0


def test_matches_reference_vectors():
    """Same seeded inputs as tests/golden/make_golden.py fed to the reference's attention_math."""
    from mindiesd import _cabi
    z = np.load(G / "dense.npz")
    for tag, dtype, head_first, sq, skv in (("bf16_bsnd", torch.bfloat16, False, 160, 333),
                                            ("fp16_bnsd", torch.float16, True, 130, 257)):
        shape_q = (1, 2, sq, 128) if head_first else (1, sq, 2, 128)
        shape_k = (1, 2, skv, 128) if head_first else (1, skv, 2, 128)
        q, k, v = inputs.randn(21, *shape_q, dtype=dtype), inputs.randn(22, *shape_k, dtype=dtype), \
            inputs.randn(23, *shape_k, dtype=dtype)
        out = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), head_first=head_first)
        _check(out, torch.from_numpy(z[tag]))
    _status_ok()


@pytest.mark.parametrize("b,n,sq,skv,head_first", [
    (1, 1, 1, 1, True),          # a single token
    (1, 2, 127, 127, True),      # one ragged block
    (1, 2, 128, 128, False),     # exactly one block
    (2, 3, 129, 300, True),      # tails on both sides, batch > 1
    (1, 2, 256, 255, False),
    (1, 4, 1000, 1000, False),
    (2, 2, 2048, 640, True),
    (1, 1, 4100, 4100, True),
])
def test_shapes_and_tails(b, n, sq, skv, head_first):
    from mindiesd import _cabi
    shape_q = (b, n, sq, 128) if head_first else (b, sq, n, 128)
    shape_k = (b, n, skv, 128) if head_first else (b, skv, n, 128)
    q, k, v = (inputs.randn(40 + i, *s, dtype=torch.bfloat16) for i, s in enumerate((shape_q, shape_k, shape_k)))
    out, lse = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), head_first=head_first, want_lse=True)
    _check(out, oa.attention_math(q, k, v, head_first=head_first))
    qq, kk = (q, k) if head_first else (q.transpose(1, 2), k.transpose(1, 2))
    want_lse = torch.logsumexp(qq.float() @ kk.float().transpose(-1, -2) * 128 ** -0.5, -1)
    assert (lse.cpu() - want_lse).abs().max().item() < 1e-3
    _status_ok()


def test_config_c1_fp32_inputs():
    """B1 N12 S2048 D128 fp32 inputs (k with a per-channel offset): the kernel computes in bf16 on
    the tensor cores, so the fp32 inputs are rounded once and the comparison is made against the
    reference formula evaluated in fp32 on the UNROUNDED inputs, at the bf16 tolerance."""
    import workloads
    from mindiesd import _cabi
    q, k, v = workloads.make_qkv(workloads.C1, "cpu", seed=1)
    want = oa.attention_math(q, k, v, head_first=True)
    out = _cabi.attention(q.cuda().bfloat16(), k.cuda().bfloat16(), v.cuda().bfloat16(), head_first=True,
                          out_dtype=torch.float32)
    _check(out, want)
    _status_ok()


def test_strided_views_and_gqa():
    from mindiesd import _cabi
    # q/k/v as head slices of one packed [B, S, 3*N, D] buffer (the Ulysses receive buffer layout)
    packed = inputs.randn(50, 1, 700, 6, 128, dtype=torch.bfloat16).cuda()
    q, k, v = packed[:, :, 0:2], packed[:, :, 2:4], packed[:, :, 4:6]
    out = _cabi.attention(q, k, v, head_first=False)
    _check(out, oa.attention_math(q.cpu(), k.cpu(), v.cpu(), head_first=False))
    # grouped-query: 4 query heads share 2 kv heads
    q = inputs.randn(51, 1, 4, 512, 128, dtype=torch.bfloat16)
    k, v = inputs.randn(52, 1, 2, 640, 128, dtype=torch.bfloat16), inputs.randn(53, 1, 2, 640, 128, dtype=torch.bfloat16)
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda())
    _check(out, oa.attention_math(q, k.repeat_interleave(2, 1), v.repeat_interleave(2, 1), head_first=True))
    _status_ok()


def test_large_logits_do_not_overflow():
    """Scores far beyond the lag the running max is allowed: exercises the O rescale path."""
    from mindiesd import _cabi
    q = inputs.randn(60, 1, 1, 512, 128, dtype=torch.bfloat16) * 6
    k = inputs.randn(61, 1, 1, 1024, 128, dtype=torch.bfloat16) * 6
    k[:, :, 512:] *= 2  # later blocks raise the row max sharply
    v = inputs.randn(62, 1, 1, 1024, 128, dtype=torch.bfloat16)
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda())
    _check(out, oa.attention_math(q.float(), k.float(), v.float(), head_first=True), max_abs=4e-2, mean_abs=4e-3)
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("jump", ["lower_half", "upper_half", "one_key_lower", "one_key_upper", "every_block"])
def test_row_max_jumps_inside_a_key_block(jump, dtype):
    """The running max jumps far beyond its allowed lag in the first 64 keys of a block only, in the last 64
    only, at a single key, or block after block: every way the kernel's speculative exponentials can fail
    their row-sum test and be taken again."""
    from mindiesd import _cabi
    q = inputs.randn(63, 1, 2, 384, 128, dtype=dtype) * 4
    k = inputs.randn(64, 1, 2, 1280, 128, dtype=dtype) * 4
    v = inputs.randn(65, 1, 2, 1280, 128, dtype=dtype)
    if jump == "lower_half":
        k[:, :, 512:576] *= 3
    elif jump == "upper_half":
        k[:, :, 704:768] *= 3
    elif jump == "one_key_lower":
        k[:, :, 640 + 5] *= 6
    elif jump == "one_key_upper":
        k[:, :, 640 + 100] *= 6
    else:
        for b in range(1, 10):
            k[:, :, 128 * b + (37 if b % 2 else 91)] *= 1.0 + 0.6 * b
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda())
    _check(out, oa.attention_math(q.float(), k.float(), v.float(), head_first=True), max_abs=4e-2, mean_abs=4e-3)
    _status_ok()


def test_wan_1p3b_shape_rows():
    """Config C2 (B1 N12 S32760, RoPE'd q/k) on 2 heads: a fixed subset of query rows against the
    oracle, which is the full formula restricted to those rows."""
    import workloads
    from mindiesd import _cabi
    q, k, v = workloads.make_qkv(workloads.C2, "cpu", seed=2, heads=2)
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda())
    for rows in (slice(0, 256), slice(16384, 16640), slice(32760 - 200, 32760)):
        want = oa.attention_math_chunked(q, k, v, head_first=True, q_rows=rows)
        _check(out[:, :, rows], want)
    _status_ok()


def test_linearity_in_v_at_full_size():
    """Size-independent property at the Wan-14B sequence length (S = 75600, 2 heads): attention is
    linear in v, so out(v1 + v2) = out(v1) + out(v2) up to rounding, and out(ones) = ones."""
    import workloads
    from mindiesd import _cabi
    q, k, v = workloads.make_qkv(workloads.C3, "cuda", seed=3, heads=2)
    v2 = torch.roll(v, 1, dims=2)
    o1, o2 = _cabi.attention(q, k, v, out_dtype=torch.float32), _cabi.attention(q, k, v2, out_dtype=torch.float32)
    o12 = _cabi.attention(q, k, (v.float() + v2.float()).bfloat16(), out_dtype=torch.float32)
    assert (o12 - (o1 + o2)).abs().max().item() < 2e-2
    ones = _cabi.attention(q, k, torch.ones_like(v), out_dtype=torch.float32)
    assert (ones - 1).abs().max().item() < 1e-3
    _status_ok()


def test_rejects_bad_arguments():
    from mindiesd import _cabi
    q = torch.zeros(1, 1, 128, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q, q, q)  # head_dim 64
    q = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q, q, q, scale=-1.0)
