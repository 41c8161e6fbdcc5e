"""GPU checks of the e4m3 quantiser and the FP8 attention kernel through the C ABI.
Bar: cosine similarity >= 0.995 against fp32 attention of the unquantised inputs."""
import pytest
import torch

import inputs
from oracle import attention as oa
from oracle import quant as oq

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("row_block", [128, 256, 512])
def test_block_quant_matches_oracle(row_block):
    from mindiesd import _cabi
    x = inputs.randn(90, 1, 3, 1000, 128, dtype=torch.bfloat16) * 3
    x[:, :, 256:384] = 0  # an all-zero block keeps scale 1
    want_q, want_s = oq.block_quant(x, row_block)
    got_q, got_s = _cabi.fa_block_quant(x.cuda(), row_block)
    assert torch.equal(got_s.cpu(), want_s)
    assert torch.equal(got_q.cpu().view(torch.uint8), want_q.view(torch.uint8))
    # BSND input, same bytes out
    got_q2, got_s2 = _cabi.fa_block_quant(x.transpose(1, 2).contiguous().cuda(), row_block, head_first=False)
    assert torch.equal(got_q2, got_q) and torch.equal(got_s2, got_s)


def test_channel_quant_matches_oracle():
    from mindiesd import _cabi
    x = inputs.randn(91, 2, 2, 777, 128, dtype=torch.float16)
    x[..., 5] *= 8
    want_q, want_s = oq.channel_quant(x)
    got_q, got_s = _cabi.fa_block_quant(x.cuda(), per_channel=True)
    assert torch.equal(got_s.cpu(), want_s)
    assert torch.equal(got_q.cpu().view(torch.uint8), want_q.view(torch.uint8))


def test_rotated_block_quant_close_to_oracle():
    """The kernel's tensor-core product with the +-1 matrix (1/sqrt(128) folded into the scale) and the
    oracle's fp32 matrix product round differently, so the comparison
    is on dequantised values: within one e4m3 step (2^-3 relative) of the oracle's."""
    from mindiesd import _cabi
    x = inputs.randn(95, 1, 2, 600, 128, dtype=torch.bfloat16)
    x[..., 3] *= 8
    want_q, want_s = oq.block_quant(x, 128, rotate=True)
    got_q, got_s = _cabi.fa_block_quant(x.cuda(), 128, rotate=True)
    assert torch.allclose(got_s.cpu(), want_s, rtol=1e-5)
    deq = lambda q8, sc: q8.float() * sc.repeat_interleave(128, 2)[:, :, :600, None]  # noqa: E731
    a, b = deq(got_q.cpu(), got_s.cpu()), deq(want_q, want_s)
    assert ((a - b).abs() <= 0.13 * b.abs() + 1e-3).all()
    # the rotation is orthogonal: norms are preserved up to the quantisation error
    assert abs(a.norm().item() / x.float().norm().item() - 1) < 0.01


@pytest.mark.parametrize("row_block,dtype,head_first", [(128, torch.bfloat16, True), (256, torch.float16, False),
                                                        (512, torch.bfloat16, True)])
def test_learned_rotation_fused_with_quant(row_block, dtype, head_first):
    """x @ rot on the tensor cores inside the quantiser against the oracle's quantisation of the exact
    product.  The kernel accumulates the products in fp32 in its own order, so scales agree to 1e-5
    and the e4m3 bytes may differ where a value sits on a rounding boundary: compared on dequantised
    values, within one e4m3 step."""
    from mindiesd import _cabi
    s = 1000
    x = inputs.randn(96, 2, 3, s, 128, dtype=dtype)
    x[..., 9] *= 8
    rot = torch.linalg.qr(inputs.randn(97, 128, 128).double())[0].to(dtype)  # a random orthogonal matrix
    y = (x.double() @ rot.double()).float()
    want_q, want_s = oq.block_quant(y, row_block)
    xin = x if head_first else x.transpose(1, 2).contiguous()
    got_q, got_s = _cabi.fa_rotate_quant(xin.cuda(), rot.cuda(), row_block, head_first=head_first)
    assert _cabi.device_status() == 0
    assert got_q.shape == (2, 3, s, 128) and got_s.shape == want_s.shape
    assert torch.allclose(got_s.cpu(), want_s, rtol=1e-5)
    deq = lambda q8, sc: q8.float() * sc.repeat_interleave(row_block, 2)[:, :, :s, None]  # noqa: E731
    a, b = deq(got_q.cpu(), got_s.cpu()), deq(want_q, want_s)
    assert ((a - b).abs() <= 0.13 * b.abs() + 1e-3).all()
    same = (got_q.cpu().view(torch.uint8) == want_q.view(torch.uint8)).float().mean().item()
    assert same > 0.99, same
    # through the operator and the layer function
    import mindiesd  # noqa: F401
    from mindiesd.layers.quant.block_quant import fa_block_quant_preprocess
    q2, s2 = fa_block_quant_preprocess(xin.cuda(), block_size=row_block, layout="BNSD" if head_first else "BSND",
                                       rot=rot.cuda())
    assert torch.equal(q2.view(torch.uint8), got_q.view(torch.uint8)) and torch.equal(s2.squeeze(-1), got_s)


def test_fp8_hook_with_learned_rotations():
    """FP8RotateQuantFA with q_rot / k_rot weights (the reference's configuration) keeps the cosine bar."""
    from mindiesd import FP8RotateQuantFA
    q, k, v = _outlier_inputs(120, 2, 1500)
    rot = torch.linalg.qr(inputs.randn(123, 128, 128).double())[0].to(torch.bfloat16)
    hook = FP8RotateQuantFA("blk", {"blk.q_rot": rot, "blk.k_rot": rot}, v_per_channel=True).cuda()
    out = hook(q.cuda(), k.cuda(), v.cuda(), layout="BNSD")
    want = oa.attention_math(q.float(), k.float(), v.float(), head_first=True)
    assert out.dtype == torch.bfloat16 and out.shape == q.shape
    assert oq.cosine(out.cpu(), want) >= 0.995


def _outlier_inputs(seed, n, s):
    q, k, v = (inputs.randn(seed + i, 1, n, s, 128, dtype=torch.bfloat16) for i in range(3))
    for x in (q, k, v):
        x[..., 17] *= 8  # about 1 % of the channels carry 8x larger values
    return q, k, v


@pytest.mark.parametrize("v_mode", ["channel", "block256"])
@pytest.mark.parametrize("s", [300, 2048, 5000])
def test_fp8_attention_cosine(s, v_mode):
    from mindiesd import _cabi
    q, k, v = _outlier_inputs(100, 2, s)
    want = oa.attention_math(q.float(), k.float(), v.float(), head_first=True)
    q8, qs = _cabi.fa_block_quant(q.cuda(), 128, rotate=True)
    k8, ks = _cabi.fa_block_quant(k.cuda(), 256, rotate=True)
    if v_mode == "channel":
        v8, vs = _cabi.fa_block_quant(v.cuda(), per_channel=True)
        vb = 0
    else:
        v8, vs = _cabi.fa_block_quant(v.cuda(), 256)
        vb = 256
    out = _cabi.attention(q8, k8, v8, q_scale=qs, k_scale=ks, v_scale=vs, k_scale_block=256, v_scale_block=vb,
                          out_dtype=torch.bfloat16)
    cos = oq.cosine(out.cpu(), want)
    assert cos >= 0.995, cos
    assert _cabi.device_status() == 0


def test_fp8_attention_k_block_128():
    from mindiesd import _cabi
    q, k, v = _outlier_inputs(110, 1, 1111)
    want = oa.attention_math(q.float(), k.float(), v.float(), head_first=True)
    q8, qs = _cabi.fa_block_quant(q.cuda(), 128, rotate=True)
    k8, ks = _cabi.fa_block_quant(k.cuda(), 128, rotate=True)
    v8, vs = _cabi.fa_block_quant(v.cuda(), per_channel=True)
    out = _cabi.attention(q8, k8, v8, q_scale=qs, k_scale=ks, v_scale=vs, k_scale_block=128, v_scale_block=0,
                          out_dtype=torch.float32)
    assert oq.cosine(out.cpu(), want) >= 0.995
