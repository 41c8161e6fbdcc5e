"""GPU tests of the Python layer API (the reference's function names and signatures) and of
torch.ops.mindiesd.*, checked against the CPU oracle."""
import pytest
import torch

import inputs
from oracle import attention as oa
from oracle import quant as oq
from oracle import rainfusion as orf

pytestmark = pytest.mark.gpu


def _close(out, want, max_abs=2e-2, mean_abs=2e-3):
    d = (out.float().cpu() - want.float()).abs()
    assert d.max().item() <= max_abs and d.mean().item() <= mean_abs, (d.max().item(), d.mean().item())


@pytest.mark.parametrize("head_first", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_attention_forward(head_first, dtype):
    from mindiesd import attention_forward
    shape = (2, 3, 333, 128) if head_first else (2, 333, 3, 128)
    q, k, v = (inputs.randn(120 + i, *shape, dtype=dtype) for i in range(3))
    want = oa.attention_math(q, k, v, head_first=head_first)
    for kwargs in ({}, {"opt_mode": "static"}, {"opt_mode": "manual", "op_type": "ascend_laser_attention", "layout": "BSND"}):
        out = attention_forward(q.cuda(), k.cuda(), v.cuda(), head_first=head_first, **kwargs)
        assert out.shape == q.shape and out.dtype == dtype
        _close(out, want)
    # the unfused formula runs on the same device and agrees with the kernel
    unfused = attention_forward(q.cuda(), k.cuda(), v.cuda(), fused=False, head_first=head_first)
    _close(unfused, want, 1e-2, 1e-3)


def test_attention_forward_errors():
    from mindiesd import attention_forward, ParametersInvalid
    q = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ParametersInvalid):
        attention_forward(q[0], q, q)
    with pytest.raises(ParametersInvalid):
        attention_forward(q, q, q, scale=1)
    with pytest.raises(ParametersInvalid):
        attention_forward(q, q, q, fused=1)
    with pytest.raises(ParametersInvalid):
        attention_forward(q, q, q, opt_mode="fastest")
    with pytest.raises(ParametersInvalid):
        attention_forward(q, q, q, opt_mode="manual", op_type="nope")
    with pytest.raises(ParametersInvalid) as e:
        attention_forward("q", q, q)
    assert str(e.value).startswith("[MIE06E000001]")


def test_la_operator():
    from mindiesd.layers import _custom_ops as ops
    q, k, v = (inputs.randn(130 + i, 1, 2, 300, 128, dtype=torch.float16) for i in range(3))
    lse, out = ops.laser_attention(q.cuda(), k.cuda(), v.cuda(), scale_value=128 ** -0.5, head_num=2)
    assert out.dtype == torch.float32 and lse.shape == (1, 2, 300)
    _close(out, oa.attention_math(q.float(), k.float(), v.float(), head_first=True), 5e-3, 5e-4)
    with pytest.raises(Exception):
        torch.ops.mindiesd.la(q.cuda()[0], k.cuda()[0], v.cuda()[0])


@pytest.mark.parametrize("d,dtype", [(64, torch.float16), (88, torch.float16), (40, torch.bfloat16), (96, torch.bfloat16)])
def test_head_dims_of_the_reference_shape_list(d, dtype):
    """Head dims 40, 64, 88 and 96 (the reference's shape list, tests/plugin/test_la.csv:2-13, at reduced
    sequence length and head count) through `la` and `attention_forward`: zero channels are appended up to
    the kernel's 128 and cut off again."""
    from mindiesd import attention_forward
    from mindiesd.layers import _custom_ops as ops
    q, k, v = (inputs.randn(140 + i, 2, 3, 530, d, dtype=dtype) for i in range(3))
    want = oa.attention_math(q.float(), k.float(), v.float(), scale=d ** -0.5, head_first=True)
    lse, out = ops.laser_attention(q.cuda(), k.cuda(), v.cuda(), scale_value=d ** -0.5, head_num=3)
    assert out.shape == q.shape and out.dtype == torch.float32 and lse.shape == (2, 3, 530)
    _close(out, want, 1e-2, 1e-3)
    out2 = attention_forward(q.cuda(), k.cuda(), v.cuda(), head_first=True)  # default scale 1 / sqrt(d)
    assert out2.shape == q.shape and out2.dtype == dtype
    _close(out2, want, 2e-2, 2e-3)
    out3 = attention_forward(*(x.transpose(1, 2).contiguous().cuda() for x in (q, k, v)))
    _close(out3.transpose(1, 2), want, 2e-2, 2e-3)


def _sparse_reference(q, k, v, grid, txt, sparsity, layout):
    """The reference pipeline on CPU with oracle pieces: permute, pool, mask, block-sparse attention,
    inverse permute.  BNSD fp32 result in the caller's token order."""
    if layout == "BSND":
        q, k, v = (x.transpose(1, 2) for x in (q, k, v))
    qp, kp = orf.pooled_means(q.float(), k.float(), grid, txt, 128, "BNSD")
    mask = orf.blockwise_mask(qp, kp, txt, sparsity, q.shape[-1] ** -0.5, 128, grid, "BNSD")
    qr, kr, vr = (orf.rearrange(x, grid, txt, "BNSD") for x in (q, k, v))
    nb = (qr.shape[2] + 127) // 128
    out = oa.block_sparse_attention(qr, kr, vr, mask[:, :, :nb, :nb].numpy())
    return orf.inv_rearrange(out, grid, txt, "BNSD"), mask


@pytest.mark.parametrize("sparse_type", ["rf_v2", "rf_v3"])
@pytest.mark.parametrize("layout,grid", [("BNSD", (3, 16, 24)), ("BSND", (3, 30, 52))])
def test_sparse_attention(sparse_type, layout, grid):
    from mindiesd import sparse_attention
    q, k = inputs.structured_qk(140, 2, grid, 128)
    v = inputs.randn(141, *q.shape, dtype=torch.bfloat16)
    if layout == "BSND":
        q, k, v = (x.transpose(1, 2).contiguous() for x in (q, k, v))
    want, _ = _sparse_reference(q, k, v, grid, 0, 0.6, layout)
    out = sparse_attention(q.cuda(), k.cuda(), v.cuda(), head_num=2, input_layout=layout, sparse_type=sparse_type,
                           block_size=128, latent_shape_q=grid, latent_shape_k=grid, sparsity=0.6)
    assert out.shape == q.shape
    _close(out.transpose(1, 2) if layout == "BSND" else out, want)


def test_sparse_attention_sparsity_zero_equals_dense():
    from mindiesd import sparse_attention, attention_forward
    grid = (2, 24, 45)
    q, k, v = (inputs.randn(150 + i, 1, 2, 2 * 24 * 45, 128, dtype=torch.bfloat16).cuda() for i in range(3))
    dense = attention_forward(q, k, v, head_first=True)
    for st in ("rf_v2", "rf_v3", None):
        out = sparse_attention(q, k, v, head_num=2, input_layout="BNSD", sparse_type=st, latent_shape_q=grid,
                               latent_shape_k=grid, sparsity=0.0)
        _close(out, dense.cpu(), 1e-2, 1e-3)


def test_bsa_v3_mask_cache_and_first_frame():
    from mindiesd.layers.flash_attn.sparse_flash_attn_rf_v3 import bsa_sparse_attention_v3
    grid = (3, 16, 24)
    q, k = inputs.structured_qk(160, 2, grid, 128)
    v = inputs.randn(161, *q.shape, dtype=torch.bfloat16)
    out, mask = bsa_sparse_attention_v3(q.cuda(), k.cuda(), v.cuda(), grid, sparsity=0.7, input_layout="BNSD")
    assert mask.dtype == torch.int8 and mask.shape == (1, 2, 9, 9)
    assert mask[:, :, :3].all() and mask[:, :, :, :3].all()  # 384 tokens per frame = 3 first-frame blocks
    out2, mask2 = bsa_sparse_attention_v3(q.cuda(), k.cuda(), v.cuda(), grid, sparsity=0.7, input_layout="BNSD",
                                          cached_mask=mask)
    assert mask2 is mask and torch.equal(out2, out)


def test_rf_v2_helpers_keep_reference_semantics():
    from mindiesd.layers.flash_attn import sparse_flash_attn_rf_v2 as rf
    grid, txt = (3, 30, 52), 256
    q, k = inputs.structured_qk(170, 2, grid, 64, txt)
    v = inputs.randn(171, *q.shape, dtype=torch.bfloat16)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    q_, k_, v_, pool = rf.do_tensor_rearrange_pooling(qc, kc, vc, txt, 128, grid, grid, "BNSD")
    assert torch.equal(q_.cpu(), orf.rearrange(q, grid, txt, "BNSD"))
    assert pool.shape == (3, 2, 37 + 2, 64)
    assert torch.equal(rf.do_tensor_inv_rearrange(q_, txt, grid, grid, "BNSD"), qc)
    mask = rf.get_blockwise_mask(pool, txt, 0.5, 64 ** -0.5, 128, grid, grid, "BNSD", return_binary=True)
    qp, kp = orf.pooled_means(q.float(), k.float(), grid, txt, 128, "BNSD")
    assert torch.equal(mask.cpu(), orf.blockwise_mask(qp, kp, txt, 0.5, 64 ** -0.5, 128, grid, "BNSD"))
    sel, num = rf.get_blockwise_mask(pool, txt, 0.5, 64 ** -0.5, 128, grid, grid, "BNSD")
    assert sel.shape == (39, 2, 39) and num.shape == (39, 2)
    assert torch.equal(rf.get_mask_index(mask.bool())[0].transpose(0, 1).cpu(), sel.cpu())
    x = inputs.randn(172, 1, 2, 300, 16).cuda()
    assert (rf.avgpool(x, 128, "BNSD").cpu() - orf.avgpool(x.cpu(), 128, "BNSD")).abs().max().item() < 1e-6
    y = rf.rearrange_with_remaining(x[:, :, :128], (2, 8, 8), (2, 8, 8), "BNSD")
    assert torch.equal(rf.inv_rearrange_with_remaining(y, (2, 8, 8), (2, 8, 8), "BNSD"), x[:, :, :128])


def test_block_sparse_operator_errors_and_lse():
    from mindiesd.layers import _custom_ops as ops
    q, k, v = (inputs.randn(180 + i, 1, 2, 256, 128, dtype=torch.bfloat16).cuda() for i in range(3))
    mask = torch.ones(1, 2, 2, 2, dtype=torch.int8, device="cuda")
    with pytest.raises(RuntimeError):
        ops.block_sparse_attention(q, q, q, mask, q_input_layout="BSND", kv_input_layout="BSND")
    with pytest.raises(RuntimeError):
        ops.block_sparse_attention(q, q, q, mask, q_input_layout="TND", kv_input_layout="TND")  # lengths required
    out, lse = ops.block_sparse_attention(q, k, v, mask, num_key_value_heads=2, scale_value=128 ** -0.5,
                                          actual_seq_lengths=[256], actual_seq_lengths_kv=[256], softmax_lse_flag=1)
    assert lse.shape == (1, 2, 256, 1) and lse.dtype == torch.float32
    _close(out, oa.attention_math(q.cpu(), k.cpu(), v.cpu(), head_first=True))
    with pytest.raises(RuntimeError):
        ops.rain_fusion_attention(q, q, q, mask, mask, [128, 128], q_input_layout="BSND", kv_input_layout="BSND")


def test_fp8_hook():
    from mindiesd import FP8RotateQuantFA
    from mindiesd.layers.quant.block_quant import fa_block_quant_preprocess
    torch.manual_seed(0)
    rot, _ = torch.linalg.qr(torch.randn(128, 128))
    weights = {"blk.q_rot": rot, "blk.k_rot": rot}  # one orthogonal rotation on q and k leaves q k^T unchanged
    for layout, fa in (("BNSD", FP8RotateQuantFA("blk", weights).cuda()), ("BSND", FP8RotateQuantFA().cuda())):
        shape = (1, 2, 1000, 128) if layout == "BNSD" else (1, 1000, 2, 128)
        q, k, v = (inputs.randn(190 + i, *shape, dtype=torch.bfloat16) for i in range(3))
        out = fa(q.cuda(), k.cuda(), v.cuda(), layout=layout)
        assert out.shape == q.shape and out.dtype == torch.bfloat16
        want = oa.attention_math(q.float(), k.float(), v.float(), head_first=layout == "BNSD")
        assert oq.cosine(out.cpu(), want) >= 0.995
    xq, xs = fa_block_quant_preprocess(q.cuda(), block_size=256, layout="BSND")
    assert xq.shape == (1, 2, 1000, 128) and xs.shape == (1, 2, 4, 1) and xq.dtype == torch.float8_e4m3fn
    with pytest.raises(ValueError):
        fa(q.cuda(), k.cuda(), v.cuda(), layout="SBH")


def test_ops_trace_with_fake_tensors():
    from torch._subclasses.fake_tensor import FakeTensorMode
    import mindiesd  # noqa: F401
    with FakeTensorMode():
        q = torch.empty(1, 2, 1024, 128, dtype=torch.bfloat16, device="cuda")
        out, lse = torch.ops.mindiesd.block_sparse_attention(q, q, q, None)
        assert out.shape == q.shape and lse.shape == (1, 2, 1024, 1)
        lse, out = torch.ops.mindiesd.la(q, q, q)
        assert out.dtype == torch.float32
        smask, sct = torch.ops.mindiesd.sparse_block_estimate(q, q, causal=False)
        assert smask.shape == (1, 2, 8, 32) and smask.dtype == torch.int8 and sct.shape == (1, 2, 8)
        out = torch.ops.mindiesd.ada_block_sparse_attention(q, q, q, smask, sct, causal=False)
        assert out.shape == q.shape and out.dtype == q.dtype


def test_attention_forward_host_pipeline():
    from mindiesd import attention_forward_host, ParametersInvalid
    q, k, v = (inputs.randn(210 + i, 1, 6, 700, 128, dtype=torch.bfloat16).pin_memory() for i in range(3))
    want = oa.attention_math(q, k, v, head_first=True)
    for chunks in (1, 3, 6, None, 3):  # 6: more chunks than staging slots; None: the default; 3 again: buffers re-made
        out = attention_forward_host(q, k, v, head_chunks=chunks)
        assert out.is_pinned() and not out.is_cuda
        _close(out, want)
    first = attention_forward_host(q, k, v, head_chunks=6).clone()
    assert torch.equal(attention_forward_host(q, k, v, head_chunks=6), first)  # staging reuse across calls
    with pytest.raises(ParametersInvalid):
        attention_forward_host(q, k, v, head_chunks=4)
    with pytest.raises(ParametersInvalid):
        attention_forward_host(q.cuda(), k, v)


def test_attention_forward_varlen():
    from mindiesd import attention_forward_varlen, ParametersInvalid
    lens_q, lens_k = [300, 1, 515], [300, 77, 640]
    q = inputs.randn(220, sum(lens_q), 2, 128, dtype=torch.bfloat16)
    k, v = (inputs.randn(221 + i, sum(lens_k), 2, 128, dtype=torch.bfloat16) for i in range(2))
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32)
    out = attention_forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu_q, cu_k)
    assert out.shape == q.shape
    for i in range(3):
        qs, ks = slice(int(cu_q[i]), int(cu_q[i + 1])), slice(int(cu_k[i]), int(cu_k[i + 1]))
        want = oa.attention_math(q[qs][None], k[ks][None], v[ks][None], head_first=False)[0]
        _close(out[qs], want)
    with pytest.raises(ParametersInvalid):
        attention_forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu_q, cu_k, max_seqlen_q=515)
    with pytest.raises(ParametersInvalid):
        attention_forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu_q, cu_k, dropout_p=0.1)
    with pytest.raises(ParametersInvalid):
        attention_forward_varlen(q.cuda()[None], k.cuda(), v.cuda(), cu_q, cu_k)
