"""The three Wan2.1-14B 720p configurations at their own sequence length (S = 75600 = 21x45x80, 591 blocks of
128, tail 80) on two heads, checked row-for-row against the CPU oracle on fixed slices of query rows:
the oracle evaluates the full formula for exactly those rows against all 75600 keys.

    dense bf16 (config 3's tensors)    max-abs 2e-2, mean-abs 2e-3 vs oracle.attention_math_chunked
    FP8 (config 4's generator: N(0,1), 1 % of the channels x8)   cosine >= 0.995 vs fp32 attention of the
                                        unquantised inputs, through the FP8RotateQuantFA hook
    RainFusion block-sparse at the 591-block grid   same tolerance vs oracle.block_sparse_attention on the
                                        mask the GPU built (which test_gpu_rainfusion checks bit for bit)
"""
import pytest
import torch

import workloads
from oracle import attention as oa
from oracle import quant as oq

pytestmark = pytest.mark.gpu
SLICES = (slice(0, 256), slice(37760, 38016), slice(75600 - 256, 75600))  # first tiles, middle, ragged tail


def _check(out, want, max_abs=2e-2, mean_abs=2e-3):
    diff = (out.float().cpu() - want.float()).abs()
    assert not torch.isnan(out.float()).any()
    assert diff.max().item() <= max_abs, diff.max().item()
    assert diff.mean().item() <= mean_abs, diff.mean().item()


def test_dense_rows_at_wan_14b_720p():
    from mindiesd import _cabi
    q, k, v = workloads.make_qkv(workloads.C3, "cuda", seed=5, heads=2)
    out = _cabi.attention(q, k, v)
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    for rows in SLICES:
        want = oa.attention_math_chunked(qc, kc, vc, head_first=True, q_rows=rows)
        _check(out[:, :, rows], want)
    assert _cabi.device_status() == 0


def test_fp8_rows_at_wan_14b_720p():
    from mindiesd import _cabi, FP8RotateQuantFA
    q, k, v = workloads.make_qkv(workloads.C4, "cuda", seed=6, heads=2)
    qc, kc, vc = q.cpu().float(), k.cpu().float(), v.cpu().float()
    for per_channel in (True, False):  # per-channel v scales (the benchmark's contract) and the hook's 256-token blocks
        out = FP8RotateQuantFA(v_per_channel=per_channel).cuda()(q, k, v, layout="BNSD")
        assert out.dtype == q.dtype and out.shape == q.shape
        got, want = [], []
        for rows in SLICES:
            want.append(oa.attention_math_chunked(qc, kc, vc, head_first=True, q_rows=rows))
            got.append(out[:, :, rows].float().cpu())
        cos = oq.cosine(torch.cat(got, 2), torch.cat(want, 2))
        assert cos >= 0.995, (per_channel, cos)
    assert _cabi.device_status() == 0


def test_block_sparse_rows_at_wan_14b_720p():
    from mindiesd import _cabi
    grid = workloads.C3.grid
    q, k, v = workloads.make_qkv(workloads.C3, "cuda", seed=7, heads=2)
    mask = _cabi.rf_block_mask(q, k, grid, 0, 0.75, True)
    qp, kp, vp = (_cabi.rf_rearrange(x, grid, 0, True) for x in (q, k, v))
    out = _cabi.attention(qp, kp, vp, block_mask=mask, out_dtype=torch.float32)
    blocks = (0, 28, 300, 590)  # first frame (dense row), the block that straddles frames 0/1, middle, ragged tail
    want = oa.block_sparse_attention(qp.cpu(), kp.cpu(), vp.cpu(), mask.cpu().numpy(), q_blocks=blocks)
    for qb in blocks:
        rows = slice(qb * 128, min((qb + 1) * 128, 75600))
        _check(out[:, :, rows], want[:, :, rows])
        eb, ok, worst = oa.ref_compare(want[:, :, rows], out[:, :, rows].cpu(), 2 ** -6)  # the reference's own bar
        assert ok, (qb, eb, worst)
    assert _cabi.device_status() == 0
