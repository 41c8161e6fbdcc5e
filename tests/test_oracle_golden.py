"""Pins the CPU oracle against vectors produced by MindIE-SD's own Python code
(tests/golden/make_golden.py).  CPU only."""
from pathlib import Path

import numpy as np
import pytest
import torch

import inputs
from oracle import ada_bsa as oada
from oracle import attention as oa
from oracle import rainfusion as orf

G = Path(__file__).resolve().parent / "golden"


def _unpack(z, name):
    shape = tuple(z[f"{name}_mask_shape"])
    n = int(np.prod(shape))
    return np.unpackbits(z[f"{name}_mask_bits"])[:n].reshape(shape).astype(np.int8)


def test_permutation_matches_reference():
    z = np.load(G / "permutation.npz")
    for (t, h, w) in inputs.PERM_GRIDS:
        src = orf.window_permutation(t, h, w)
        for layout in ("BNSD", "BSND"):
            assert np.array_equal(src, z[f"{t}x{h}x{w}_{layout}"].astype(np.int64)), (t, h, w, layout)
        assert np.array_equal(np.sort(src), np.arange(t * h * w))


@pytest.mark.parametrize("layout", ["BNSD", "BSND"])
def test_rearrange_round_trip(layout):
    for (t, h, w) in inputs.PERM_GRIDS[:4]:
        for txt in (0, 37):
            s = t * h * w + txt
            x = inputs.randn(1, 1, 2, s, 8)
            if layout == "BSND":
                x = x.transpose(1, 2).contiguous()
            y = orf.rearrange(x, (t, h, w), txt, layout)
            assert torch.equal(orf.inv_rearrange(y, (t, h, w), txt, layout), x)
            dim = 2 if layout == "BNSD" else 1
            if txt:  # text moves from the front to the back
                assert torch.equal(y.narrow(dim, s - txt, txt), x.narrow(dim, 0, txt))


def test_avgpool_matches_reference():
    z = np.load(G / "avgpool.npz")
    x = inputs.randn(3, 1, 2, 300, 16)
    assert np.array_equal(orf.avgpool(x, 128, "BNSD").numpy(), z["bnsd"])
    assert np.array_equal(orf.avgpool(x.transpose(1, 2).contiguous(), 128, "BSND").numpy(), z["bsnd"])
    # known answer of the reference's own test: block means of 0..255
    t = torch.arange(256, dtype=torch.float32).reshape(1, 1, 256, 1)
    out = orf.avgpool(t, 128, "BNSD")
    assert abs(out[0, 0, 0, 0].item() - 63.5) < 1e-4 and abs(out[0, 0, 1, 0].item() - 191.5) < 1e-4
    assert orf.avgpool(torch.ones(1, 1, 64, 4), 128, "BNSD").shape == (1, 1, 1, 4)  # tail only


@pytest.mark.parametrize("case", inputs.MASK_CASES, ids=[c[0] for c in inputs.MASK_CASES])
def test_blockwise_mask_matches_reference(case):
    name, grid, txt, heads, dim, sparsity, layout, seed = case
    z = np.load(G / "mask.npz")
    want = _unpack(z, name)
    q, k = inputs.structured_qk(seed, heads, grid, dim, txt)
    q, k = q.float(), k.float()
    if layout == "BSND":
        q, k = q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous()
    qp, kp = orf.pooled_means(q, k, grid, txt, 128, layout)
    if f"{name}_qpool" in z.files:
        assert np.array_equal(qp.numpy(), z[f"{name}_qpool"])
    scale = dim ** -0.5
    got = orf.blockwise_mask(qp, kp, txt, sparsity, scale, 128, grid, layout)
    assert np.array_equal(got.numpy(), want)
    # thresholding the raw float64 scores keeps the same set (the softmax is monotone per row)
    raw = orf.blockwise_mask(qp, kp, txt, sparsity, scale, 128, grid, layout, use_softmax=False)
    assert np.array_equal(raw.numpy(), want)
    if f"{name}_select_idx" in z.files:
        sel, num = orf.select_lists(got)
        assert np.array_equal(sel.numpy(), z[f"{name}_select_idx"].astype(np.int64))
        assert np.array_equal(num.numpy(), z[f"{name}_select_num"].astype(np.int64))


def test_mask_index_matches_reference():
    z = np.load(G / "mask_index.npz")
    idx, num = orf.mask_index(z["mask"])
    assert np.array_equal(idx.numpy(), z["index"].astype(np.int64))
    assert np.array_equal(num.numpy(), z["mask"].sum(-1))
    # known answers of the reference's own test
    m = np.zeros((1, 1, 4, 4), dtype=bool)
    m[0, 0, 0, 0] = m[0, 0, 0, 2] = True
    idx, _ = orf.mask_index(m)
    assert idx[0, 0, 0].tolist() == [0, 2, -1, -1]
    idx, _ = orf.mask_index(np.ones((1, 1, 4, 4), dtype=bool))
    assert idx[0, 0, 3].tolist() == [0, 1, 2, 3]


def test_dense_attention_matches_reference():
    z = np.load(G / "dense.npz")
    for tag, dtype, head_first, sq, skv in (("fp32_bnsd", torch.float32, True, 200, 200),
                                            ("bf16_bsnd", torch.bfloat16, False, 160, 333),
                                            ("fp16_bnsd", torch.float16, True, 130, 257)):
        shape_q = (1, 2, sq, 128) if head_first else (1, sq, 2, 128)
        shape_k = (1, 2, skv, 128) if head_first else (1, skv, 2, 128)
        q, k, v = inputs.randn(21, *shape_q, dtype=dtype), inputs.randn(22, *shape_k, dtype=dtype), \
            inputs.randn(23, *shape_k, dtype=dtype)
        want = torch.from_numpy(z[tag])
        got = oa.attention_math(q, k, v, head_first=head_first).float()
        assert torch.equal(got, want), tag
        chunked = oa.attention_math_chunked(q, k, v, head_first=head_first, rows=64).float()
        tol = 0 if dtype == torch.float32 else 2e-2  # chunking may change the blocking of the low-precision GEMM
        assert (chunked - want).abs().max().item() <= max(tol, 1e-6), tag


def test_block_sparse_attention_matches_reference():
    z = np.load(G / "block_sparse.npz")
    q, k, v = (inputs.randn(31 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    got = oa.block_sparse_attention(q, k, v, z["mask"], 128)
    want = torch.from_numpy(z["out"])
    assert (got - want).abs().max().item() < 1e-6
    assert torch.count_nonzero(want[0, 0, 128:256]) == 0  # the row that keeps nothing
    assert oa.ref_compare(want, got, 2 ** -6)[1]


def test_sparse_block_estimate_matches_reference():
    """The restated estimator against the reference's numpy golden, bit for bit (the golden's mixed
    float64 / float32 comparison included), and the single-precision decision against it: the two
    may differ in one block per row, the one whose score is the row's guard."""
    z = np.load(G / "estimate.npz")
    for (name, grid, heads, threshold, row_sparse, seed) in inputs.ESTIMATE_CASES:
        q, k = inputs.structured_qk(seed, heads, grid, 128)
        q, k = q.float().numpy(), k.float().numpy()
        shape = tuple(z[f"{name}_shape"])
        want = np.unpackbits(z[f"{name}_bits"])[:int(np.prod(shape))].reshape(shape).astype(bool)
        got, count, score = oada.sparse_block_estimate(q, k, 128 ** -0.5 / 8, threshold, row_sparse,
                                                       golden_rounding=True)
        assert np.array_equal(got, want), (name, int((got != want).sum()))
        assert np.array_equal(count, got.sum(-1)), name
        assert got[..., 0].all() and got[..., -1].all(), name
        assert np.allclose(score.sum(-1)[..., :-1], 16.0, atol=1e-9), name  # 16 rows of softmax mass per block
        plain, _, _ = oada.sparse_block_estimate(q, k, 128 ** -0.5 / 8, threshold, row_sparse)
        assert not (want & ~plain).any(), name
        assert (plain & ~want).sum(-1).max() <= 1, name


def test_sparse_block_estimate_causal_matches_reference():
    """The causal branch of the restated estimator against the reference's numpy golden run with
    causal=True (tests/golden/ada_causal.npz), bit for bit."""
    z = np.load(G / "ada_causal.npz")
    for (name, grid, heads, threshold, row_sparse, seed) in inputs.ESTIMATE_CASES:
        q, k = inputs.structured_qk(seed, heads, grid, 128)
        q, k = q.float().numpy(), k.float().numpy()
        shape = tuple(z[f"{name}_shape"])
        want = np.unpackbits(z[f"{name}_bits"])[:int(np.prod(shape))].reshape(shape).astype(bool)
        got, count, _ = oada.sparse_block_estimate(q, k, 128 ** -0.5 / 8, threshold, row_sparse, golden_rounding=True,
                                                   causal=True)
        assert np.array_equal(got, want), (name, int((got != want).sum()))
        assert np.array_equal(count, got.sum(-1)), name
        assert not np.triu(got, 1).any(), name      # nothing above the diagonal
        assert got[..., 0].all(), name              # the first block always stays
        plain, _, _ = oada.sparse_block_estimate(q, k, 128 ** -0.5 / 8, threshold, row_sparse, causal=True)
        assert not (want & ~plain).any(), name
        assert (plain & ~want).sum(-1).max() <= 1, name


def test_ada_attention_causal_golden_is_token_level_causality_when_the_diagonal_is_kept():
    """ada_block_sparse_attention_cpu(causal=True) adds a triangle to the LAST kept columns of a row
    (tests/plugin/test_adablocksparseattention.py:69-72).  For a mask that keeps every row's own block
    that is ordinary token-level causality inside the kept blocks, which is what the oracle's
    attention_math with a keep-mask computes."""
    z = np.load(G / "ada_causal.npz")
    q, k, v = (inputs.randn(41 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    mask = torch.from_numpy(z["attention_mask"])[..., :3]
    want = torch.from_numpy(z["attention_out"])
    tri = torch.tril(torch.ones(300, 300, dtype=torch.bool))
    for n in range(2):
        keep = mask[0, n].bool().repeat_interleave(128, 0).repeat_interleave(128, 1)[:300, :300] & tri
        got = oa.attention_math(q[:, n:n + 1].float(), k[:, n:n + 1].float(), v[:, n:n + 1].float(), attn_mask=keep,
                                head_first=True)
        assert (got - want[:, n:n + 1]).abs().max().item() < 1e-4, n


def test_ada_attention_golden_is_the_block_sparse_golden():
    z = np.load(G / "ada_attention.npz")
    q, k, v = (inputs.randn(41 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    got = oa.block_sparse_attention(q, k, v, z["mask"], 128)
    want = torch.from_numpy(z["out"])
    assert (got - want).abs().max().item() < 1e-6
    assert torch.count_nonzero(want[0, 1, 256:]) == 0  # the row that keeps nothing


def test_temporal_band_extension():
    band = orf.temporal_band((4, 16, 16), 0, 1)  # 256 tokens per frame, two blocks per frame
    assert band.shape == (8, 8)
    assert band[0, 3] and not band[0, 4] and band[7, 4] and not band[7, 3]
    assert np.array_equal(band, band.T)


def test_rope_oracle_matches_reference_vectors():
    """oracle.rope against rotary_position_embedding(fused=False) of the reference (rope.npz)."""
    import make_golden
    from oracle import rope as orope
    z = np.load(G / "rope.npz")
    for name, xs, head_first, ts, tdt, xdt, mode, seed in make_golden.ROPE_CASES:
        x = inputs.randn(seed, *xs, dtype=xdt)
        cos, sin = inputs.randn(seed + 100, *ts, dtype=tdt), inputs.randn(seed + 200, *ts, dtype=tdt)
        got = orope.rotary_position_embedding(x, cos, sin, mode, head_first)
        assert got.dtype == xdt
        assert torch.equal(got.float(), torch.from_numpy(z[name])), name
