"""GPU parity of adaptive block-sparse attention: the cumulative-mass block estimate (through the C
ABI and through torch.ops.mindiesd.sparse_block_estimate) and the attention over its mask.

The estimator's decision is a threshold on floating-point sums, so parity is stated as the
reference's own plugin test states it (tests/plugin/test_sparseblockestimate.py:225-239: fewer than
2 % of the selected blocks differ, fewer than 1 % are omitted) and, more strictly, as: every row that
differs from the oracle's is a correct decision up to rounding (a score within 1e-3 of the row's
guard, or a running sum within 1e-5 of the limit), and at most 1 % of the kept blocks differ."""
from pathlib import Path

import numpy as np
import pytest
import torch

import inputs
from oracle import ada_bsa as oada
from oracle import attention as oa

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"
SCALE = 128 ** -0.5 / 8


def _row_explained(got, score, threshold, row_sparse, keep_sink=True, keep_recent=True):
    """True if a mask row that differs from the oracle's is still a correct decision up to rounding:
    the kept prefix may be one block longer or shorter when its running sum is within 1e-5 of the
    limit, and a block may fall on either side when its score is within 1e-3 of the guard."""
    cols = score.size
    row = np.array(score, dtype=np.float64)
    if keep_recent:
        row[-1] = 0
    order = -np.sort(-row)
    cum, limit = order.cumsum(), threshold * order.sum()
    k0 = int((cum < limit).sum())
    plausible = {k0}
    if k0 >= 1 and cum[k0 - 1] >= limit * (1 - 1e-5):
        plausible.add(k0 - 1)
    if k0 < cols and cum[k0] <= limit * (1 + 1e-5):
        plausible.add(k0 + 1)
    for k in plausible:
        cnt = k + 1
        if row_sparse > 0 and cnt > row_sparse * cols:
            cnt = int(row_sparse * cols)
        guard = order[max(1, min(cnt, cols)) - 1]
        keep = row >= guard
        if keep_sink:
            keep[0] = True
        if keep_recent:
            keep[-1] = True
        bad = np.flatnonzero(keep != got)
        if all(abs(row[j] - guard) <= 1e-3 * guard for j in bad):
            return True
    return False


def _explained_by_ties(got, want, score, threshold, row_sparse, name, **flags):
    """Asserts that every row of `got` that differs from `want` is a correct decision up to rounding;
    returns the number of differing bits."""
    for (b, n, i) in np.argwhere((got != want).any(-1)):
        assert _row_explained(got[b, n, i], score[b, n, i], threshold, row_sparse, **flags), (name, b, n, i)
    return int((got != want).sum())


@pytest.mark.parametrize("case", inputs.ESTIMATE_CASES, ids=[c[0] for c in inputs.ESTIMATE_CASES])
def test_estimate_against_oracle_and_reference_vectors(case):
    import mindiesd  # noqa: F401
    from mindiesd import _cabi
    name, grid, heads, threshold, row_sparse, seed = case
    q, k = inputs.structured_qk(seed, heads, grid, 128)
    s = q.shape[2]
    want, count, score = oada.sparse_block_estimate(q.float().numpy(), k.float().numpy(), SCALE, threshold, row_sparse)
    blocks = want.shape[-1]
    if s % 8 == 0:
        mask, cnt = _cabi.sparse_block_estimate(q.cuda(), k.cuda(), SCALE, threshold, row_sparse)
    else:  # the operator completes the last group with zero tokens
        mask, cnt = torch.ops.mindiesd.sparse_block_estimate(
            query=q.cuda(), key=k.cuda(), input_layout="BNSD", stride=8, sparse_size=128, num_heads=heads,
            num_key_value_heads=heads, scale_value=SCALE, threshold=threshold, causal=False, keep_sink=True,
            keep_recent=True, row_sparse=row_sparse)
    assert _cabi.device_status() == 0
    assert mask.shape == (1, heads, blocks, (blocks + 31) // 32 * 32) and mask.dtype == torch.int8
    assert cnt.shape == (1, heads, blocks) and cnt.dtype == torch.int32
    m = mask.cpu().numpy()
    assert not m[..., blocks:].any()
    got = m[..., :blocks].astype(bool)
    assert np.array_equal(cnt.cpu().numpy(), got.sum(-1))
    assert got[..., 0].all() and got[..., -1].all()
    ndiff = _explained_by_ties(got, want, score, threshold, row_sparse, name)
    assert ndiff <= 0.01 * want.sum(), (name, ndiff)
    # The reference's own acceptance figures against its golden (which may drop the guard block of a row).
    z = np.load(G / "estimate.npz")
    shape = tuple(z[f"{name}_shape"])
    golden = np.unpackbits(z[f"{name}_bits"])[:int(np.prod(shape))].reshape(shape).astype(bool)
    assert (golden & ~got).sum() <= 0.01 * golden.sum(), name            # omitted blocks
    assert ((got != golden).sum(-1) <= 1 + (got != want).sum(-1)).all(), name  # at most the guard block per row


@pytest.mark.parametrize("case", inputs.ESTIMATE_CASES, ids=[c[0] for c in inputs.ESTIMATE_CASES])
def test_estimate_causal_against_oracle_and_reference_vectors(case):
    """causal=True: the golden's causal branch (tests/plugin/test_sparseblockestimate.py:73-76, 127-143),
    restated in oracle.ada_bsa and pinned to the golden's own output (tests/golden/ada_causal.npz).  Same
    bar as the other branch: every differing row explained by rounding at its guard, at most 1 % of the
    kept blocks, and the reference's acceptance figures against the golden."""
    import mindiesd  # noqa: F401
    from mindiesd import _cabi
    name, grid, heads, threshold, row_sparse, seed = case
    q, k = inputs.structured_qk(seed, heads, grid, 128)
    want, count, score = oada.sparse_block_estimate(q.float().numpy(), k.float().numpy(), SCALE, threshold, row_sparse,
                                                    causal=True)
    blocks = want.shape[-1]
    mask, cnt = torch.ops.mindiesd.sparse_block_estimate(
        query=q.cuda(), key=k.cuda(), input_layout="BNSD", stride=8, sparse_size=128, num_heads=heads,
        num_key_value_heads=heads, scale_value=SCALE, threshold=threshold, causal=True, keep_sink=True,
        keep_recent=True, row_sparse=row_sparse)
    assert _cabi.device_status() == 0
    got = mask.cpu().numpy()[..., :blocks].astype(bool)
    assert np.array_equal(cnt.cpu().numpy(), got.sum(-1))
    assert not np.triu(got, 1).any() and got[..., 0].all()
    assert np.array_equal(got[..., :2, :], want[..., :2, :])  # rows 0 and 1: everything up to their own block
    ndiff = 0
    for (b, n, i) in np.argwhere((got != want).any(-1)):
        # the row ranks the blocks its chunk saw, up to its own, with the last of them cleared: that is the
        # other branch's rule on the truncated row with keep_recent's clearing but without its forcing
        seen = int(np.flatnonzero(score[b, n, i] > 0).max()) + 1 if (score[b, n, i] > 0).any() else i + 1
        m = min(i + 1, seen)
        g = got[b, n, i, :m].copy()
        last = g[-1]
        g[-1] = True  # _row_explained forces the last block; compare the rest, then the last one by hand
        assert _row_explained(g, score[b, n, i, :m], threshold, row_sparse), (name, b, n, i)
        ndiff += int((got[b, n, i] != want[b, n, i]).sum())
    assert ndiff <= max(1, 0.01 * want.sum()), (name, ndiff)
    z = np.load(G / "ada_causal.npz")
    shape = tuple(z[f"{name}_shape"])
    golden = np.unpackbits(z[f"{name}_bits"])[:int(np.prod(shape))].reshape(shape).astype(bool)
    assert (golden & ~got).sum() <= 0.01 * golden.sum(), name
    assert ((got != golden).sum(-1) <= 1 + (got != want).sum(-1)).all(), name


def test_ada_attention_causal_matches_reference_vectors():
    """ada_block_sparse_attention(causal=True) on a lower-triangular block mask against the reference's
    numpy golden run with causal=True, at the reference's own bar (ref_compare, 2^-6)."""
    import mindiesd  # noqa: F401
    z = np.load(G / "ada_causal.npz")
    q, k, v = (inputs.randn(41 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    mask = torch.from_numpy(z["attention_mask"]).cuda()
    out = torch.ops.mindiesd.ada_block_sparse_attention(
        query=q.cuda(), key=k.cuda(), value=v.cuda(), sparse_mask=mask, sparse_count_table=mask.sum(-1, dtype=torch.int32),
        input_layout="BNSD", sparse_size=128, num_heads=2, num_key_value_heads=2, scale_value=128 ** -0.5, causal=True)
    eb, ok, worst = oa.ref_compare(torch.from_numpy(z["attention_out"]), out.cpu().float(), 2 ** -6)
    assert ok, (eb, worst)


def test_estimate_bsnd_fp16_and_flags():
    import mindiesd  # noqa: F401
    q, k = inputs.structured_qk(61, 2, (2, 32, 32), 128, dtype=torch.float16)
    want, _, score = oada.sparse_block_estimate(q.float().numpy(), k.float().numpy(), SCALE, 0.8, 1.0,
                                                keep_sink=False, keep_recent=False)
    qb, kb = q.transpose(1, 2).contiguous().cuda(), k.transpose(1, 2).contiguous().cuda()
    mask, cnt = torch.ops.mindiesd.sparse_block_estimate(
        query=qb, key=kb, input_layout="BSND", stride=8, sparse_size=128, num_heads=2, num_key_value_heads=2,
        scale_value=SCALE, threshold=0.8, causal=False, keep_sink=False, keep_recent=False, row_sparse=1.0)
    got = mask.cpu().numpy()[..., :want.shape[-1]].astype(bool)
    ndiff = _explained_by_ties(got, want, score, 0.8, 1.0, "flags", keep_sink=False, keep_recent=False)
    assert ndiff <= 0.01 * want.sum()
    with pytest.raises(RuntimeError):
        torch.ops.mindiesd.sparse_block_estimate(query=qb, key=kb, input_layout="TND", causal=False)


def test_estimate_long_sequence_one_head_per_pass():
    """32 760 tokens (the 480p grid), 3 heads, scratch for a single head: passes reuse the scratch."""
    from mindiesd import _cabi
    q, k = inputs.structured_qk(62, 3, (21, 30, 52), 128)
    want, _, score = oada.sparse_block_estimate(q.float().numpy(), k.float().numpy(), SCALE, 0.6, 0.5)
    one = _cabi.lib().mindiesd_sparse_block_estimate_scratch_bytes(1, 1, q.shape[2])
    scratch = torch.empty(one, dtype=torch.uint8, device="cuda")
    mask, cnt = _cabi.sparse_block_estimate(q.cuda(), k.cuda(), SCALE, 0.6, 0.5, scratch=scratch)
    full, cnt2 = _cabi.sparse_block_estimate(q.cuda(), k.cuda(), SCALE, 0.6, 0.5)
    assert torch.equal(mask, full) and torch.equal(cnt, cnt2)
    got = mask.cpu().numpy()[..., :want.shape[-1]].astype(bool)
    ndiff = _explained_by_ties(got, want, score, 0.6, 0.5, "long")
    assert ndiff <= 0.01 * want.sum()
    assert (cnt.cpu().numpy() <= int(0.5 * want.shape[-1]) + 2).all()  # row cap (+ first and last block)
    assert _cabi.device_status() == 0


def test_ada_attention_matches_reference_vectors():
    import mindiesd  # noqa: F401
    z = np.load(G / "ada_attention.npz")
    q, k, v = (inputs.randn(41 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    mask = torch.from_numpy(z["mask"]).cuda()
    sct = mask.sum(-1, dtype=torch.int32)
    want = torch.from_numpy(z["out"])
    out = torch.ops.mindiesd.ada_block_sparse_attention(
        query=q.cuda(), key=k.cuda(), value=v.cuda(), sparse_mask=mask, sparse_count_table=sct, input_layout="BNSD",
        sparse_size=128, num_heads=2, num_key_value_heads=2, scale_value=128 ** -0.5, causal=False)
    assert out.dtype == torch.bfloat16 and out.shape == q.shape
    eb, ok, worst = oa.ref_compare(want, out.cpu().float(), 2 ** -6)  # the reference's bar for this operator
    assert ok, (eb, worst)
    assert torch.count_nonzero(out[0, 1, 256:]) == 0  # the row that keeps nothing
    qb, kb, vb = (x.transpose(1, 2).contiguous().cuda() for x in (q, k, v))
    out_b = torch.ops.mindiesd.ada_block_sparse_attention(
        query=qb, key=kb, value=vb, sparse_mask=mask, sparse_count_table=sct, input_layout="BSND", sparse_size=128,
        num_heads=2, num_key_value_heads=2, scale_value=128 ** -0.5, causal=False)
    assert torch.equal(out_b.transpose(1, 2), out)
    # causal=True (the schema's default): the token-level triangle inside the kept blocks, which is what the
    # golden's in-block triangle (tests/plugin/test_adablocksparseattention.py:69-72) amounts to for a
    # lower-triangular mask that keeps the diagonal blocks
    tri = torch.tril(torch.ones(1, 2, 3, 3, dtype=torch.int8)).cuda()
    out_c = torch.ops.mindiesd.ada_block_sparse_attention(
        query=q.cuda(), key=k.cuda(), value=v.cuda(), sparse_mask=tri, sparse_count_table=tri.sum(-1, dtype=torch.int32),
        input_layout="BNSD", sparse_size=128, num_heads=2, num_key_value_heads=2, scale_value=128 ** -0.5, causal=True)
    keep = torch.tril(torch.ones(300, 300, dtype=torch.bool))
    want_c = oa.attention_math(q, k, v, attn_mask=keep, head_first=True)
    assert (out_c.cpu().float() - want_c.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("layout", ["BNSD", "BSND"])
def test_sparse_attention_ada_bsa_end_to_end(layout):
    """sparse_attention(sparse_type="ada_bsa") against the oracle's attention over the mask the GPU chose
    (the mask itself is checked above)."""
    from mindiesd import sparse_attention
    from mindiesd.layers.flash_attn.sparse_flash_attn_ada_bsa import get_estimate_mask
    q, k = inputs.structured_qk(63, 2, (2, 24, 40), 128)  # 1920 tokens
    v = inputs.randn(64, 1, 2, q.shape[2], 128, dtype=torch.bfloat16)
    args = (q, k, v) if layout == "BNSD" else tuple(x.transpose(1, 2).contiguous() for x in (q, k, v))
    dev = tuple(x.cuda() for x in args)
    out = sparse_attention(*dev, head_num=2, input_layout=layout, sparse_type="ada_bsa", cdf_threshold=0.7,
                           sparsity=0.25)
    smask, sct = get_estimate_mask(*dev, scale=128 ** -0.5, head_num=2, input_layout=layout, sparsity=0.25,
                                   cdf_threshold=0.7)
    blocks = 15
    assert smask.shape == (1, 2, blocks, 32) and int(sct.max()) <= int(0.75 * blocks) + 2
    assert 0.2 < smask[..., :blocks].float().mean().item() < 0.95
    want = oa.block_sparse_attention(q, k, v, smask.cpu().numpy(), 128)
    got = out.cpu().float() if layout == "BNSD" else out.cpu().float().transpose(1, 2)
    assert (got - want).abs().max().item() < 2e-2 and (got - want).abs().mean().item() < 2e-3


def test_full_threshold_is_dense_attention():
    """The reference's own acceptance of the layer (tests/layers/flash_attn/test_sparse_attention.py:123-142):
    cdf_threshold = 1.0 and sparsity = 0.0 keep every block, so the result is dense attention."""
    from mindiesd import attention_forward, sparse_attention
    q, k, v = (inputs.randn(70 + i, 1, 9600, 3, 128, dtype=torch.float16).cuda() for i in range(3))
    out = sparse_attention(q, k, v, scale=128 ** -0.5, head_num=3, input_layout="BSND", inner_precise=0,
                           sparse_type="ada_bsa", cdf_threshold=1.0, sparsity=0.0)
    dense = attention_forward(q, k, v, head_first=False)
    assert torch.equal(out, dense)
    smask, sct = torch.ops.mindiesd.sparse_block_estimate(
        query=q, key=k, input_layout="BSND", num_heads=3, num_key_value_heads=3, scale_value=128 ** -0.5 / 8,
        threshold=1.0, causal=False, row_sparse=1.0)
    assert bool((smask[..., :75] == 1).all()) and bool((sct == 75).all())
