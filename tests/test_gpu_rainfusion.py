"""GPU parity of the RainFusion kernels through the C ABI: permutation, pooled means, block mask
(bit-exact against the vectors of the reference and against the oracle) and block-sparse attention."""
from pathlib import Path

import numpy as np
import pytest
import torch

import inputs
from oracle import attention as oa
from oracle import rainfusion as orf

pytestmark = pytest.mark.gpu
G = Path(__file__).resolve().parent / "golden"


def _unpack(z, name):
    shape = tuple(z[f"{name}_mask_shape"])
    return np.unpackbits(z[f"{name}_mask_bits"])[:int(np.prod(shape))].reshape(shape).astype(np.int8)


@pytest.mark.parametrize("grid", inputs.PERM_GRIDS + [(21, 30, 52)])
@pytest.mark.parametrize("head_first", [True, False])
def test_permutation_bit_exact(grid, head_first):
    from mindiesd import _cabi
    t, h, w = grid
    for txt in (0, 77):
        s = t * h * w + txt
        x = inputs.randn(5, 1, 2, s, 16, dtype=torch.bfloat16)
        layout = "BNSD" if head_first else "BSND"
        if not head_first:
            x = x.transpose(1, 2).contiguous()
        y = _cabi.rf_rearrange(x.cuda(), grid, txt, head_first)
        assert torch.equal(y.cpu(), orf.rearrange(x, grid, txt, layout))
        back = _cabi.rf_rearrange(y, grid, txt, head_first, inverse=True)
        assert torch.equal(back.cpu(), x)
    # 4-byte elements
    x = inputs.randn(6, 1, 1, t * h * w, 8)
    y = _cabi.rf_rearrange(x.cuda(), grid, 0, True)
    assert torch.equal(y.cpu(), orf.rearrange(x, grid, 0, "BNSD"))
    assert _cabi.device_status() == 0


def test_ragged_small_grid_is_rejected():
    from mindiesd import _cabi
    x = torch.zeros(1, 1, 3 * 5 * 7, 16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.rf_rearrange(x, (3, 5, 7), 0, True)  # the reference's permutation is undefined there


def test_pooled_means():
    from mindiesd import _cabi
    z = np.load(G / "avgpool.npz")
    x = inputs.randn(3, 1, 2, 300, 16)
    got = _cabi.rf_pool(x.cuda(), None, 0, True).cpu()
    assert (got - torch.from_numpy(z["bnsd"])).abs().max().item() < 1e-6  # the reference accumulates in fp32
    grid, txt = (3, 30, 52), 200
    q, _ = inputs.structured_qk(16, 2, grid, 128, txt)
    want, _ = orf.pooled_means(q.double(), q.double(), grid, txt, 128, "BNSD")
    got = _cabi.rf_pool(q.cuda(), grid, txt, True).cpu()
    assert got.shape == want.shape
    assert torch.equal(got, want.float())  # exact sum, one rounding


@pytest.mark.parametrize("case", inputs.MASK_CASES, ids=[c[0] for c in inputs.MASK_CASES])
def test_block_mask_bit_exact(case):
    """0 differing bits against the mask the reference produced from the fp32 upcast of the same
    bf16 data; the compacted lists equal the reference's too."""
    from mindiesd import _cabi
    name, grid, txt, heads, dim, sparsity, layout, seed = case
    z = np.load(G / "mask.npz")
    want = _unpack(z, name)
    q, k = inputs.structured_qk(seed, heads, grid, dim, txt)
    head_first = layout == "BNSD"
    if not head_first:
        q, k = q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous()
    mask, sel, num = _cabi.rf_block_mask(q.cuda(), k.cuda(), grid, txt, sparsity, head_first, want_lists=True)
    diff = int((mask.cpu().numpy() != want).sum())
    assert diff == 0, f"{diff} of {want.size} mask bits differ (min margin {z.get(name + '_min_margin')})"
    sel_o, num_o = orf.select_lists(torch.from_numpy(want))
    assert torch.equal(sel.cpu(), sel_o) and torch.equal(num.cpu(), num_o)
    if f"{name}_select_idx" in z.files:
        assert np.array_equal(sel.cpu().numpy(), z[f"{name}_select_idx"].astype(np.int64))
    # fp32 inputs take the same path
    mask32 = _cabi.rf_block_mask(q.float().cuda(), k.float().cuda(), grid, txt, sparsity, head_first)
    assert torch.equal(mask32, mask)
    assert _cabi.device_status() == 0


def test_temporal_band_and_first_frame_switch():
    from mindiesd import _cabi
    grid = (4, 16, 24)
    q, k = inputs.structured_qk(33, 2, grid, 128)
    base = _cabi.rf_block_mask(q.cuda(), k.cuda(), grid, 0, 0.75, True, protect_first_frame=False).cpu()
    prot = _cabi.rf_block_mask(q.cuda(), k.cuda(), grid, 0, 0.75, True, protect_first_frame=True).cpu()
    fb = (16 * 24 + 127) // 128
    assert prot[:, :, :fb].all() and prot[:, :, :, :fb].all()
    assert torch.equal(prot[:, :, fb:, fb:], base[:, :, fb:, fb:])
    band = _cabi.rf_block_mask(q.cuda(), k.cuda(), grid, 0, 0.75, True, protect_first_frame=True, temporal_band=1).cpu()
    want = prot.bool() | torch.from_numpy(orf.temporal_band(grid, 0, 1))[None, None]
    assert torch.equal(band.bool(), want)


def test_block_sparse_attention_matches_reference_vectors():
    from mindiesd import _cabi
    z = np.load(G / "block_sparse.npz")
    q, k, v = (inputs.randn(31 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    mask = torch.from_numpy(z["mask"]).cuda()
    out, lse = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), block_mask=mask, out_dtype=torch.float32, want_lse=True)
    want = torch.from_numpy(z["out"])
    eb, ok, mx = oa.ref_compare(want, out.cpu(), 2 ** -6)  # the tolerance of the reference's own test
    assert ok, (eb, mx)
    assert torch.count_nonzero(out[0, 0, 128:256]) == 0 and torch.isinf(lse[0, 0, 128:256]).all()


@pytest.mark.parametrize("head_first", [True, False])
def test_block_sparse_mask_and_list_agree_with_oracle(head_first):
    from mindiesd import _cabi
    b, n, s = 2, 3, 1500
    shape = (b, n, s, 128) if head_first else (b, s, n, 128)
    q, k, v = (inputs.randn(70 + i, *shape, dtype=torch.bfloat16) for i in range(3))
    nb = (s + 127) // 128
    m = (np.random.RandomState(9).rand(1, n, nb, nb) < 0.35)
    m[:, :, np.arange(nb), np.arange(nb)] = True
    mask = torch.from_numpy(np.repeat(m, b, 0).astype(np.int8))
    to_bnsd = (lambda x: x) if head_first else (lambda x: x.transpose(1, 2))
    want = oa.block_sparse_attention(to_bnsd(q), to_bnsd(k), to_bnsd(v), mask.numpy())
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), head_first=head_first, block_mask=mask.cuda())
    diff = (to_bnsd(out).float().cpu() - want).abs()
    assert diff.max().item() <= 2e-2 and diff.mean().item() <= 2e-3
    sel, num = orf.select_lists(mask)
    out2 = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), head_first=head_first, select_idx=sel.cuda(),
                           select_num=num.cuda())
    assert torch.equal(out2, out)  # the list walk visits the same blocks in the same order
    assert _cabi.device_status() == 0


@pytest.mark.parametrize("grid,txt,head_first", [
    ((3, 40, 80), 0, True),      # aligned: every frame in 8x8 windows
    ((2, 21, 32), 0, True),      # five remainder rows per frame; the first frame stays in raster order
    ((3, 40, 80), 256, False),   # text tokens move from the front to the back; BSND
    ((3, 13, 24), 0, True),      # 5 remainder rows, 312 tokens per frame: blocks straddle frames and windows
])
def test_permutation_inside_the_attention_kernel(grid, txt, head_first):
    """The window permutation applied by the attention kernel's own loads and stores against the
    materialised pipeline (permute q, k, v; attention; inverse permute): the kernel sees the same rows in
    the same tile order either way, so the outputs are bit-equal."""
    from mindiesd import _cabi
    n, s = 2, txt + grid[0] * grid[1] * grid[2]
    shape = (1, n, s, 128) if head_first else (1, s, n, 128)
    q, k, v = (inputs.randn(85 + i, *shape, dtype=torch.bfloat16).cuda() for i in range(3))
    nb = (grid[0] * grid[1] * grid[2] + 127) // 128 + (txt + 127) // 128
    assert nb == (s + 127) // 128  # image and text blocks coincide with blocks of the whole sequence here
    m = np.random.RandomState(11).rand(1, n, nb, nb) < 0.4
    m[:, :, np.arange(nb), np.arange(nb)] = True
    mask = torch.from_numpy(m.astype(np.int8)).cuda()
    qp, kp, vp = (_cabi.rf_rearrange(x, grid, txt, head_first) for x in (q, k, v))
    want = _cabi.rf_rearrange(_cabi.attention(qp, kp, vp, head_first=head_first, block_mask=mask), grid, txt, head_first,
                              inverse=True)
    got = _cabi.attention(q, k, v, head_first=head_first, block_mask=mask, perm_grid=grid, perm_txt=txt)
    assert torch.equal(got, want)
    # inputs permuted beforehand, only the output put back by the kernel (what the layer API does)
    got1 = _cabi.attention(qp, kp, vp, head_first=head_first, block_mask=mask, perm_grid=grid, perm_txt=txt,
                           perm_inputs_permuted=True)
    assert torch.equal(got1, want)
    sel, num = orf.select_lists(mask.cpu())
    got2 = _cabi.attention(q, k, v, head_first=head_first, select_idx=sel.cuda(), select_num=num.cuda(), perm_grid=grid,
                           perm_txt=txt)
    assert torch.equal(got2, want)
    assert _cabi.device_status() == 0


def test_permutation_inside_the_kernel_needs_eight_token_runs():
    from mindiesd import _cabi
    grid = (3, 30, 52)  # four remainder columns: runs of four tokens
    s = grid[0] * grid[1] * grid[2]
    q = torch.zeros(1, 1, s, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q, q, q, perm_grid=grid)
    # ... but putting only the output back works on any grid
    x = inputs.randn(89, 1, 1, s, 128, dtype=torch.bfloat16).cuda()
    xp = _cabi.rf_rearrange(x, grid, 0, True)
    want = _cabi.rf_rearrange(_cabi.attention(xp, xp, xp), grid, 0, True, inverse=True)
    assert torch.equal(_cabi.attention(xp, xp, xp, perm_grid=grid, perm_inputs_permuted=True), want)
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q, q, q, perm_grid=(3, 40, 80))  # does not match the sequence length


def test_full_mask_equals_dense():
    from mindiesd import _cabi
    q, k, v = (inputs.randn(80 + i, 1, 2, 900, 128, dtype=torch.bfloat16).cuda() for i in range(3))
    mask = torch.ones(1, 2, 8, 8, dtype=torch.int8, device="cuda")
    assert torch.equal(_cabi.attention(q, k, v, block_mask=mask), _cabi.attention(q, k, v))


def _pairs_are_a_matching(pairs, q_blocks):
    flat = pairs.reshape(-1).tolist()
    used = sorted(x for x in flat if x >= 0)
    assert used == list(range(q_blocks)), "every query block exactly once"
    assert flat.count(-1) == q_blocks % 2 and all(p[0] >= 0 for p in pairs.tolist())


@pytest.mark.parametrize("q_blocks", [9, 16])
def test_paired_query_blocks_give_the_same_bits(q_blocks):
    """Query blocks paired by the overlap of their key lists (mindiesd_rf_pair_blocks) instead of by index: the
    table is a perfect matching, and the attention output does not change by a bit -- for a block mask and for
    the lists made from it, with a ragged tail, bf16 and fp16."""
    from mindiesd import _cabi
    s_q = q_blocks * 128 - 37
    kv_blocks = 11
    s_kv = kv_blocks * 128 - 5
    gen = torch.Generator().manual_seed(7)
    mask = (torch.rand(1, 3, q_blocks, kv_blocks, generator=gen) < 0.4).to(torch.int8)
    mask[..., 0] = 1  # no empty row
    mask[:, :, 1] = mask[:, :, q_blocks - 2]  # far-apart rows with identical lists: the pairing should find them
    mask = mask.cuda()
    pairs = _cabi.rf_pair_blocks(mask)
    assert pairs.shape == (1, 3, (q_blocks + 1) // 2, 2)
    for h in range(3):
        _pairs_are_a_matching(pairs[0, h].cpu(), q_blocks)
    hit = [sorted(p) == [1, q_blocks - 2] for h in range(3) for p in pairs[0, h].cpu().tolist()]
    assert sum(hit) >= 2  # (a row may have been taken by an even closer partner in one head)
    for dtype in (torch.bfloat16, torch.float16):
        q = inputs.randn(90, 1, 3, s_q, 128, dtype=dtype).cuda()
        k, v = (inputs.randn(91 + i, 1, 3, s_kv, 128, dtype=dtype).cuda() for i in range(2))
        plain, lse0 = _cabi.attention(q, k, v, block_mask=mask, want_lse=True)
        paired, lse1 = _cabi.attention(q, k, v, block_mask=mask, q_pairs=pairs, want_lse=True)
        assert torch.equal(plain, paired) and torch.equal(lse0, lse1)
        idx, num = orf.select_lists(mask.cpu())  # the same blocks as compacted lists
        listed = _cabi.attention(q, k, v, select_idx=idx.cuda(), select_num=num.cuda(), q_pairs=pairs)
        assert torch.equal(plain, listed)
    assert _cabi.device_status() == 0


def test_pairing_is_refused_where_it_does_not_apply():
    from mindiesd import _cabi
    q, k, v = (inputs.randn(95 + i, 1, 1, 512, 128, dtype=torch.bfloat16).cuda() for i in range(3))
    mask = torch.ones(1, 1, 4, 4, dtype=torch.int8, device="cuda")
    pairs = _cabi.rf_pair_blocks(mask)
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q, k, v, q_pairs=pairs)  # dense: nothing to pair
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q, k, v, block_mask=mask, q_pairs=pairs, causal=True)
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q, k, v, block_mask=mask, q_pairs=pairs[:, :, :1].contiguous())  # wrong count


def test_wan_720p_pairing_cuts_the_steps_that_serve_one_tile():
    """The 21x45x80 RainFusion mask (2 heads): neighbouring query blocks share about four fifths of their key
    lists; paired by overlap, the steps a thread block takes (the union of its two lists) drop by a few
    per cent, and the layer operator, which pairs by itself, returns what the unpaired launch returns."""
    import workloads
    from mindiesd import _cabi
    grid = workloads.C3.grid
    q, k, v = workloads.make_qkv(workloads.C3, "cuda", seed=4, heads=2)
    mask = _cabi.rf_block_mask(q, k, grid, 0, 0.75, True)
    pairs = _cabi.rf_pair_blocks(mask)
    m = mask[0].bool().cpu()
    for h in range(2):
        pr = pairs[0, h].cpu()
        _pairs_are_a_matching(pr, 591)
        steps_paired = sum(int((m[h, a] | (m[h, b] if b >= 0 else m[h, a])).sum()) for a, b in pr.tolist())
        steps_index = sum(int((m[h, 2 * i] | m[h, min(2 * i + 1, 590)]).sum()) for i in range(296))
        assert steps_paired < 0.98 * steps_index, (steps_paired, steps_index)
    qp, kp, vp = (_cabi.rf_rearrange(x, grid, 0, True) for x in (q, k, v))
    plain = _cabi.attention(qp, kp, vp, block_mask=mask)
    paired = _cabi.attention(qp, kp, vp, block_mask=mask, q_pairs=pairs)
    assert torch.equal(plain, paired)
    import mindiesd  # noqa: F401  (registers torch.ops.mindiesd)
    via_op = torch.ops.mindiesd.rf_sparse_attention(qp, kp, vp, mask, None, None, list(grid), 0, 128 ** -0.5, "BNSD", True)
    assert torch.equal(via_op, _cabi.rf_rearrange(plain, grid, 0, True, inverse=True))
    assert _cabi.device_status() == 0


@pytest.mark.parametrize("layout", ["BNSD", "BSND"])
def test_a_reused_mask_brings_its_pairing_table(layout):
    """bsa_sparse_attention_v3 with `cached_mask`: the second step pairs the query blocks by overlap (the table is
    built once for the mask that came back) and returns what the first step returned, bit for bit."""
    from mindiesd.layers.flash_attn import sparse_flash_attn_rf_v3 as v3
    grid, heads = (3, 32, 64), 2   # 6144 tokens: 48 query blocks
    shape = (1, heads, 6144, 128) if layout == "BNSD" else (1, 6144, heads, 128)
    q, k, v = (inputs.randn(120 + i, *shape, dtype=torch.bfloat16).cuda() for i in range(3))
    v3._PAIR_TABLES.clear()
    out1, mask = v3.bsa_sparse_attention_v3(q, k, v, grid, sparsity=0.6, input_layout=layout)
    assert not v3._PAIR_TABLES  # a fresh mask is used as it is
    out2, mask2 = v3.bsa_sparse_attention_v3(q, k, v, grid, sparsity=0.6, input_layout=layout, cached_mask=mask)
    assert mask2 is mask and len(v3._PAIR_TABLES) == 1
    table = next(iter(v3._PAIR_TABLES.values()))
    assert table.shape == (1, heads, 24, 2)
    for h in range(heads):
        _pairs_are_a_matching(table[0, h].cpu(), 48)
    assert torch.equal(out1, out2)
    out3, _ = v3.bsa_sparse_attention_v3(q, k, v, grid, sparsity=0.6, input_layout=layout, cached_mask=mask)
    assert len(v3._PAIR_TABLES) == 1 and torch.equal(out1, out3)  # the table is reused
    from mindiesd import _cabi
    assert _cabi.device_status() == 0


def test_wan_720p_mask_density():
    """Config C3 grid (21x45x80, 591 blocks), sparsity 0.75, on 2 heads generated on the device:
    every row keeps at least ceil(591/4) = 148 blocks plus the 29 first-frame columns, and the
    device mask equals the oracle run on the same data copied to the host."""
    import workloads
    from mindiesd import _cabi
    q, k, _ = workloads.make_qkv(workloads.C3, "cuda", seed=4, heads=2)
    mask = _cabi.rf_block_mask(q, k, workloads.C3.grid, 0, 0.75, True).cpu()
    assert mask.shape == (1, 2, 591, 591)
    kept = mask[:, :, 29:].sum(-1)
    assert kept.min().item() >= 148 and 0.30 < mask.float().mean().item() < 0.36
    qp, kp = orf.pooled_means(q.cpu().float(), k.cpu().float(), workloads.C3.grid, 0, 128, "BNSD")
    want = orf.blockwise_mask(qp, kp, 0, 0.75, 128 ** -0.5, 128, workloads.C3.grid, "BNSD")
    assert int((mask != want).sum()) == 0
