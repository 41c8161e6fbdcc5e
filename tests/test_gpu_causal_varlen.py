"""GPU parity of the causal mode and of the packed variable-length launch of the attention kernel,
called through the C ABI and through `attention_forward_varlen`, against the CPU oracle
(`oracle.attention.attention_math` with a triangular keep-mask).  The causal triangle is aligned to
the last query and the last key of a sequence, as sparse_mode 3 of the reference's fused call is
(mindiesd/layers/flash_attn/attention_forward_varlen.py:133-149 of MindIE-SD); the two packed cases
are the reference's own (tests/layers/flash_attn/test_attention_forward_varlen.py:183-196), each at
both values of `causal` as there (:176-178).  Tolerance of the bf16 path: max-abs 2e-2, mean-abs 2e-3."""
import pytest
import torch

import inputs
from oracle import attention as oa

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _check(out, want):
    diff = (out.float().cpu() - want.float()).abs()
    assert not torch.isnan(out.float()).any()
    assert diff.max().item() <= MAX_ABS, diff.max().item()
    assert diff.mean().item() <= MEAN_ABS, diff.mean().item()


def _causal_keep(sq, skv):
    """keep[i, j] = j <= i + (skv - sq)."""
    i = torch.arange(sq)[:, None]
    j = torch.arange(skv)[None, :]
    return j <= i + (skv - sq)


def _oracle(q, k, v, causal, head_first):
    """attention_math; rows that see no key (their softmax is 0/0 in the formula) are zeros."""
    sq = q.shape[2] if head_first else q.shape[1]
    skv = k.shape[2] if head_first else k.shape[1]
    mask = _causal_keep(sq, skv) if causal else None
    out = oa.attention_math(q, k, v, attn_mask=mask, head_first=head_first)
    return torch.nan_to_num(out.float(), nan=0.0)


@pytest.mark.parametrize("b,n,sq,skv,head_first", [
    (1, 2, 300, 300, True),      # ragged tail and diagonal in the same block
    (1, 1, 128, 128, True),
    (2, 2, 129, 400, True),      # more keys than queries: every row sees at least 272 keys
    (1, 2, 400, 129, False),     # more queries than keys: the first 271 rows see nothing and give zeros
    (1, 3, 1000, 1000, False),
    (1, 1, 2049, 2049, True),    # odd tile count: the last pair has one tile
    (1, 2, 640, 700, True),      # offset 60: the diagonal crosses two key blocks per tile
])
def test_causal_dense(b, n, sq, skv, head_first):
    from mindiesd import _cabi
    shape_q = (b, n, sq, 128) if head_first else (b, sq, n, 128)
    shape_k = (b, n, skv, 128) if head_first else (b, skv, n, 128)
    q, k, v = (inputs.randn(700 + i, *s, dtype=torch.bfloat16) for i, s in enumerate((shape_q, shape_k, shape_k)))
    out, lse = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), head_first=head_first, causal=True, want_lse=True)
    _check(out, _oracle(q, k, v, True, head_first))
    # log-sum-exp of the visible scores; -inf where a row sees nothing
    qf, kf = (x.float() if head_first else x.float().transpose(1, 2) for x in (q, k))
    s = qf @ kf.transpose(-1, -2) * 128 ** -0.5
    s = s.masked_fill(~_causal_keep(sq, skv), float("-inf"))
    want_lse = torch.logsumexp(s, -1)
    got = lse.cpu()
    fin = torch.isfinite(want_lse)
    assert torch.equal(torch.isfinite(got), fin)
    assert (got[fin] - want_lse[fin]).abs().max().item() < 2e-2
    assert _cabi.device_status() == 0


def test_causal_fp16_and_fp32_out():
    from mindiesd import _cabi
    q, k, v = (inputs.randn(720 + i, 1, 2, 513, 128, dtype=torch.float16) for i in range(3))
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), causal=True, out_dtype=torch.float32)
    _check(out, _oracle(q, k, v, True, True))


def test_causal_with_block_mask():
    """A block mask and the triangle together: a block is walked if both allow it, and the triangle cuts
    the blocks it crosses (the in-block triangle of ada_block_sparse_attention_cpu,
    tests/plugin/test_adablocksparseattention.py:69-72 of MindIE-SD, for masks that keep the diagonal)."""
    from mindiesd import _cabi
    s = 900
    nb = (s + 127) // 128
    q, k, v = (inputs.randn(730 + i, 1, 2, s, 128, dtype=torch.bfloat16) for i in range(3))
    g = torch.Generator().manual_seed(5)
    mask = (torch.rand(1, 2, nb, nb, generator=g) < 0.5).to(torch.int8)
    mask = torch.tril(mask)
    mask[..., torch.arange(nb), torch.arange(nb)] = 1  # the diagonal block is kept
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), block_mask=mask.cuda(), causal=True)
    keep = mask.bool().repeat_interleave(128, 2).repeat_interleave(128, 3)[:, :, :s, :s] & _causal_keep(s, s)
    for n in range(2):  # the oracle takes one [q, kv] mask: a head at a time
        want = oa.attention_math(q[:, n:n + 1], k[:, n:n + 1], v[:, n:n + 1], attn_mask=keep[0, n], head_first=True)
        _check(out[:, n:n + 1], want)
    assert _cabi.device_status() == 0


def _varlen_oracle(q, k, v, cu_q, cu_k, causal):
    out = torch.zeros(q.shape, dtype=torch.float32)
    for i in range(len(cu_q) - 1):
        qs, ks = slice(cu_q[i], cu_q[i + 1]), slice(cu_k[i], cu_k[i + 1])
        if cu_q[i + 1] == cu_q[i] or cu_k[i + 1] == cu_k[i]:
            continue
        out[qs] = _oracle(q[qs][None], k[ks][None], v[ks][None], causal, False)[0]
    return out


VARLEN_CASES = {
    # the reference's two cases
    "small_batch": ([0, 76, 124], [0, 1640, 48608]),
    "large_batch": ([0, 3348, 6696, 10044, 12648, 15996, 19344, 22692, 25296, 28644, 31992, 35340, 37944, 40734, 43524,
                     46314, 48484],) * 2,
    # ragged: a one-token sequence, an empty one, a sequence without keys, lengths around the tile sizes
    "ragged": ([0, 300, 301, 301, 557, 1072, 1200], [0, 300, 377, 400, 400, 1040, 1296]),
}


@pytest.mark.parametrize("case", sorted(VARLEN_CASES))
@pytest.mark.parametrize("causal", [False, True])
def test_attention_forward_varlen_single_launch(case, causal):
    from mindiesd import _cabi, attention_forward_varlen
    cu_q, cu_k = VARLEN_CASES[case]
    heads = 3
    q = inputs.randn(740, cu_q[-1], heads, 128, dtype=torch.bfloat16)
    k, v = (inputs.randn(741 + i, cu_k[-1], heads, 128, dtype=torch.bfloat16) for i in range(2))
    out = attention_forward_varlen(q.cuda(), k.cuda(), v.cuda(), cu_q, cu_k, causal=causal)
    assert out.shape == q.shape and out.dtype == q.dtype
    _check(out, _varlen_oracle(q, k, v, cu_q, cu_k, causal))
    # cumulative lengths that already live on the device are used as they are (no host read)
    dq, dk = (torch.tensor(c, dtype=torch.int32, device="cuda") for c in (cu_q, cu_k))
    again = attention_forward_varlen(q.cuda(), k.cuda(), v.cuda(), dq, dk, causal=causal)
    assert torch.equal(again, out)
    assert _cabi.device_status() == 0


def test_varlen_through_the_c_abi_with_lse_and_gqa():
    from mindiesd import _cabi
    cu_q, cu_k = [0, 200, 777], [0, 130, 900]
    q = inputs.randn(750, 1, cu_q[-1], 4, 128, dtype=torch.bfloat16)
    k, v = (inputs.randn(751 + i, 1, cu_k[-1], 2, 128, dtype=torch.bfloat16) for i in range(2))
    dq, dk = (torch.tensor(c, dtype=torch.int32, device="cuda") for c in (cu_q, cu_k))
    out, lse = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), head_first=False, cu_seqlens_q=dq, cu_seqlens_kv=dk,
                               want_lse=True)
    kk, vv = (x.repeat_interleave(2, dim=2) for x in (k, v))
    _check(out[0], _varlen_oracle(q[0], kk[0], vv[0], cu_q, cu_k, False))
    for i in range(2):
        s = torch.einsum("qnd,knd->nqk", q[0, cu_q[i]:cu_q[i + 1]].float(), kk[0, cu_k[i]:cu_k[i + 1]].float()) * 128 ** -0.5
        assert (lse[0, :, cu_q[i]:cu_q[i + 1]].cpu() - torch.logsumexp(s, -1)).abs().max().item() < 2e-2
    # not combined with block sparsity
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.attention(q.cuda(), k.cuda(), v.cuda(), head_first=False, cu_seqlens_q=dq, cu_seqlens_kv=dk,
                        block_mask=torch.ones(1, 4, 7, 8, dtype=torch.int8, device="cuda"))
    assert _cabi.device_status() == 0
