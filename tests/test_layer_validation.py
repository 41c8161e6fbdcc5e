"""Argument checks of the layer API that run before any kernel: the rejections the reference's own tests
expect (tests/layers/flash_attn/test_attention_forward_varlen.py:210-346, test_attn_forward.py,
tests/layers/test_rope.py of MindIE-SD), with the same exception type and the same message fragments.  No
device is needed: everything here fails on the host."""
import pytest
import torch


def _qkv(total=24, heads=2, dim=64):
    return tuple(torch.randn(total, heads, dim) for _ in range(3))


CU = torch.tensor([0, 10, 24], dtype=torch.int32)


@pytest.mark.parametrize("which", ["q", "k", "v"])
def test_varlen_wants_three_dimensional_operands(which):
    from mindiesd import attention_forward_varlen, ParametersInvalid
    q, k, v = _qkv()
    args = dict(q=q, k=k, v=v)
    args[which] = torch.randn(24, 64)
    with pytest.raises(ParametersInvalid, match=f"Expected {which} to be 3D"):
        attention_forward_varlen(cu_seqlens_q=CU, cu_seqlens_k=CU, dropout_p=0.0, **args)


def test_varlen_rejects_dropout():
    from mindiesd import attention_forward_varlen, ParametersInvalid
    q, k, v = _qkv()
    with pytest.raises(ParametersInvalid, match="dropout_p should be set to 0.0 during evaluation"):
        attention_forward_varlen(q, k, v, CU, CU, dropout_p=0.1)


@pytest.mark.parametrize("name,value,shown", [
    ("max_seqlen_q", 128, "max_seqlen_q=128"),
    ("max_seqlen_k", 128, "max_seqlen_k=128"),
    ("window_size", 64, "window_size=64"),
    ("softcap", 30.0, "softcap=30.0"),
    ("alibi_slopes", torch.randn(4), "alibi_slopes="),
    ("deterministic", True, "deterministic=True"),
    ("return_attn_probs", True, "return_attn_probs=True"),
    ("block_table", torch.tensor([0, 1, 2], dtype=torch.int32), "block_table="),
])
def test_varlen_reserved_arguments_must_stay_none(name, value, shown):
    from mindiesd import attention_forward_varlen, ParametersInvalid
    q, k, v = _qkv()
    with pytest.raises(ParametersInvalid) as err:
        attention_forward_varlen(q, k, v, CU, CU, **{name: value})
    assert shown in str(err.value) and "Unsupported parameters in varlen attention" in str(err.value)


def test_varlen_lengths_must_end_at_the_token_count():
    from mindiesd import attention_forward_varlen, ParametersInvalid
    q, k, v = _qkv()
    short = torch.tensor([0, 10, 20], dtype=torch.int32)
    with pytest.raises(ParametersInvalid, match="cumulative lengths"):
        attention_forward_varlen(q, k, v, short, CU)
    with pytest.raises(ParametersInvalid, match="cumulative lengths"):
        attention_forward_varlen(q, k, v, torch.tensor([24], dtype=torch.int32), torch.tensor([24], dtype=torch.int32))


def test_attention_forward_checks_types_and_ranks():
    from mindiesd import attention_forward, ParametersInvalid
    q = torch.randn(1, 16, 2, 64)
    with pytest.raises(ParametersInvalid, match="input query must be torch.Tensor"):
        attention_forward([1, 2], q, q)
    with pytest.raises(ParametersInvalid, match="dimensional of input key must be 4"):
        attention_forward(q, q[0], q)
    with pytest.raises(ParametersInvalid, match="input fused must be bool"):
        attention_forward(q, q, q, fused=1)
    with pytest.raises(ParametersInvalid, match="input attn_mask must be torch.Tensor"):
        attention_forward(q, q, q, attn_mask=[0])
    with pytest.raises(ParametersInvalid, match="input scale must be float"):
        attention_forward(q, q, q, scale=1)


def test_attention_forward_checks_the_mode_keywords():
    from mindiesd import attention_forward, ParametersInvalid
    q = torch.randn(1, 16, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(ParametersInvalid, match="'opt_mode':eager is invalid"):
        attention_forward(q, q, q, opt_mode="eager")
    with pytest.raises(ParametersInvalid, match="Unsupported FA type: 'flash3'"):
        attention_forward(q, q, q, opt_mode="manual", op_type="flash3")
    with pytest.raises(ParametersInvalid, match="Unsupported layout: 'SBH'"):
        attention_forward(q, q, q, opt_mode="manual", op_type="fused_attn_score", layout="SBH")
    with pytest.raises(ParametersInvalid, match="takes no attn_mask"):
        attention_forward(q, q, q, attn_mask=torch.zeros(16, 16))
    with pytest.raises(ParametersInvalid, match="supports bfloat16 and float16"):
        attention_forward(q.float(), q.float(), q.float())


def test_attention_forward_unfused_is_the_reference_formula_on_any_device():
    """fused=False never reaches a kernel: softmax(q k^T * scale [+ mask]) v, in both layouts."""
    from mindiesd import attention_forward
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(2, 10, 3, 16, generator=g) for _ in range(3))
    want = torch.softmax(torch.einsum("bqnd,bknd->bnqk", q, k) * 16 ** -0.5, -1)
    want = torch.einsum("bnqk,bknd->bqnd", want, v)
    got = attention_forward(q, k, v, fused=False)
    assert torch.allclose(got, want, atol=1e-5)
    got_hf = attention_forward(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), fused=False, head_first=True)
    assert torch.allclose(got_hf.transpose(1, 2), want, atol=1e-5)


def test_sparse_attention_checks_layout_and_type():
    from mindiesd import sparse_attention, ParametersInvalid
    q = torch.randn(1, 2, 256, 128, dtype=torch.bfloat16)
    with pytest.raises(ParametersInvalid, match="input_layout must in"):
        sparse_attention(q, q, q, head_num=2, input_layout="SBH", sparse_type="rf_v2")
    with pytest.raises(ParametersInvalid, match="sparse_type must be"):
        sparse_attention(q, q, q, head_num=2, input_layout="BNSD", sparse_type="topk")


def test_rotary_embedding_checks_its_arguments():
    from mindiesd import rotary_position_embedding, ParametersInvalid
    x = torch.randn(1, 8, 2, 16)
    cos, sin = torch.randn(8, 16), torch.randn(8, 16)
    with pytest.raises(ParametersInvalid, match="input cos must be torch.Tensor"):
        rotary_position_embedding(x, [1.0], sin, fused=False)
    with pytest.raises(ParametersInvalid, match="input rotated_mode must be str"):
        rotary_position_embedding(x, cos, sin, rotated_mode=1, fused=False)
    with pytest.raises(ParametersInvalid, match="input x must be a 4"):
        rotary_position_embedding(x[0], cos, sin, fused=False)
    with pytest.raises(ParametersInvalid, match="must be a 2 or 4"):
        rotary_position_embedding(x, cos[None], sin[None], fused=False)
    with pytest.raises(ParametersInvalid, match="Unsupported rotated_mode"):
        rotary_position_embedding(x, cos, sin, rotated_mode="rotated_quarter", fused=False)
    with pytest.raises(ParametersInvalid, match="runs on a CUDA device"):
        rotary_position_embedding(x, cos, sin, fused=True)


def test_ulysses_rejects_bad_piece_sizes_and_transports():
    from mindiesd.parallel.ulysses import _piece_sizes
    from mindiesd import ParametersInvalid
    assert _piece_sizes([2, 3], 5, 75600, 1) == [2, 3]
    assert _piece_sizes(5, 10, 75600, 1) == [2] * 5
    with pytest.raises(ParametersInvalid, match="must divide"):
        _piece_sizes(3, 10, 75600, 1)
    with pytest.raises(ParametersInvalid, match="adding up"):
        _piece_sizes([2, 2], 5, 75600, 1)
    with pytest.raises(ParametersInvalid, match="adding up"):
        _piece_sizes([0, 5], 5, 75600, 1)


def test_results_are_remembered_per_attention_shape():
    """tests/layers/flash_attn/test_attn_lru_cache.py of MindIE-SD, plus the eviction order."""
    from mindiesd.layers.flash_attn.common import AttentionParam, attn_cache, lru_cache_by_attn_param
    calls = []

    @lru_cache_by_attn_param(maxsize=2)
    def pick(param):
        calls.append(param.batch_size)
        return "case 0" if param.batch_size > 10 else "case 1"

    attn_cache.clear()
    big = AttentionParam(20, 16, 64, 128, 128, torch.float32, False)
    small = AttentionParam(2, 16, 64, 128, 128, torch.float32, False)
    other = AttentionParam(3, 16, 64, 128, 128, torch.float32, True)
    assert pick(big) == "case 0" and big.to_hash() in attn_cache and attn_cache[big.to_hash()] == "case 0"
    assert pick(small) == "case 1" and pick(big) == "case 0" and calls == [20, 2]  # the second call of `big` was remembered
    pick(other)  # a third shape: the least recently used one (small) goes
    assert small.to_hash() not in attn_cache and big.to_hash() in attn_cache and len(attn_cache) == 2
    attn_cache.clear()
