"""The give-up path of the attention kernel's bounded waits, exercised from the host without faulting
or hanging the GPU: a test field of the C ABI makes every loader withhold its first key block (no
copy is started, none is announced), the consumer's wait runs into a shortened time limit, the thread
blocks unwind, mark their rows with NaN and leave status 101 with the wait's number; the context
stays usable and the next launch is correct.  Plus two shapes in which warps legitimately wait for
the whole life of their thread block."""
import ctypes as C

import pytest
import torch

import inputs
from oracle import attention as oa

pytestmark = pytest.mark.gpu


def _detail():
    from mindiesd import _cabi
    out = (C.c_int32 * 8)()
    assert _cabi.lib().mindiesd_device_status_detail(out) == 0
    return list(out)


def test_withheld_copy_gives_up_cleanly_and_the_next_launch_is_correct():
    from mindiesd import _cabi
    assert _cabi.device_status() == 0
    q, k, v = (inputs.randn(800 + i, 1, 2, 700, 128, dtype=torch.bfloat16).cuda() for i in range(3))
    out = torch.zeros_like(q)
    lse_probe = _cabi.attention(q, k, v, out=out, wait_limit_us=20000, test_withhold=1)
    torch.cuda.synchronize()  # the kernel returned by itself: no fault, no hang
    detail = _detail()
    assert detail[0] == 101            # a bounded wait gave up
    # ... the MMA thread's wait for a key/value block, a softmax warp's wait for the scores that depend on it, or
    # the loader's wait for the ring slot the withheld copy never frees: every role times its own wait, they all
    # started within microseconds of each other, and whichever runs out first reports
    assert detail[1] in (1, 11, 12, 17, 20, 21), detail
    assert torch.isnan(out.float()).all()  # rows of a block that unwound are marked, never plausible numbers
    assert lse_probe is out
    # while the word is set, later launches leave at once and mark their rows too
    out2 = torch.zeros_like(q)
    _cabi.attention(q, k, v, out=out2)
    torch.cuda.synchronize()
    assert torch.isnan(out2.float()).all()
    assert _cabi.device_status() == 101  # reading clears it
    assert _cabi.device_status() == 0
    good = _cabi.attention(q, k, v)
    want = oa.attention_math(q.cpu(), k.cpu(), v.cpu(), head_first=True)
    assert (good.float().cpu() - want.float()).abs().max().item() <= 2e-2
    assert _cabi.device_status() == 0


def test_idle_tile_waits_for_the_whole_block_life_without_giving_up():
    """256 query rows against 131072 keys with a block mask that keeps every key block for the first
    tile and none for the second: the second tile's warps sit on one barrier until the thread block is
    done.  The wait is bounded by time, not by attempts, so its length does not matter."""
    from mindiesd import _cabi
    skv = 128 * 1024
    q = inputs.randn(810, 1, 1, 256, 128, dtype=torch.bfloat16)
    k, v = (inputs.randn(811 + i, 1, 1, skv, 128, dtype=torch.bfloat16) for i in range(2))
    mask = torch.zeros(1, 1, 2, skv // 128, dtype=torch.int8)
    mask[0, 0, 0] = 1
    out = _cabi.attention(q.cuda(), k.cuda(), v.cuda(), block_mask=mask.cuda())
    assert _cabi.device_status() == 0
    want = oa.attention_math(q[:, :, :128], k, v, head_first=True)
    assert (out[:, :, :128].float().cpu() - want.float()).abs().max().item() <= 2e-2
    assert torch.count_nonzero(out[:, :, 128:]).item() == 0  # rows that keep nothing give zeros


def test_block_sparse_lse_with_actual_length_below_padded_length():
    """block_sparse_attention in BNSD with actual_seq_lengths < S and softmax_lse_flag: the
    log-sum-exp goes to [B, N, S, 1] at the row's own position, rows past the real length are -inf."""
    import mindiesd  # noqa: F401  (registers the operators)
    b, n, s, real = 2, 2, 384, 300
    q, k, v = (inputs.randn(820 + i, b, n, s, 128, dtype=torch.bfloat16).cuda() for i in range(3))
    mask = torch.ones(b, n, 3, 3, dtype=torch.int8, device="cuda")
    out, _ = torch.ops.mindiesd.block_sparse_attention(
        query=q, key=k, value=v, block_sparse_mask=mask, actual_seq_lengths=[real] * b, actual_seq_lengths_kv=[real] * b,
        num_key_value_heads=n, scale_value=128 ** -0.5, softmax_lse_flag=1)
    _, lse = torch.ops.mindiesd.block_sparse_attention(
        query=q, key=k, value=v, block_sparse_mask=mask, actual_seq_lengths=[real] * b, actual_seq_lengths_kv=[real] * b,
        num_key_value_heads=n, scale_value=128 ** -0.5, softmax_lse_flag=1)
    assert lse.shape == (b, n, s, 1)
    sc = q[:, :, :real].float() @ k[:, :, :real].float().transpose(-1, -2) * 128 ** -0.5
    want = torch.logsumexp(sc, -1)
    assert (lse[:, :, :real, 0] - want).abs().max().item() < 2e-2
    assert torch.isinf(lse[:, :, real:, 0]).all() and (lse[:, :, real:, 0] < 0).all()
    want_out = oa.attention_math(q[:, :, :real].cpu(), k[:, :, :real].cpu(), v[:, :, :real].cpu(), head_first=True)
    assert (out[:, :, :real].float().cpu() - want_out.float()).abs().max().item() <= 2e-2
    assert torch.count_nonzero(out[:, :, real:]).item() == 0


def test_layer_api_raises_when_asked_to_check(monkeypatch):
    """MINDIESD_CHECK_STATUS=1: the layer entry reads the status word after its call and raises."""
    from mindiesd import _cabi, attention_forward, ModelExecError
    assert _cabi.device_status() == 0
    q, k, v = (inputs.randn(830 + i, 1, 300, 2, 128, dtype=torch.bfloat16).cuda() for i in range(3))
    _cabi.attention(q, k, v, head_first=False, wait_limit_us=20000, test_withhold=1)  # sets the word
    monkeypatch.setenv("MINDIESD_CHECK_STATUS", "1")
    with pytest.raises(ModelExecError):
        attention_forward(q, k, v)
    out = attention_forward(q, k, v)  # the word was cleared by the check: back to normal
    want = oa.attention_math(q.cpu(), k.cpu(), v.cpu(), head_first=False)
    assert (out.float().cpu() - want.float()).abs().max().item() <= 2e-2
