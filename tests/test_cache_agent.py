"""Host logic of the attention cache and the block-mask cache (CPU only): which (step, block) calls
compute and which reuse, following the schedule of MindIE-SD's AttentionCache
(mindiesd/cache_agent/attention_cache.py:22-31)."""
import pytest

from mindiesd import CacheAgent, CacheConfig, ConfigError, ParametersInvalid


def _expected_reuse(step, start, interval, end):
    return start < step <= end and (step - start) % interval != 0


@pytest.mark.parametrize("start,interval,end", [(0, 2, 10000), (2, 3, 8), (1, 4, 5)])
def test_attention_cache_schedule(start, interval, end):
    blocks, steps = 3, 10
    agent = CacheAgent(CacheConfig("attention_cache", blocks, steps, step_start=start, step_interval=interval, step_end=end))
    for run in range(2):  # the counters wrap after steps_count steps and the cache is dropped
        calls = []
        for step in range(steps):
            for block in range(blocks):
                out = agent.apply(lambda s=step, b=block: calls.append((s, b)) or (s, b))
                if _expected_reuse(step, start, interval, end):
                    last = max(s for s in range(step) if not _expected_reuse(s, start, interval, end))
                    assert out == (last, block)
                else:
                    assert out == (step, block)
        assert calls == [(s, b) for s in range(steps) for b in range(blocks) if not _expected_reuse(s, start, interval, end)]


def test_cache_agent_pass_through_and_errors():
    n = []
    agent = CacheAgent(CacheConfig("attention_cache", 2, 4, step_interval=1))
    for _ in range(8):
        agent.apply(lambda: n.append(1))
    assert len(n) == 8
    with pytest.raises(ParametersInvalid):
        agent.apply(3)
    with pytest.raises(ConfigError):
        CacheAgent(CacheConfig("nope", 2, 4))
    with pytest.raises(ConfigError):
        CacheAgent(CacheConfig("dit_block_cache", 2, 4))
    with pytest.raises(ConfigError):
        CacheAgent(CacheConfig("attention_cache", 0, 4))
    with pytest.raises(ConfigError):
        CacheAgent(CacheConfig("attention_cache", 2, 4, step_start=5, step_end=3))


def test_block_mask_cache_hands_the_kept_mask_back():
    blocks, steps = 2, 6
    agent = CacheAgent(CacheConfig("block_mask_cache", blocks, steps, step_start=0, step_interval=3))
    seen = []

    def attention(tag, cached_mask=None):
        seen.append((tag, cached_mask))
        return f"out{tag}", cached_mask if cached_mask is not None else f"mask{tag}"

    for step in range(steps):
        for block in range(blocks):
            assert agent.apply(attention, (step, block)) == f"out{(step, block)}"
    for (step, block), cached in seen:
        if step % 3 == 0:
            assert cached is None  # the builder runs
        else:
            assert cached == f"mask{(step - step % 3, block)}"


def test_default_host_chunks():
    from mindiesd.layers.flash_attn.host_io import default_host_chunks
    assert default_host_chunks(40, 75600) == 40   # one head per chunk still launches two waves
    assert default_host_chunks(12, 32760) == 4    # 128 thread blocks per head: three heads per chunk
    assert default_host_chunks(2, 300) == 1
    assert default_host_chunks(7, 1 << 20) == 7


def test_fp8_hook_rejects_a_single_rotation_matrix():
    """q k^T survives the rotation only if both operands are rotated: a checkpoint that lacks one of the
    two matrices is an error, as it is in MindIE-SD (its matmul receives None, quantization/layer.py:284-285)."""
    import torch
    from mindiesd import FP8RotateQuantFA
    rot = torch.eye(128)
    FP8RotateQuantFA("blk", {"blk.q_rot": rot, "blk.k_rot": rot})
    FP8RotateQuantFA("blk", {})
    for name in ("q_rot", "k_rot"):
        with pytest.raises(ParametersInvalid):
            FP8RotateQuantFA("blk", {f"blk.{name}": rot})
