"""The mask builder entry point that allocates nothing (`mindiesd_rf_block_mask_static`).

Some hosts of the library hand all device memory to their own arena, or run a step loop where a
cudaMalloc would stall the device, so they cannot give the ordinary entry point a scratch buffer
per call.  This variant keeps its scratch in a fixed 4 MiB array inside the library.  The test
calls it through the C ABI twice in a row on different inputs -- the second call finds the first
call's values in the shared array -- and requires the same mask and block lists, bit for bit, as
the ordinary entry point gives.  It runs last so that a failure here cannot hide another test.
"""
import ctypes

import pytest
import torch

import inputs

pytestmark = pytest.mark.gpu


def test_static_scratch_variant_matches_ordinary_entry_point_twice():
    from mindiesd import _cabi
    cases = [((3, 30, 52), 200, 2, 0.6, 301), ((2, 24, 45), 0, 3, 0.25, 302)]
    for grid, txt, heads, sparsity, seed in cases:
        q, k = inputs.structured_qk(seed, heads, grid, 128, txt)
        q, k = q.cuda(), k.cuda()
        want = _cabi.rf_block_mask(q, k, grid, txt, sparsity, True, want_lists=True)
        before = torch.cuda.memory_allocated()
        got = _cabi.rf_block_mask_static(q, k, grid, txt, sparsity, True, want_lists=True)
        blocks = want[0].shape[-1]
        outputs = blocks * blocks * heads + 8 * blocks * heads * blocks + 8 * blocks * heads
        assert torch.cuda.memory_allocated() - before <= outputs + 3 * 512  # only the three output tensors
        for g, w in zip(got, want):
            assert torch.equal(g, w)
    assert _cabi.device_status() == 0


def test_static_scratch_variant_rejects_sizes_beyond_its_capacity():
    from mindiesd import _cabi
    lib = _cabi.lib()
    lib.mindiesd_rf_block_mask_static_capacity.restype = ctypes.c_size_t
    assert lib.mindiesd_rf_block_mask_static_capacity() == 4 << 20
    grid = (21, 45, 80)  # 591 blocks: 40 heads need 12 MiB of pooled means
    q = torch.zeros(1, 40, 75600, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_cabi.NativeLibraryError, match="capacity"):
        _cabi.rf_block_mask_static(q, q, grid, 0, 0.75, True)
