"""Generates the fixtures in this directory by running MindIE-SD's own Python code on CPU.

    python tests/golden/make_golden.py /path/to/MindIE-SD [rope|causal]

(`rope` regenerates only the rotary-embedding fixture, `causal` only the causal ada_bsa fixture.)

The reference is imported with `torch_npu` replaced by a mock, exactly as its own CPU test runner
does (tests/run.py:29-41 of MindIE-SD); only its pure-torch functions are called:
attention_forward(fused=False), rotary_position_embedding(fused=False), avgpool, rearrange_with_remaining, inv_rearrange_with_remaining,
do_tensor_rearrange_pooling, get_blockwise_mask, get_mask_index, and the numpy goldens of its plugin tests
(tests/plugin/test_block_sparse_attention.py, test_sparseblockestimate.py,
test_adablocksparseattention.py).  Masks are stored bit-packed.
"""
import importlib.util
import os
import sys
from importlib.util import spec_from_loader
from pathlib import Path
from unittest.mock import MagicMock

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import inputs  # noqa: E402


def import_reference(root):
    os.environ["MINDIE_LOG_TO_FILE"] = "false"
    os.environ["MINDIE_TEST_MODE"] = "CPU"
    mock = MagicMock()
    mock.__spec__ = spec_from_loader("torch_npu", loader=None)
    mock.npu.device_count = MagicMock(return_value=0)
    mock.npu.is_available = MagicMock(return_value=False)
    sys.modules["torch_npu"] = mock
    torch.npu = mock.npu
    sys.path.insert(0, root)
    import mindiesd  # noqa: F401
    from mindiesd.layers.flash_attn import sparse_flash_attn_rf_v2 as rf
    from mindiesd.layers.flash_attn.attention_forward import attention_forward
    mods = []
    for name in ("test_block_sparse_attention", "test_sparseblockestimate", "test_adablocksparseattention"):
        spec = importlib.util.spec_from_file_location("ref_" + name, os.path.join(root, "tests", "plugin", name + ".py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods.append(mod)
    return rf, attention_forward, mods


ROPE_CASES = [
    # (name, shape of x, head_first, table shape, table dtype, x dtype, mode, seed)
    ("half_bsnd_fp32tab", (2, 37, 3, 128), False, (37, 128), torch.float32, torch.bfloat16, "rotated_half", 61),
    ("inter_bnsd_fp32tab", (1, 2, 50, 128), True, (1, 1, 50, 128), torch.float32, torch.bfloat16, "rotated_interleaved", 62),
    ("half_bsnd_fp16", (2, 64, 8, 16), False, (1, 64, 1, 16), torch.float32, torch.float16, "rotated_half", 63),
    ("inter_bsnd_bf16tab", (1, 33, 2, 64), False, (1, 33, 1, 64), torch.bfloat16, torch.bfloat16, "rotated_interleaved", 64),
    ("half_sbnd_fp32", (20, 2, 3, 32), False, (20, 1, 1, 32), torch.float32, torch.float32, "rotated_half", 65),
]


def make_rope(root):
    """rotary_position_embedding(fused=False) of the reference on seeded inputs."""
    import_reference(root)
    from mindiesd.layers.rope import rotary_position_embedding
    out = {}
    for name, xs, head_first, ts, tdt, xdt, mode, seed in ROPE_CASES:
        x = inputs.randn(seed, *xs, dtype=xdt)
        cos, sin = inputs.randn(seed + 100, *ts, dtype=tdt), inputs.randn(seed + 200, *ts, dtype=tdt)
        y = rotary_position_embedding(x, cos, sin, mode, head_first, False)
        assert y.dtype == xdt
        out[name] = y.float().numpy()
    np.savez_compressed(HERE / "rope.npz", **out)


def make_causal(root):
    """The causal branches of the two ada_bsa goldens: the estimator's mask on the structured cases, and the
    attention over a lower-triangular block mask that keeps the diagonal blocks."""
    _, _, (_, est, ada) = import_reference(root)
    out = {}
    for (name, grid, heads, threshold, row_sparse, seed) in inputs.ESTIMATE_CASES:
        q, k = inputs.structured_qk(seed, heads, grid, 128)
        q, k = q.float().numpy(), k.float().numpy()
        m = est.sparse_estimate_cpu(q, k, True, blocksize=128, stride=8, threshold=threshold, force_sparse=row_sparse)
        out[f"{name}_shape"] = np.array(m.shape, dtype=np.int32)
        out[f"{name}_bits"] = np.packbits(m.reshape(-1))
        print("causal", name, m.shape, "density %.4f" % m.mean())
    q, k, v = (inputs.randn(41 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    mask = torch.zeros(1, 2, 3, 32, dtype=torch.int8)
    mask[..., :3] = torch.tril(torch.ones(3, 3, dtype=torch.int8))
    mask[0, 1, 2, 1] = 0  # a hole below the diagonal
    o = ada.ada_block_sparse_attention_cpu(q, k, v, mask, causal=True, blocksize=128)
    out["attention_mask"] = mask.numpy()
    out["attention_out"] = o.numpy()
    np.savez_compressed(HERE / "ada_causal.npz", **out)


def main(root):
    rf, attention_forward, (bsa, est, ada) = import_reference(root)
    torch.set_num_threads(8)
    make_rope(root)
    make_causal(root)

    # 1. permutations: the reference applied to a tensor whose value is its own token index
    perm = {}
    for (t, h, w) in inputs.PERM_GRIDS:
        s = t * h * w
        ids = torch.arange(s, dtype=torch.float32)
        for layout in ("BNSD", "BSND"):
            x = ids.reshape(1, 1, s, 1) if layout == "BNSD" else ids.reshape(1, s, 1, 1)
            y = rf.rearrange_with_remaining(x, (t, h, w), (t, h, w), layout)
            back = rf.inv_rearrange_with_remaining(y, (t, h, w), (t, h, w), layout)
            assert torch.equal(back, x)
            perm[f"{t}x{h}x{w}_{layout}"] = y.reshape(-1).to(torch.int32).numpy()
    np.savez_compressed(HERE / "permutation.npz", **perm)

    # 2. avgpool known answers (tail block included), both layouts
    x = inputs.randn(3, 1, 2, 300, 16)
    np.savez_compressed(
        HERE / "avgpool.npz",
        bnsd=rf.avgpool(x, 128, "BNSD").numpy(),
        bsnd=rf.avgpool(x.transpose(1, 2).contiguous(), 128, "BSND").numpy())

    # 3. masks: reference invoked on fp32 upcasts of bf16 data
    out = {}
    for (name, grid, txt, heads, dim, sparsity, layout, seed) in inputs.MASK_CASES:
        q, k = inputs.structured_qk(seed, heads, grid, dim, txt)
        q, k = q.float(), k.float()
        if layout == "BSND":
            q, k = q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous()
        v = torch.zeros_like(q)
        q_, k_, _, pool = rf.do_tensor_rearrange_pooling(q, k, v, txt, 128, grid, grid, layout)
        scale = dim ** -0.5
        mask = rf.get_blockwise_mask(pool, txt, sparsity, scale, 128, grid, grid, layout, return_binary=True)
        out[f"{name}_mask_shape"] = np.array(mask.shape, dtype=np.int32)
        out[f"{name}_mask_bits"] = np.packbits(mask.numpy().astype(bool).reshape(-1))
        if name in ("aligned", "text_ragged"):
            sel, num = rf.get_blockwise_mask(pool, txt, sparsity, scale, 128, grid, grid, layout)
            out[f"{name}_select_idx"] = sel.numpy().astype(np.int32)
            out[f"{name}_select_num"] = num.numpy().astype(np.int32)
            out[f"{name}_qpool"] = torch.chunk(pool, 3, dim=0)[0].numpy()
        # margin of the decision: smallest relative gap between the threshold and the next score below it
        qp, kp, _ = torch.chunk(pool, 3, dim=0)
        if layout == "BSND":
            qp, kp = qp.transpose(1, 2), kp.transpose(1, 2)
        sc = torch.einsum("bnld,bnsd->bnls", qp.double(), kp.double())
        keep = int(np.ceil(sc.shape[-1] * (1 - sparsity)))
        srt = sc.sort(-1, descending=True).values
        if keep < sc.shape[-1]:
            gap = (srt[..., keep - 1] - srt[..., keep]).abs() / srt[..., keep - 1].abs().clamp_min(1e-30)
            out[f"{name}_min_margin"] = np.array(gap.min().item())
        print(name, tuple(mask.shape), "density %.4f" % mask.float().mean().item(),
              "min margin", out.get(f"{name}_min_margin"))
    np.savez_compressed(HERE / "mask.npz", **out)

    # 4. get_mask_index
    m = torch.from_numpy(np.random.RandomState(5).rand(1, 2, 9, 9) < 0.4)
    np.savez_compressed(HERE / "mask_index.npz", mask=m.numpy(), index=rf.get_mask_index(m).numpy().astype(np.int32))

    # 5. dense attention, the unfused reference formula
    dense = {}
    for tag, dtype, head_first, sq, skv in (("fp32_bnsd", torch.float32, True, 200, 200),
                                            ("bf16_bsnd", torch.bfloat16, False, 160, 333),
                                            ("fp16_bnsd", torch.float16, True, 130, 257)):
        shape_q = (1, 2, sq, 128) if head_first else (1, sq, 2, 128)
        shape_k = (1, 2, skv, 128) if head_first else (1, skv, 2, 128)
        q, k, v = inputs.randn(21, *shape_q, dtype=dtype), inputs.randn(22, *shape_k, dtype=dtype), \
            inputs.randn(23, *shape_k, dtype=dtype)
        o = attention_forward(q, k, v, fused=False, head_first=head_first)
        dense[tag] = o.float().numpy()
    np.savez_compressed(HERE / "dense.npz", **dense)

    # 6. block-sparse attention, the numpy golden of the reference's plugin test
    q, k, v = (inputs.randn(31 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    mask = torch.from_numpy((np.random.RandomState(34).rand(1, 2, 3, 3) < 0.5).astype(np.int8))
    mask[0, 0, 1, :] = 0  # a row that keeps nothing
    o = bsa.block_sparse_attention_cpu(q, k, v, mask, 128)
    np.savez_compressed(HERE / "block_sparse.npz", mask=mask.numpy(), out=o.numpy())

    # 7. ada_bsa: the estimator's numpy golden on structured inputs (bf16 values, fp32 arithmetic)
    out = {}
    for (name, grid, heads, threshold, row_sparse, seed) in inputs.ESTIMATE_CASES:
        q, k = inputs.structured_qk(seed, heads, grid, 128)
        q, k = q.float().numpy(), k.float().numpy()
        m = est.sparse_estimate_cpu(q, k, False, blocksize=128, stride=8, threshold=threshold, force_sparse=row_sparse)
        out[f"{name}_shape"] = np.array(m.shape, dtype=np.int32)
        out[f"{name}_bits"] = np.packbits(m.reshape(-1))
        print(name, m.shape, "density %.4f" % m.mean())
    np.savez_compressed(HERE / "estimate.npz", **out)

    # 8. ada_bsa: the attention golden (mask columns padded to a multiple of 32, as the operator takes them)
    q, k, v = (inputs.randn(41 + i, 1, 2, 300, 128, dtype=torch.bfloat16) for i in range(3))
    mask = torch.zeros(1, 2, 3, 32, dtype=torch.int8)
    mask[..., :3] = torch.from_numpy((np.random.RandomState(44).rand(1, 2, 3, 3) < 0.6).astype(np.int8))
    mask[0, 1, 2, :] = 0  # a row that keeps nothing
    o = ada.ada_block_sparse_attention_cpu(q, k, v, mask, causal=False, blocksize=128)
    np.savez_compressed(HERE / "ada_attention.npz", mask=mask.numpy(), out=o.numpy())


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3) or (len(sys.argv) == 3 and sys.argv[2] not in ("rope", "causal")):
        raise SystemExit("usage: python tests/golden/make_golden.py <path of a MindIE-SD source tree> [rope|causal]")
    if len(sys.argv) == 3:
        {"rope": make_rope, "causal": make_causal}[sys.argv[2]](sys.argv[1])
    else:
        main(sys.argv[1])
