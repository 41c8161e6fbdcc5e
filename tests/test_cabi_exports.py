"""CPU checks of the boundary: the C-ABI library loads, exports every function the public header
declares, and the Python-side structs have the sizes the header implies.  No compute."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "mindiesd_b200.h"


def _declared_functions():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|size_t)\s+(mindiesd_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mindiesd import _cabi
    lib = ctypes.CDLL(str(_cabi.library_path()))
    names = _declared_functions()
    assert "mindiesd_attention_fwd" in names and len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/mindiesd_b200.h but not exported"
    lib.mindiesd_abi_version.restype = ctypes.c_int
    assert lib.mindiesd_abi_version() == 3


def test_struct_layouts_match_the_header(tmp_path):
    """Compiles a tiny C program that prints sizeof() of every argument struct."""
    import shutil
    import subprocess
    from mindiesd import _cabi
    cc = shutil.which("gcc")
    if cc is None:
        pytest.skip("no C compiler")
    structs = {"mindiesd_attn_args": _cabi.AttnArgs, "mindiesd_rearrange_args": _cabi.RearrangeArgs,
               "mindiesd_mask_args": _cabi.MaskArgs, "mindiesd_pool_args": _cabi.PoolArgs,
               "mindiesd_pooled_mask_args": _cabi.PooledMaskArgs, "mindiesd_quant_args": _cabi.QuantArgs,
               "mindiesd_estimate_args": _cabi.EstimateArgs, "mindiesd_rotate_quant_args": _cabi.RotateQuantArgs,
               "mindiesd_pair_args": _cabi.PairArgs}
    src = tmp_path / "sz.c"
    body = "".join(f'printf("{n} %zu\\n", sizeof({n}));' for n in structs)
    src.write_text(f'#include <stdio.h>\n#include "mindiesd_b200.h"\nint main(void){{{body}return 0;}}\n')
    exe = tmp_path / "sz"
    subprocess.run([cc, "-I", str(HEADER.parent), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    for line in out.strip().splitlines():
        name, size = line.split()
        assert ctypes.sizeof(structs[name]) == int(size), name


def test_invalid_arguments_return_codes_without_a_gpu():
    """Argument checks that precede any CUDA call."""
    from mindiesd import _cabi
    lib = _cabi.lib()
    assert lib.mindiesd_attention_fwd(None, None) == -1
    a = _cabi.AttnArgs()
    assert lib.mindiesd_attention_fwd(ctypes.byref(a), None) == -1  # NULL tensors
    a.q = a.k = a.v = a.out = 4096
    a.head_dim = 64
    assert lib.mindiesd_attention_fwd(ctypes.byref(a), None) == -2  # head_dim
    r = _cabi.RearrangeArgs()
    assert lib.mindiesd_rf_rearrange(ctypes.byref(r), None) == -1
    q = _cabi.QuantArgs()
    assert lib.mindiesd_fa_block_quant(ctypes.byref(q), None) == -1
    rq = _cabi.RotateQuantArgs()
    assert lib.mindiesd_fa_rotate_quant(ctypes.byref(rq), None) == -1
    rq.x = rq.rot = rq.out = rq.scales = 4096
    rq.batch = rq.heads = 1
    rq.seq, rq.head_dim, rq.row_block = 256, 128, 100
    assert lib.mindiesd_fa_rotate_quant(ctypes.byref(rq), None) == -2  # row_block
    e = _cabi.EstimateArgs()
    assert lib.mindiesd_sparse_block_estimate(ctypes.byref(e), None) == -1
    e.q = e.k = e.mask = e.count = e.scratch = 4096
    e.batch = e.heads = e.kv_heads = 1
    e.head_dim, e.stride, e.sparse_size, e.scale, e.threshold = 128, 8, 128, 0.01, 0.9
    e.seq = 1001
    assert lib.mindiesd_sparse_block_estimate(ctypes.byref(e), None) == -2  # not a multiple of 8 tokens
    e.seq, e.causal, e.causal_key_tokens = 1024, 1, 2000
    assert lib.mindiesd_sparse_block_estimate(ctypes.byref(e), None) == -5  # more key tokens than tokens
    e.causal = e.causal_key_tokens = 0
    assert lib.mindiesd_sparse_block_estimate_scratch_bytes(1, 40, 75600) == 4 * 9472 * (37 * 16 + 37) * 4
    pa = _cabi.PairArgs()
    assert lib.mindiesd_rf_pair_blocks(None, None) == -1
    assert lib.mindiesd_rf_pair_blocks(ctypes.byref(pa), None) == -1  # NULL mask and table
    pa.mask = pa.pairs = 4096
    pa.batch = pa.heads = pa.kv_blocks = 1
    assert lib.mindiesd_rf_pair_blocks(ctypes.byref(pa), None) == -2  # no query blocks
    pa.q_blocks, pa.kv_blocks = 8, 2000
    assert lib.mindiesd_rf_pair_blocks(ctypes.byref(pa), None) < 0    # beyond the capacity of one thread block
    mv = _cabi.UlyssesMoveArgs()
    assert lib.mindiesd_ulysses_move(ctypes.byref(mv), None) < 0
    ro = _cabi.RopeArgs()
    assert lib.mindiesd_rope(ctypes.byref(ro), None) == -1
    with pytest.raises(_cabi.NativeLibraryError):
        _cabi.check(-2, "x")


def test_operator_library_registers_reference_schemas():
    import torch
    import mindiesd  # noqa: F401  (loads the operator library)
    la = str(torch.ops.mindiesd.la.default._schema)
    assert "Tensor? atten_mask=None" in la and "bool is_highPrecision=True" in la and "int next_tokens=1" in la
    bsa = str(torch.ops.mindiesd.block_sparse_attention.default._schema)
    assert "int[] block_shape=" in bsa and "int softmax_lse_flag=0" in bsa and "int num_key_value_heads=1" in bsa
    est = str(torch.ops.mindiesd.sparse_block_estimate.default._schema)
    assert "int[]? actual_seq_lengths=None" in est and "bool keep_recent=True" in est and "float row_sparse=1" in est
    ada = str(torch.ops.mindiesd.ada_block_sparse_attention.default._schema)
    assert "Tensor sparse_count_table" in ada and "int pre_tokens=214748647" in ada and "-> Tensor" in ada
    rf = str(torch.ops.mindiesd.rainfusionattention.default._schema)
    assert "Tensor select_num_idx" in rf and "str q_input_layout=\"TND\"" in rf and "int inner_precise=1" in rf
