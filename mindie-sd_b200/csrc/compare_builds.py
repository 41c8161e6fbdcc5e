"""Times several builds of the C-ABI library against one another in ONE process on one GPU.

    python mindie-sd_b200/csrc/build.py --variant /tmp/m5.so -D SDB_FA_BF16_MODE=5
    python mindie-sd_b200/csrc/compare_builds.py dense 3 4 product /tmp/m5.so

Arguments: workload (dense | c2 | fp8 | sparse), repetitions, launches per repetition, then the libraries:
paths of .so files, or `product` for the one the package loads.  `path+pairs` (sparse only) runs that library
with the query blocks paired by the overlap of their key lists (mindiesd_rf_pair_blocks of the product library).

Why one process: at the benchmark shape the attention kernel runs under the power cap, and a few per cent lie
between two boxes, or between a cold and a warm GPU.  Here every build sees the same inputs, the same GPU and
the same thermal state, the builds alternate within every repetition, and the first build's output is the
reference the others are compared with (max abs difference; builds that differ only in code placement must
give 0).  Prints per build the median and minimum milliseconds per launch, dense-equivalent TFLOP/s at the
median, the SM clock sampled while its launches ran, and every repetition.
"""
from __future__ import annotations

import ctypes as C
import statistics
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
for _p in (ROOT, ROOT / "mindie-sd_b200"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

import workloads  # noqa: E402
from mindiesd import _cabi  # noqa: E402


def sm_clock() -> float:
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits", "-i",
                              str(torch.cuda.current_device())], capture_output=True, text=True).stdout
        return float(out.split()[0])
    except Exception:  # noqa: BLE001
        return float("nan")


def main(argv):
    if len(argv) < 5:
        raise SystemExit(__doc__)
    wl, reps, launches, names = argv[1], int(argv[2]), int(argv[3]), argv[4:]
    cfg = workloads.C2 if wl == "c2" else workloads.C3
    q, k, v = workloads.make_qkv(workloads.C4 if wl == "fp8" else cfg, "cuda", seed=0)
    b, n, s, d = q.shape
    out = torch.empty(q.shape, dtype=torch.bfloat16, device="cuda")
    scales = mask = pairs = None
    if wl == "fp8":
        q, qs = _cabi.fa_block_quant(q, 128, rotate=True)
        k, ks = _cabi.fa_block_quant(k, 128, rotate=True)
        v, vs = _cabi.fa_block_quant(v, per_channel=True)
        scales = (qs, ks, vs)
    if wl == "sparse":
        mask = _cabi.rf_block_mask(q, k, cfg.grid, 0, 0.75, True)
        q, k, v = (_cabi.rf_rearrange(x, cfg.grid, 0, True) for x in (q, k, v))
        pairs = _cabi.rf_pair_blocks(mask)
        print(f"block mask density {mask.float().mean().item():.4f}")

    def args_for(with_pairs):
        a = _cabi.AttnArgs()
        a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
        a.batch, a.heads, a.kv_heads, a.seq_q, a.seq_kv, a.head_dim = b, n, n, s, s, d
        for f in ("q_stride", "k_stride", "v_stride", "o_stride"):
            getattr(a, f)[:] = _cabi.strides_bns(q, True)
        a.in_dtype, a.out_dtype = (3 if wl == "fp8" else 0), 0
        a.scale = d ** -0.5
        a.block_size = 128
        if scales:
            a.q_scale, a.k_scale, a.v_scale = (t.data_ptr() for t in scales)
            a.k_scale_block, a.v_scale_block = 128, 0
        if mask is not None:
            a.sparse_mode = _cabi.SPARSE_MASK
            a.block_mask = mask.data_ptr()
            a.mask_stride[:] = [mask.stride(0), mask.stride(1), mask.stride(2)]
            if with_pairs:
                a.q_pairs, a.q_pair_count = pairs.data_ptr(), pairs.shape[-2]
        return a

    libs, args_of = {}, {}
    for name in names:
        path, _, opt = name.partition("+")
        handle = C.CDLL(str(_cabi.library_path()) if path == "product" else path)
        handle.mindiesd_attention_fwd.restype = C.c_int
        handle.mindiesd_attention_fwd.argtypes = [C.c_void_p, C.c_void_p]
        libs[name] = handle
        args_of[name] = args_for(opt == "pairs")
    stream = _cabi.current_stream_ptr(q.device)
    ref = None
    for name, handle in libs.items():
        out.zero_()
        rc = handle.mindiesd_attention_fwd(C.byref(args_of[name]), stream)
        torch.cuda.synchronize()
        probe = out[0, :2, ::997].float().clone()
        ref = probe if ref is None else ref
        print(f"{name}: rc {rc}, max abs difference to the first build {(probe - ref).abs().max().item():.2e}", flush=True)

    times = {name: [] for name in names}
    clocks = {name: [] for name in names}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(reps):
        for name, handle in libs.items():
            handle.mindiesd_attention_fwd(C.byref(args_of[name]), stream)
            e0.record()
            for _ in range(launches):
                handle.mindiesd_attention_fwd(C.byref(args_of[name]), stream)
            e1.record()
            clocks[name].append(sm_clock())  # sampled while the launches run
            torch.cuda.synchronize()
            times[name].append(e0.elapsed_time(e1) / launches)
    flops = 4.0 * b * n * s * s * d
    print(f"== {wl}: ms per launch (median of {reps} x {launches}), min, dense-equivalent TFLOP/s, SM MHz, repetitions")
    for name in names:
        med = statistics.median(times[name])
        print(f"{name:24s} {med:9.3f} {min(times[name]):9.3f} {flops / med / 1e9:9.1f} {statistics.median(clocks[name]):7.0f}   "
              + " ".join(f"{x:.2f}" for x in times[name]), flush=True)
    if _cabi.device_status() != 0:
        raise SystemExit("a kernel set the device status word")


if __name__ == "__main__":
    main(sys.argv)
