"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

The unit of work is one self-attention layer of the Wan2.1-14B 720p shape (B1 N40 S75600 D128, bf16,
dense): 117.05 TFLOP.  N = 1 runs the dense tcgen05 kernel on one GPU, one layer per step; N > 1 (under
torchrun, one rank per GPU) runs the same layer sequence-parallel with the Ulysses wrapper, a step
repeating the layer (`config.layers_per_step`) so that the timed region lasts about two seconds at
every N; the total work per layer is fixed ("strong" scaling) and `value` is the whole job's
dense-equivalent TFLOP/s.  Before the timed region every rank of an N > 1 run checks its Ulysses output
bit for bit against the single-GPU kernel on the unsharded tensors (`config.parity`), and after it the
rank's own heads are timed through the attention kernel alone in the same power state, so that
`config.phases_of_one_layer.exposed_ms` is what the exchange costs after all overlap.  `--ulysses-pieces
2,3` and `--ulysses-transport nccl|peer` override the library's choices.  Rank 0 prints one JSON line.  Inputs are seeded synthetic tensors of the named shapes (no dataset exists for this path);
3.1 GB of operands per step exceed the 126 MB L2, so no L2 flush is needed between steps.

Other single-GPU workloads of the same path (`--workload sparse|sparse_layer|fp8|fp8_layer|mask|quant|rotate_quant|rearrange|estimate|ada_layer|c2|ulysses_move|ulysses_move_rope`) print the
same kind of line for their kernel; `--impl reference` times the CPU oracle (the reference's
unfused torch formula) on the host cores for the same metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "mindie-sd_b200", ROOT / "tests" / "golden"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import torch  # noqa: E402

HEAD_DIM = 128
# DRAM bytes one launch of the dense kernel moves at the benchmark shape, from one ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum); None until a capture has been taken.
DENSE_DRAM_TRAFFIC_BYTES = 3.204e9  # 320.4 MB captured at 4 heads (259.9 read + 60.4 written), scaled by 10 (traffic is per head)


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def physical_gpu_index(local_index):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [x for x in vis.split(",") if x != ""]
        if local_index < len(ids) and ids[local_index].isdigit():
            return int(ids[local_index])
    return local_index


def timed(fn, steps, warmup, barrier=None):
    """Runs fn() warmup + steps times; returns elapsed milliseconds of the timed steps on the
    current stream (CUDA events, synchronised on both sides)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return e0.elapsed_time(e1)


# ---------------------------------------------------------------------------------------------------
# CPU oracle legs
# ---------------------------------------------------------------------------------------------------
def cpu_attention_sample(seq, target_seconds=12.0, repeats=1):
    """The reference's unfused attention formula on the host cores for one head and a block of
    query rows against the full key/value sequence (fp32 on bf16-rounded values).  The block is
    sized from a short probe so that the timed part takes about target_seconds."""
    from oracle import attention as oa
    g = torch.Generator().manual_seed(1234)
    k = (0.5 * torch.randn(1, 1, seq, HEAD_DIM, generator=g)).bfloat16().float()
    v = (0.5 * torch.randn(1, 1, seq, HEAD_DIM, generator=g)).bfloat16().float()

    def run(rows):
        q = (0.5 * torch.randn(1, 1, rows, HEAD_DIM, generator=g)).bfloat16().float()
        t0 = time.perf_counter()
        oa.attention_math_chunked(q, k, v, head_first=True, rows=1024)
        return time.perf_counter() - t0

    run(256)
    probe = run(1024)
    rows = int(min(seq, max(1024, 1024 * target_seconds / max(probe, 1e-6))))
    rows -= rows % 128 or 0
    # On a box with many cores a whole head takes less than the target: then several heads are timed in a row.
    heads = int(max(1, min(8, round(target_seconds / max(probe * rows / 1024, 1e-6))))) if rows >= seq - 127 else 1

    def sample():
        return sum(run(rows) for _ in range(heads))

    best = min(sample() for _ in range(repeats))
    flops = 4.0 * heads * rows * seq * HEAD_DIM
    return {"value": flops / best / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{heads} head(s) x {rows} query rows x {seq} keys, fp32 on bf16-rounded values, {best:.2f} s"}, best, flops


WORKLOAD = "wan2.1-14b-720p dense self-attention, B1 N40 S75600 D128 (21x45x80 latent grid)"


def use_all_host_cores():
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs are meant to use the cores the
    process may run on."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    return torch.get_num_threads()


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_all_host_cores()
    seq = 75600
    times, flops = [], 0.0
    info = None
    for i in range(args.warmup + args.steps):
        info, t, flops = cpu_attention_sample(seq, target_seconds=6.0)
        if i >= args.warmup:
            times.append(t)
    value = flops * len(times) / sum(times) / 1e12
    info["value"] = value
    line = {
        "impl": "reference", "metric": "attention_dense_equiv_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * 75600.0 * 75600 * 40 * 4 * HEAD_DIM / (value * 1e12),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "note": "CPU oracle (the reference's unfused torch formula) on the host cores; each step is a "
                           "bounded sample; ms_per_step is the full layer extrapolated by FLOPs"},
        "cpu_baseline": info,
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# GPU workloads
# ---------------------------------------------------------------------------------------------------
def ulysses_parity(q_full, k_full, v_full, step_out, rank, world, heads_checked):
    """The sequence-parallel result against the single-GPU kernel on the same seeded tensors: this rank
    runs the dense kernel on whole heads of the UNSHARDED q, k, v (it generated them) and requires its
    rows of those heads to be bit-equal in the Ulysses output.  Same kernel, same tiles, same order of
    key blocks: any difference is an error of the exchange."""
    from mindiesd import _cabi
    s_loc = q_full.shape[1] // world
    rows = slice(rank * s_loc, (rank + 1) * s_loc)
    equal = True
    for h in heads_checked:
        want = _cabi.attention(q_full[:, :, h:h + 1], k_full[:, :, h:h + 1], v_full[:, :, h:h + 1], head_first=False)
        equal = equal and torch.equal(step_out[:, :, h], want[:, rows, 0])
    return equal


def dense_or_ulysses(args, rank, world, device):
    import workloads
    from mindiesd import _cabi, ulysses_attention
    import torch.distributed as dist

    cfg = workloads.C3
    if args.heads:  # reduced head count: only for short profiler captures, named in the output
        cfg = workloads.Config(cfg.name, cfg.batch, args.heads, cfg.grid, cfg.seq, cfg.dtype)
    q, k, v = workloads.make_qkv(cfg, device, seed=0, layout="BSND")  # [1, S, 40, 128]
    s_loc = cfg.seq // world
    barrier = (lambda: dist.barrier()) if world > 1 else None
    parity = None
    pieces = None
    if world > 1:
        from mindiesd.parallel import default_head_pieces, default_transport
        if args.ulysses_transport is None:
            args.ulysses_transport = default_transport(device=device)  # what the library picks on this group
        if args.ulysses_pieces:
            pieces = [int(x) for x in args.ulysses_pieces.split(",")]
        elif args.ulysses_chunks:
            pieces = [cfg.heads // world // args.ulysses_chunks] * args.ulysses_chunks
        else:
            pieces = default_head_pieces(cfg.heads // world, cfg.seq)
        qs, ks, vs = (x[:, rank * s_loc:(rank + 1) * s_loc].contiguous() for x in (q, k, v))
        checked = sorted({0, cfg.heads // 2 + 1, cfg.heads - 1})  # heads of the first, a middle and the last rank
        ok = ulysses_parity(q, k, v, ulysses_attention(qs, ks, vs, head_chunks=pieces, transport=args.ulysses_transport),
                            rank, world, checked)
        flag = torch.tensor([1 if ok else 0], device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        parity = {"heads": checked, "equal": bool(flag.item()), "against": "single-GPU kernel on the unsharded tensors, torch.equal, every rank"}
        if not parity["equal"]:
            raise SystemExit(f"rank {rank}: the sequence-parallel output differs from the single-GPU kernel")
        del q, k, v
        q, k, v = qs, ks, vs
    torch.cuda.empty_cache()
    launches_per_layer = 1 if world == 1 else 3 * len(pieces)
    if world == 1:
        out = torch.empty_like(q)
        layer = lambda: _cabi.attention(q, k, v, head_first=False, out=out)  # noqa: E731
    else:
        layer = lambda: ulysses_attention(q, k, v, head_chunks=pieces, transport=args.ulysses_transport)  # noqa: E731

    # The timed region should last about two seconds at every GPU count, so that every N runs in the
    # same power state (a short region finishes before the power cap engages): a step repeats the
    # layer `layers` times.
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    layer()
    torch.cuda.synchronize()
    e0.record()
    layer()
    e1.record()
    torch.cuda.synchronize()
    probe = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(probe, op=dist.ReduceOp.MAX)
    layers = 1 if args.layers_per_step == 0 and world == 1 else (
        args.layers_per_step or max(1, round(2000.0 / (probe.item() * args.steps))))

    def step():
        for _ in range(layers):
            layer()

    sampler = ClockSampler(physical_gpu_index(device.index))
    sampler.start()
    ms = timed(step, args.steps, args.warmup, barrier)
    clocks = sampler.stop()

    phases = None
    if world > 1:  # one more, untimed, call with CUDA events around each phase
        prof = {}
        ulysses_attention(q, k, v, head_chunks=pieces, profile=prof, transport=args.ulysses_transport)
        t = torch.tensor([prof.get(n, 0.0) for n in ("pack", "exchange_in", "attention", "exchange_out", "unpack")],
                         dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        phases = dict(zip(("pack_ms", "exchange_in_ms", "attention_ms", "exchange_out_ms", "unpack_ms"),
                          (round(x, 4) for x in t.tolist())))
        # What the layer would cost if only this rank's attention ran: the same kernel on this rank's heads of
        # the full sequence, repeated like the layer so that it runs in the same power state.  The difference
        # to the timed layer is what the exchange costs after all overlap.
        aq, ak, av = workloads.make_qkv(cfg, device, seed=1, heads=cfg.heads // world, layout="BSND")
        ao = torch.empty_like(aq)

        def alone():
            for _ in range(layers):
                _cabi.attention(aq, ak, av, head_first=False, out=ao)

        alone_steps = max(2, args.steps // 2)
        a = torch.tensor([timed(alone, alone_steps, 1, barrier) / (alone_steps * layers)], dtype=torch.float64, device=device)
        dist.all_reduce(a, op=dist.ReduceOp.MAX)
        phases["attention_alone_ms"] = round(a.item(), 4)
        del aq, ak, av, ao

    # End to end through the public Python API with host buffers: every step copies this rank's
    # q, k, v from pinned host memory and reads its output back, copies pipelined with the kernels.
    from mindiesd import attention_forward_host
    from mindiesd.layers.flash_attn.host_io import default_host_chunks
    e2e_chunks = None
    if world == 1:
        hq, hk, hv = (torch.empty(x.transpose(1, 2).shape, dtype=x.dtype, pin_memory=True).copy_(x.transpose(1, 2))
                      for x in (q, k, v))  # head-first pinned copies
        e2e_chunks = args.e2e_chunks if args.e2e_chunks and cfg.heads % args.e2e_chunks == 0 else default_host_chunks(cfg.heads, cfg.seq)
    else:
        hq, hk, hv = (torch.empty(x.shape, dtype=x.dtype, pin_memory=True).copy_(x) for x in (q, k, v))
    ho = torch.empty(hq.shape, dtype=q.dtype, pin_memory=True)

    def e2e_step():
        if world == 1:
            attention_forward_host(hq, hk, hv, out=ho, head_chunks=e2e_chunks)
        else:
            from mindiesd.parallel import ulysses_attention_host
            # its own piece sizes unless they were given: the copies over PCIe want smaller pieces than NVLink does
            ulysses_attention_host(hq, hk, hv, out=ho,
                                   head_chunks=pieces if (args.ulysses_pieces or args.ulysses_chunks) else None)

    e2e_steps = max(1, args.steps)
    e2e_ms = timed(e2e_step, e2e_steps, 1, barrier) if not args.kernel_only else float("nan")

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    status = _cabi.device_status()
    if rank != 0:
        return None
    peaks = measured_peaks()
    ms_step = ms / args.steps
    ms_layer = ms_step / layers
    value = cfg.flops / (ms_layer * 1e-3) / 1e12
    config = {"workload": WORKLOAD if not args.heads else WORKLOAD.replace("N40", f"N{cfg.heads}") + " [heads reduced]",
              "layout": "BSND",
              "parallelism": "single GPU" if world == 1 else
              f"ulysses sp{world}, local heads in pieces of {pieces}, exchange over {args.ulysses_transport}",
              "layers_per_step": layers, "ms_per_layer": ms_layer, "flops_per_layer": cfg.flops,
              "l2": "operands (3.1 GB per layer) exceed L2; no flush",
              "tflops_per_gpu": value / world, "kernel_status": status}
    if clocks.get("sm_mhz"):
        # time x clock: what the layer costs in SM cycles, comparable across runs at different power states
        config["ms_per_layer_x_sm_mhz"] = ms_layer * clocks["sm_mhz"]
    if parity is not None:
        config["parity"] = parity
    if phases is not None:
        exposed = max(0.0, ms_layer - phases["attention_alone_ms"])
        config["phases_of_one_layer"] = dict(phases, exposed_ms=round(exposed, 4),
                                             note="pack .. unpack: CUDA events of one untimed layer, summed over its "
                                                  "pieces (spans on different streams overlap), max over ranks; "
                                                  "attention_alone: this rank's heads through the kernel with nothing "
                                                  "else running, timed like the layer; exposed = timed ms per layer "
                                                  "minus attention_alone")
    line = {
        "metric": "attention_dense_equiv_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": config,
        "clocks": clocks,
        "e2e": {"value": cfg.flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": 3 * q.numel() * q.element_size() * world,
                "d2h_bytes_per_step": q.numel() * q.element_size() * world,
                "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
                "api": f"mindiesd.attention_forward_host ({e2e_chunks} head chunks, copies overlapped)" if world == 1
                       else "mindiesd.parallel.ulysses_attention_host (copies pipelined piece by piece)"},
        "gpu_launches": launches_per_layer * layers * args.steps,
    }
    if world == 1:
        peak = peaks["bf16_tflops_sustained"]
        line["roofline"] = {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TFLOP/s", "frac": value / peak,
                            "traffic": DENSE_DRAM_TRAFFIC_BYTES, "peak_source": peaks["source"] + " cuBLAS bf16, sustained",
                            "frac_of_burst": value / peaks["bf16_tflops"], "frac_of_nominal_2250": value / 2250.0,
                            "kernel": "fa_fwd_kernel<bf16>", "flops_per_launch": cfg.flops}
        if not args.kernel_only:
            use_all_host_cores()
            cpu, _, _ = cpu_attention_sample(cfg.seq, target_seconds=16.0)
            line["cpu_baseline"] = cpu
            if not args.no_secondary:
                del q, k, v, out, hq, hk, hv, ho
                torch.cuda.empty_cache()
                line["config"]["secondary"] = secondary_lines(args, device, value, clocks)
    return line


def secondary_lines(args, device, dense_value, dense_clocks):
    """The sparse and FP8 workloads of the same shape, measured in the same run as the headline, so that
    their ratios to the dense kernel are taken on one GPU in one power state."""
    res = {}
    for name in ("sparse", "fp8"):
        sub = argparse.Namespace(**vars(args))
        sub.workload, sub.steps, sub.warmup, sub.heads = name, max(3, min(args.steps, 10)), 3, 0
        line = single_gpu_workload(sub, device)
        entry = {"ms_per_step": line["ms_per_step"], "dense_equiv_tflops": line["value"], "clocks": line["clocks"],
                 "speedup_over_dense": line["value"] / dense_value}
        sm, dsm = line["clocks"].get("sm_mhz"), dense_clocks.get("sm_mhz")
        if sm and dsm:
            # at equal clocks: ratio of (time x median SM MHz)
            entry["speedup_over_dense_at_equal_clocks"] = (line["value"] / sm) / (dense_value / dsm)
        for key in ("block_density", "executed_tflop", "sparsity_arg", "cosine_vs_bf16_kernel_heads_0_1"):
            if key in line["config"]:
                entry[key] = line["config"][key]
        entry["roofline_frac"] = line["roofline"]["frac"]
        res[name] = entry
        torch.cuda.empty_cache()
    return res


def single_gpu_workload(args, device):
    """Secondary kernels of the path at the benchmark shape; each prints the same kind of line."""
    import workloads
    from mindiesd import _cabi
    cfg = workloads.C3
    peaks = measured_peaks()
    name = args.workload
    src = workloads.C4 if name in ("fp8", "fp8_layer", "quant", "rotate_quant") else (workloads.C2 if name == "c2" else cfg)
    if args.heads:
        cfg = workloads.Config(cfg.name, cfg.batch, args.heads, cfg.grid, cfg.seq, cfg.dtype)
    q, k, v = workloads.make_qkv(src, device, seed=0, heads=args.heads or None)
    launches, bound, extra = 1, "tensor", {}
    if name == "c2":
        cfg = workloads.C2
        out = torch.empty_like(q)
        step = lambda: _cabi.attention(q, k, v, out=out)  # noqa: E731
        work, unit = cfg.flops, "TFLOP/s"
        label = "wan2.1-1.3b dense self-attention, B1 N12 S32760 D128, 3-D RoPE on q,k"
    elif name == "sparse":
        mask = _cabi.rf_block_mask(q, k, cfg.grid, 0, args.sparsity, True, temporal_band=args.band)
        qr, kr, vr = (_cabi.rf_rearrange(x, cfg.grid, 0, True) for x in (q, k, v))
        del q, k, v
        out = torch.empty_like(qr)
        step = lambda: _cabi.attention(qr, kr, vr, block_mask=mask, out=out)  # noqa: E731
        density = mask.float().mean().item()
        work, unit = cfg.flops, "TFLOP/s"
        extra = {"block_density": density, "sparsity_arg": args.sparsity, "temporal_band": args.band,
                 "executed_tflop": cfg.flops * density / 1e12}
        label = "RainFusion block-sparse attention (mask prebuilt, tokens pre-permuted), B1 N40 S75600 D128"
    elif name == "sparse_layer":
        # The whole RainFusion layer through the public API, every step: mask builder, three
        # permutations, block-sparse attention, inverse permutation.
        from mindiesd import sparse_attention
        step = lambda: sparse_attention(q, k, v, head_num=cfg.heads, input_layout="BNSD", sparse_type="rf_v3",  # noqa: E731
                                        block_size=128, latent_shape_q=cfg.grid, latent_shape_k=cfg.grid,
                                        sparsity=args.sparsity)
        work, unit, launches = cfg.flops, "TFLOP/s", 7
        label = ("RainFusion layer via mindiesd.sparse_attention(rf_v3): mask + permute + sparse attention + inverse, "
                 "B1 N40 S75600 D128")
        extra = {"sparsity_arg": args.sparsity}
    elif name == "fp8_layer":
        # The whole FP8 layer through the public hook: rotate + quantise q, k, v, then FP8 attention.
        from mindiesd import FP8RotateQuantFA
        hook = FP8RotateQuantFA(v_per_channel=True).to(device)
        step = lambda: hook(q, k, v, layout="BNSD")  # noqa: E731
        work, unit, launches = cfg.flops, "TFLOP/s", 6
        label = "FP8 layer via mindiesd.FP8RotateQuantFA: Hadamard + e4m3 quantisation of q, k, v + FP8 attention, B1 N40 S75600 D128"
    elif name == "fp8":
        q8, qs = _cabi.fa_block_quant(q, 128, rotate=True)
        k8, ks = _cabi.fa_block_quant(k, 128, rotate=True)
        v8, vs = _cabi.fa_block_quant(v, per_channel=True)
        # what quantisation costs in accuracy, on the first two heads: cosine between the FP8 output and the
        # bf16 kernel's output on the unquantised operands (flattened over rows and channels, per head)
        want = _cabi.attention(q[:, :2], k[:, :2], v[:, :2]).float()
        del q, k, v
        out = torch.empty(q8.shape, dtype=torch.bfloat16, device=device)
        step = lambda: _cabi.attention(q8, k8, v8, q_scale=qs, k_scale=ks, v_scale=vs, k_scale_block=128,  # noqa: E731
                                       v_scale_block=0, out=out)
        step()
        got = out[:, :2].float()
        cos = torch.nn.functional.cosine_similarity(got.flatten(2), want.flatten(2), dim=-1)
        extra = {"cosine_vs_bf16_kernel_heads_0_1": [round(x, 6) for x in cos.flatten().tolist()]}
        del want, got
        work, unit = cfg.flops, "TFLOP/s"
        label = "FP8-e4m3 attention (operands pre-quantised), B1 N40 S75600 D128"
    elif name == "mask":
        scratch = torch.empty(_cabi.lib().mindiesd_rf_block_mask_scratch_bytes(1, cfg.heads, cfg.seq, HEAD_DIM),
                              dtype=torch.uint8, device=device)
        step = lambda: _cabi.rf_block_mask(q, k, cfg.grid, 0, 0.75, True, scratch=scratch)  # noqa: E731
        work = 2.0 * q.numel() * 2 + cfg.heads * 591 * 591  # read q and k once, write the int8 mask
        unit, bound, launches = "GB/s", "hbm", 2
        label = "RainFusion mask builder (pool + mask kernels), B1 N40 S75600 D128, sparsity 0.75"
    elif name == "quant":
        step = lambda: _cabi.fa_block_quant(q, 128, rotate=True)  # noqa: E731
        work = q.numel() * 3.0  # 2 bytes in, 1 byte out per element
        unit, bound = "GB/s", "hbm"
        label = "e4m3 block quantisation with Hadamard rotation of one operand, B1 N40 S75600 D128"
    elif name == "estimate":
        # The ada_bsa mask builder: a K = 1024 contraction per pair of 8-token groups on the tensor cores,
        # softmax and 16 x 16 block sums, then the cumulative-mass decision.
        scratch = torch.empty(_cabi.lib().mindiesd_sparse_block_estimate_scratch_bytes(1, cfg.heads, cfg.seq),
                              dtype=torch.uint8, device=device)
        step = lambda: _cabi.sparse_block_estimate(q, k, HEAD_DIM ** -0.5 / 8, args.cdf, 1.0 - args.sparsity,  # noqa: E731
                                                   scratch=scratch)
        groups = cfg.seq // 8
        work, unit = 2.0 * cfg.heads * groups * groups * 8 * HEAD_DIM, "TFLOP/s"
        launches = 2 * ((cfg.heads + 3) // 4)
        label = f"ada_bsa sparse block estimate, B1 N{cfg.heads} S75600 D128, cdf threshold {args.cdf}"
        extra = {"flops_per_step": work, "metric_note": "TFLOP/s of the estimator's own contraction, not dense-equivalent"}
    elif name == "ada_layer":
        from mindiesd import sparse_attention
        step = lambda: sparse_attention(q, k, v, head_num=cfg.heads, input_layout="BNSD", sparse_type="ada_bsa",  # noqa: E731
                                        block_size=128, cdf_threshold=args.cdf, sparsity=args.sparsity)
        work, unit, launches = cfg.flops, "TFLOP/s", 2 * ((cfg.heads + 3) // 4) + 1
        from mindiesd.layers.flash_attn.sparse_flash_attn_ada_bsa import get_estimate_mask
        smask, _ = get_estimate_mask(q, k, v, scale=HEAD_DIM ** -0.5, head_num=cfg.heads, sparsity=args.sparsity,
                                     cdf_threshold=args.cdf)
        extra = {"block_density": smask[..., :591].float().mean().item(), "cdf_threshold": args.cdf,
                 "sparsity_arg": args.sparsity}
        del smask
        label = ("ada_bsa layer via mindiesd.sparse_attention(ada_bsa): block estimate + block-sparse attention, "
                 "B1 N40 S75600 D128")
    elif name == "rotate_quant":
        rot = torch.linalg.qr(torch.randn(128, 128, device=device, dtype=torch.float64))[0].to(q.dtype)
        step = lambda: _cabi.fa_rotate_quant(q, rot, 128)  # noqa: E731
        work = q.numel() * 3.0
        unit, bound = "GB/s", "hbm"
        label = "learned 128x128 rotation fused with e4m3 block quantisation of one operand, B1 N40 S75600 D128"
    elif name == "rearrange":
        step = lambda: _cabi.rf_rearrange(q, cfg.grid, 0, True)  # noqa: E731
        work = q.numel() * 4.0
        unit, bound = "GB/s", "hbm"
        label = "RainFusion window permutation of one operand, B1 N40 S75600 D128"
    elif name in ("ulysses_move", "ulysses_move_rope"):
        # The re-shard kernel of the sequence-parallel layer on one GPU at the 8-GPU shape: this rank's
        # 9450 token rows of q, k, v, a piece of 3 local heads packed for 8 destinations (all local here).
        del q, k, v
        world, rows, piece = 8, cfg.seq // 8, 3
        g = torch.Generator(device=device).manual_seed(0)
        q, k, v = (torch.randn(rows, cfg.heads, HEAD_DIM, device=device, dtype=torch.bfloat16, generator=g) for _ in range(3))
        send = torch.empty(world, rows, 3 * piece, HEAD_DIM, device=device, dtype=torch.bfloat16)
        ptrs = [send[r].data_ptr() for r in range(world)]
        kw = {}
        if name == "ulysses_move_rope":
            cos, sin = (torch.randn(rows, HEAD_DIM, device=device, generator=g) for _ in range(2))
            kw = dict(cos=cos, sin=sin, rope_mode=1)
        step = lambda: _cabi.ulysses_move((q, k, v), ptrs, send.stride(1), rows, world, cfg.heads // world, 0, piece, **kw)  # noqa: E731
        work = 2.0 * send.numel() * 2  # every packed element is read once and written once
        unit, bound = "GB/s", "hbm"
        label = ("Ulysses re-shard kernel, one piece of 3 local heads of q, k, v for 8 destinations, 9450 rows x 40 heads x 128"
                 + (", rotary embedding applied on the way" if kw else "") + "; 174 MB per launch, partly L2-resident between launches")
    else:
        raise SystemExit(f"unknown workload {name}")
    sampler = ClockSampler(physical_gpu_index(device.index))
    sampler.start()
    ms = timed(step, args.steps, args.warmup)
    clocks = sampler.stop()
    ms_step = ms / args.steps
    value = work / (ms_step * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    peak = peaks["bf16_tflops_sustained"] if bound == "tensor" else peaks["hbm_gbs"]
    # The roofline fraction is of the work actually executed: a block-sparse launch is measured by the
    # blocks it walks, not by the dense-equivalent figure of the metric.
    achieved = value * extra["executed_tflop"] * 1e12 / work if "executed_tflop" in extra else value
    return {
        "metric": "attention_dense_equiv_tflops" if unit == "TFLOP/s" else "achieved_hbm_gbs", "value": value,
        "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "e4m3" if name in ("fp8", "fp8_layer") else "bf16", "data": "synthetic",
        "config": dict({"workload": label + (f" [heads reduced to {args.heads}]" if args.heads else ""), "l2": "operands exceed L2; no flush", "kernel_status": _cabi.device_status()}, **extra),
        "clocks": clocks,
        "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "traffic": None,
                     "peak_source": peaks["source"]},
        "gpu_launches": launches * args.steps,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="dense")
    ap.add_argument("--sparsity", type=float, default=0.75)
    ap.add_argument("--band", type=int, default=-1)
    ap.add_argument("--ulysses-chunks", type=int, default=0, help="head chunks per rank of the Ulysses leg (0: the API's default)")
    ap.add_argument("--ulysses-pieces", default=None, help="local heads per piece, e.g. 2,8,8,2 (default: library choice)")
    ap.add_argument("--ulysses-transport", default=None, choices=[None, "nccl", "peer"],
                    help="how the Ulysses leg exchanges data (default: the API's)")
    ap.add_argument("--e2e-chunks", type=int, default=0, help="head chunks of the pipelined end-to-end leg (0: the API's default)")
    ap.add_argument("--cdf", type=float, default=0.9, help="cumulative-mass threshold of the ada_bsa estimate")
    ap.add_argument("--heads", type=int, default=0, help="reduced head count for profiler captures (default: the full 40)")
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end and CPU legs (profiler captures)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the sparse and FP8 legs of the headline run")
    ap.add_argument("--layers-per-step", type=int, default=0,
                    help="layers one step repeats (0: one on a single GPU, else enough for a timed region of about 2 s)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU implementation")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    try:
        if args.workload == "dense" or world > 1:
            line = dense_or_ulysses(args, rank, world, device)
        else:
            line = single_gpu_workload(args, device)
        if rank == 0 and line is not None:
            print(json.dumps(line), flush=True)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
