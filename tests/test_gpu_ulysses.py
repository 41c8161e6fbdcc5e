"""Ulysses sequence-parallel attention on real GPUs (needs at least 2): the gathered output of the
P-rank run must equal the single-GPU kernel's output on the same seeded tensors.  Ranks are child
processes over NCCL; each runs on its own device."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, head_chunks, result):
    for p in (ROOT, ROOT / "mindie-sd_b200", ROOT / "tests" / "golden"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import inputs
        from mindiesd import _cabi, rotary_position_embedding, ulysses_attention
        from mindiesd.parallel import ulysses_attention_host
        n, s = 8, 3000 if world == 2 else 4096  # 3000 / 2 = 1500 rows per rank: ragged 128-row tiles
        q, k, v = (inputs.randn(400 + i, 1, s, n, 128, dtype=torch.bfloat16).cuda() for i in range(3))
        want = _cabi.attention(q, k, v, head_first=False)
        shard = lambda x: x.chunk(world, dim=1)[rank].contiguous()  # noqa: E731
        checks = {}
        for rep in range(2):  # the second call reuses the persistent buffers
            out = ulysses_attention(shard(q), shard(k), shard(v), head_chunks=head_chunks, transport="nccl")
            torch.cuda.synchronize()
            # the same kernel on the same rows and heads: only the walk order of the heads differs
            checks[f"plain{rep}"] = torch.equal(out, shard(want))
        # rotary embedding inside the exchange == rotary_position_embedding, then attention, on one GPU
        cos, sin = (inputs.randn(410 + i, s, 128).cuda() for i in range(2))
        for mode in ("rotated_half", "rotated_interleaved"):
            qr, kr = (rotary_position_embedding(x, cos, sin, mode, head_first=False) for x in (q, k))
            want_r = _cabi.attention(qr, kr, v, head_first=False)
            cs, ss = (x.chunk(world, dim=0)[rank].contiguous() for x in (cos, sin))
            out_r = ulysses_attention(shard(q), shard(k), shard(v), head_chunks=head_chunks, rope=(cs, ss, mode),
                                      transport="nccl")
            checks[mode] = torch.equal(out_r, shard(want_r))
        # whatever transport the ranks agree on by default, and the library's own piece sizes
        from mindiesd.parallel import default_transport
        checks["default_transport_named"] = default_transport() in ("nccl", "peer")
        checks["default"] = torch.equal(ulysses_attention(shard(q), shard(k), shard(v)), shard(want))
        # operands in pinned host memory, copies pipelined with the pieces
        hq, hk, hv = (shard(x).cpu().pin_memory() for x in (q, k, v))
        for rep in range(2):
            ho = ulysses_attention_host(hq, hk, hv, head_chunks=head_chunks)
            checks[f"host{rep}"] = torch.equal(ho, shard(want).cpu())
        # the exchange over peer memory: the re-shard kernels store to / load from the other ranks' buffers
        for rep in range(2):
            out_p = ulysses_attention(shard(q), shard(k), shard(v), head_chunks=head_chunks, transport="peer")
            torch.cuda.synchronize()
            checks[f"peer{rep}"] = torch.equal(out_p, shard(want))
        cs, ss = (x.chunk(world, dim=0)[rank].contiguous() for x in (cos, sin))
        qr, kr = (rotary_position_embedding(x, cos, sin, "rotated_half", head_first=False) for x in (q, k))
        out_pr = ulysses_attention(shard(q), shard(k), shard(v), head_chunks=head_chunks, transport="peer",
                                   rope=(cs, ss, "rotated_half"))
        checks["peer_rope"] = torch.equal(out_pr, shard(_cabi.attention(qr, kr, v, head_first=False)))
        prof = {}
        ulysses_attention(shard(q), shard(k), shard(v), head_chunks=head_chunks, profile=prof)
        checks["profile"] = set(prof) == {"pack", "exchange_in", "attention", "exchange_out", "unpack"}
        checks["status"] = _cabi.device_status() == 0
        result[rank] = {k_: bool(v_) for k_, v_ in checks.items()}
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,head_chunks", [(2, 1), (2, 4), (2, (1, 3)), (4, 2)])
def test_ulysses_equals_single_gpu(world, head_chunks):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, head_chunks, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    for r in range(world):
        assert result.get(r) and all(result[r].values()), dict(result)


def test_reshard_kernel_on_one_gpu():
    """mindiesd_ulysses_move by itself (one GPU plays every rank): forward into a send buffer, with and without
    the rotary embedding, against torch indexing and the rotary oracle; the inverse restores the layout."""
    import inputs
    from oracle import rope as orope
    from mindiesd import _cabi
    world, rows, n, d = 4, 333, 8, 128
    n_loc, head0, h = n // world, 1, 1
    q, k, v = (inputs.randn(420 + i, rows, n, d, dtype=torch.bfloat16) for i in range(3))
    cos, sin = (inputs.randn(430 + i, rows, d) for i in range(2))
    for mode_name, mode in ((None, 0), ("rotated_half", 1), ("rotated_interleaved", 2)):
        send = torch.zeros(world, rows, 3 * h, d, dtype=torch.bfloat16, device="cuda")
        _cabi.ulysses_move((q.cuda(), k.cuda(), v.cuda()), [send[r].data_ptr() for r in range(world)], send.stride(1), rows,
                           world, n_loc, head0, h, cos=cos.cuda(), sin=sin.cuda(), rope_mode=mode, thread_blocks=7)
        for i, x in enumerate((q, k, v)):
            if mode and i < 2:
                x = orope.rotary_position_embedding(x[None], cos, sin, mode_name, head_first=False)[0]
            want = x.view(rows, world, n_loc, d)[:, :, head0:head0 + h].permute(1, 0, 2, 3)
            assert torch.equal(send[:, :, i * h:(i + 1) * h].cpu(), want), (mode_name, i)
    o_recv = inputs.randn(440, world, rows, h, d, dtype=torch.bfloat16).cuda()
    out = torch.zeros(rows, n, d, dtype=torch.bfloat16, device="cuda")
    _cabi.ulysses_move((out,), [o_recv[r].data_ptr() for r in range(world)], o_recv.stride(1), rows, world, n_loc, head0, h,
                       inverse=True)
    want = torch.zeros(rows, world, n_loc, d, dtype=torch.bfloat16)
    want[:, :, head0:head0 + h] = o_recv.cpu().permute(1, 0, 2, 3)
    assert torch.equal(out.cpu().view(rows, world, n_loc, d), want)
    assert _cabi.device_status() == 0
