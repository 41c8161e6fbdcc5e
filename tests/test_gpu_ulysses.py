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
        from mindiesd import _cabi, ulysses_attention
        n, s = 8, 3000 if world == 2 else 4096  # 3000 / 2 = 1500 rows per rank: ragged 128-row tiles
        q, k, v = (inputs.randn(400 + i, 1, s, n, 128, dtype=torch.bfloat16).cuda() for i in range(3))
        want = _cabi.attention(q, k, v, head_first=False)
        shard = lambda x: x.chunk(world, dim=1)[rank].contiguous()  # noqa: E731
        out = ulysses_attention(shard(q), shard(k), shard(v), head_chunks=head_chunks)
        torch.cuda.synchronize()
        # the same kernel on the same rows and heads: only the walk order of the heads differs
        ok = torch.equal(out, shard(want))
        ok = ok and _cabi.device_status() == 0
        result[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,head_chunks", [(2, 1), (2, 4), (4, 2)])
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
    assert all(result.get(r) for r in range(world)), dict(result)
