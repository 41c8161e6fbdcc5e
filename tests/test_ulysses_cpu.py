"""Ulysses data movement on CPU ranks (gloo, world size 2 and 4): the wrapper's all-to-alls, head
chunking and packing must reproduce single-process attention over the full sequence.  The local
attention is the CPU oracle, injected through `attn_fn`; no GPU is involved."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, head_chunks, batch, result):
    for p in (ROOT, ROOT / "mindie-sd_b200", ROOT / "tests" / "golden"):
        sys.path.insert(0, str(p))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import inputs
        from oracle import attention as oa
        from oracle import ulysses as ou
        from mindiesd.parallel.ulysses import ulysses_attention
        torch.set_num_threads(1)
        n, s, d = 8, 64 * world, 16
        q, k, v = (inputs.randn(200 + i, batch, s, n, d) for i in range(3))
        shard = lambda x: x.chunk(world, dim=1)[rank].contiguous()  # noqa: E731
        calls = []

        def attn(qq, kk, vv, scale):
            calls.append(tuple(qq.shape))
            return oa.attention_math(qq, kk, vv, scale=scale, head_first=False)

        out = ulysses_attention(shard(q), shard(k), shard(v), scale=d ** -0.5, head_chunks=head_chunks, attn_fn=attn)
        want = oa.attention_math(q, k, v, scale=d ** -0.5, head_first=False)
        ok = torch.allclose(out, shard(want), atol=1e-5)
        sizes = [n // world // head_chunks] * head_chunks if isinstance(head_chunks, int) else list(head_chunks)
        ok = ok and [c[2] for c in calls] == sizes and calls[0] == (batch, s, sizes[0], d)
        # the re-shard itself against the single-process restatement
        shards = [x.contiguous() for x in q.chunk(world, dim=1)]
        full = ou.seq_to_head(shards)[rank]
        ok = ok and torch.equal(ou.head_to_seq(ou.seq_to_head(shards))[rank], shards[rank])
        ok = ok and full.shape == (batch, s, n // world, d)
        result[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,head_chunks,batch", [(2, 1, 1), (2, 4, 1), (4, 2, 1), (2, 2, 2), (2, (1, 3), 1)])
def test_ulysses_matches_single_process(world, head_chunks, batch):
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, head_chunks, batch, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    assert all(result.get(r) for r in range(world)), dict(result)


def test_ulysses_rejects_indivisible_heads():
    from mindiesd.utils.exception import ParametersInvalid
    from mindiesd.parallel.ulysses import ulysses_attention
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()))
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        q = torch.zeros(1, 8, 3, 16)
        out = ulysses_attention(q, q, q, attn_fn=lambda a, b, c, s: a)  # world size 1: straight through
        assert out.shape == q.shape
        with pytest.raises(ParametersInvalid):
            ulysses_attention(q, q[:, :4], q)
    finally:
        dist.destroy_process_group()


def test_default_head_pieces_keeps_pieces_large_and_the_first_small():
    from mindiesd.parallel import default_head_chunks, default_head_pieces
    # 75 600 tokens: 296 thread blocks per head, so a piece of twenty waves needs ten heads
    assert default_head_pieces(20, 75600) == [10, 10]         # 2 GPUs
    assert default_head_pieces(10, 75600) == [10]             # 4 GPUs: the exchange over NVLink is cheaper than a cut
    assert default_head_pieces(5, 75600) == [5]               # 8 GPUs
    assert default_head_pieces(20, 4096) == [20]              # short sequences: one piece
    assert default_head_pieces(12) == [1, 1, 1, 1, 2, 2, 2, 2]  # length unknown: at most eight pieces
    assert default_head_chunks(20, 75600) == 2 and default_head_chunks(20, 4096) == 1
    # the host-operand pipeline hides copies over PCIe: eight waves per piece, and two pieces where it can
    host = dict(waves=8, split_small=True)
    assert default_head_pieces(20, 75600, **host) == [4] * 5
    assert default_head_pieces(10, 75600, **host) == [5, 5]
    assert default_head_pieces(5, 75600, **host) == [2, 3]    # two uneven pieces, the smaller first
    assert default_head_pieces(3, 75600, **host) == [3]       # too few for two pieces of four waves
