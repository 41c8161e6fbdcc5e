"""Ulysses sequence-parallel attention: every rank holds a slice of the sequence with all heads,
an all-to-all turns that into the full sequence with a slice of the heads, attention runs locally,
and a second all-to-all turns the result back.

MindIE-SD documents this pattern (docs/zh/features/parallelism.md:207-233) without shipping it;
this is the same tensor contract -- BSND in, BSND out, `N % world_size == 0` -- built differently:

* The local heads are cut into pieces.  Per piece ONE kernel (`mindiesd_ulysses_move`) reads this
  rank's q, k and v in place and writes, for every destination rank, the block that rank needs in
  the layout its attention kernel reads -- optionally applying the rotary embedding to q and k on the
  way -- and ONE all-to-all carries q, k and v together.  For B = 1 the receive buffer already is
  `[S, 3h, D]`, which the attention kernel reads through strides; it writes its output straight into
  the send buffer of the return exchange, and one kernel scatters the returned blocks into the result.
* The exchange of piece c+1 runs on an inbound stream and the return of piece c-1, with the scatter into
  the caller's output, on an outbound stream, both under piece c's attention; the pieces' attention
  kernels alternate between the caller's stream and a second one, so that a piece's thread blocks fill
  the SMs the previous piece's last wave leaves idle.  Pieces may be uneven (5 local heads -> 2 + 3), so
  that overlap exists at every world size.
* Send and receive buffers are allocated once per (shape, dtype, group) and reused by every call.
* transport="peer": the ranks map each other's receive buffers (CUDA IPC) once, and then the re-shard
  kernel IS the all-to-all: it stores each destination's block straight into that rank's receive
  buffer over NVLink, and after attention every rank's scatter kernel loads the blocks it needs straight
  from its peers' output buffers.  No send buffers, no NCCL data movement: the only collective left is a
  one-element all-reduce per piece that orders the ranks.  It is the default where the ranks of the group
  share a host and can map each other's memory; transport="nccl" (otherwise, and for B > 1 or a custom
  attention function) packs into a send buffer and calls all_to_all_single.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence, Union

import torch
import torch.distributed as dist

from ..utils.exception import ParametersInvalid
from ..utils.status import raise_if_kernel_gave_up

_ROPE_MODES = {"rotated_half": 1, "rotated_interleaved": 2}


def _default_attention(q, k, v, scale, out=None):
    # BSND views with a non-unit head-group stride: the kernel reads them through strides.
    if out is not None and q.is_cuda:
        from .. import _cabi
        return _cabi.attention(q, k, v, head_first=False, scale=scale, out=out)
    return torch.ops.mindiesd.attention_fwd(q, k, v, float(scale), False)


_COMM_STREAMS = {}
_BUFFERS = {}


def _side_streams(device):
    """(inbound, outbound, second compute) streams of a device.  Inbound carries the re-shard kernels and the
    exchange towards the attention, outbound the exchange back and the scatter into the caller's output, both
    at high priority; the second compute stream takes every other piece's attention kernel, so that a piece's
    thread blocks fill the SMs the previous piece's last wave leaves idle."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = (torch.cuda.Stream(device=device, priority=-1), torch.cuda.Stream(device=device, priority=-1),
                              torch.cuda.Stream(device=device))
    return _COMM_STREAMS[key]


def _buffers(key, shapes, dtype, device):
    """Persistent send/receive buffers of one call signature.  Allocating them per call makes the
    caching allocator grow and synchronise in the middle of the overlapped pipeline."""
    cached = _BUFFERS.get(key)
    if cached is None:
        if len(_BUFFERS) >= 4:  # a handful of shapes per process; older ones go back to the allocator
            _BUFFERS.pop(next(iter(_BUFFERS)))
        cached = [torch.empty(s, dtype=dtype, device=device) for s in shapes]
        _BUFFERS[key] = cached
    return cached


def release_buffers():
    """Frees the persistent exchange buffers (they are re-created by the next call)."""
    _BUFFERS.clear()
    _PEER_BUFFERS.clear()


_PEER_BUFFERS = {}


class _PeerBuffers:
    """Receive and output buffers of one call signature, mapped into every rank of the group.
    local[i] is this rank's buffer i; peer_ptr[r][i] the address, in THIS process, of the same buffer of
    rank r (for r == rank the local one).  The mapping goes through CUDA IPC handles exchanged once."""

    def __init__(self, shapes, dtype, device, group):
        from .. import _cabi
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.local = [torch.empty(s, dtype=dtype, device=device) for s in shapes]
        handles = [_cabi.peer_export(t) for t in self.local]
        gathered = [None] * world
        dist.all_gather_object(gathered, handles, group=group)
        with torch.cuda.device(device):
            self.peer_ptr = [[t.data_ptr() for t in self.local] if r == rank else
                             [_cabi.peer_open(h, off) for h, off in gathered[r]] for r in range(world)]
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        dist.barrier(group=group)  # nobody proceeds (or frees) before everyone has mapped


def _peer_buffers(key, shapes, dtype, device, group):
    cached = _PEER_BUFFERS.get(key)
    if cached is None:
        if len(_PEER_BUFFERS) >= 4:
            _PEER_BUFFERS.pop(next(iter(_PEER_BUFFERS)))
        cached = _PeerBuffers(shapes, dtype, device, group)
        _PEER_BUFFERS[key] = cached
    return cached


_TRANSPORT_CHOICE = {}


def _default_transport(device, group, peer_capable_call: bool) -> str:
    """"peer" where this call can use it and every rank of the group sits in one process group of one host
    whose GPUs can map each other's memory; else "nccl".  MINDIESD_ULYSSES_TRANSPORT overrides.  The ranks
    decide together, once per (device, group): each gathers every rank's host name and device index, checks peer
    access from its own device, and the choice is "peer" only if every rank's check passed."""
    import os
    import socket
    forced = os.environ.get("MINDIESD_ULYSSES_TRANSPORT")
    if forced:
        return forced
    if not peer_capable_call:
        return "nccl"
    key = (device.index, id(group))
    if key not in _TRANSPORT_CHOICE:
        world = dist.get_world_size(group)
        mine = (socket.gethostname(), device.index if device.index is not None else torch.cuda.current_device(),
                torch.cuda.device_count())
        seen = [None] * world
        dist.all_gather_object(seen, mine, group=group)
        ok = (len({h for h, _, _ in seen}) == 1 and len({i for _, i, _ in seen}) == world
              and all(n == mine[2] and i < n for _, i, n in seen)
              and all(i == mine[1] or torch.cuda.can_device_access_peer(mine[1], i) for _, i, _ in seen))
        votes = [None] * world
        dist.all_gather_object(votes, bool(ok), group=group)
        _TRANSPORT_CHOICE[key] = "peer" if all(votes) else "nccl"
    return _TRANSPORT_CHOICE[key]


def default_transport(group=None, device=None) -> str:
    """The transport `ulysses_attention(transport=None)` uses on this group for B = 1 CUDA operands and the
    default attention kernel.  Collective: every rank of the group calls it."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    return _default_transport(device, group, True)


def default_head_pieces(local_heads: int, seq: int = 1 << 30, batch: int = 1, limit: int = 8, waves: int = 20,
                        split_small: bool = False):
    """Sizes of the pieces the local heads are cut into.  A piece keeps at least `waves` waves of attention
    thread blocks (one block per 256 query rows of a head, 148 SMs).  Over NVLink the exchange of a whole
    rank's heads costs a few hundred microseconds, less than what every further piece loses to its partial
    last wave and to the exchange kernels that take SMs beside it, so pieces are large.  Measured at 75 600
    tokens, per layer, peer transport: 2 GPUs [10, 10] 51.8 ms, [6, 7, 7] 52.1 ms, [4] * 5 52.5 ms; 4 GPUs [10]
    26.1 ms, [5, 5] 26.4 ms; 8 GPUs [5] 13.1 ms, [2, 3] 13.6 ms.  20 waves give 20 heads -> [10, 10],
    10 -> [10], 5 -> [5].
    `split_small` cuts fewer heads than two such pieces in two anyway, the smaller first, where that leaves at
    least half a piece each: the host-operand pipeline uses it with `waves=8`, because there the copies over
    PCIe are what has to be hidden (20 heads -> [4] * 5, 10 -> [5, 5], 5 -> [2, 3])."""
    blocks_per_head = batch * ((seq + 255) // 256)
    min_heads = max(1, -(-waves * 148 // blocks_per_head))
    pieces = max(1, min(limit, local_heads // min_heads))
    if split_small and pieces == 1 and local_heads >= 2 * max(1, -(-min_heads // 2)) and local_heads > 1:
        pieces = 2
    base, extra = divmod(local_heads, pieces)
    return [base] * (pieces - extra) + [base + 1] * extra


def default_head_chunks(local_heads: int, seq: int = 1 << 30, batch: int = 1, limit: int = 8) -> int:
    """Number of pieces `default_head_pieces` cuts the local heads into."""
    return len(default_head_pieces(local_heads, seq, batch, limit))


def _piece_sizes(head_chunks, n_loc, seq, batch):
    if head_chunks is None:
        return default_head_pieces(n_loc, seq, batch)
    if isinstance(head_chunks, int):
        if head_chunks < 1 or n_loc % head_chunks:
            raise ParametersInvalid(f"head_chunks={head_chunks} must divide the {n_loc} local heads.")
        return [n_loc // head_chunks] * head_chunks
    sizes = [int(x) for x in head_chunks]
    if not sizes or min(sizes) < 1 or sum(sizes) != n_loc:
        raise ParametersInvalid(f"head_chunks={sizes} must be positive piece sizes adding up to the {n_loc} local heads.")
    return sizes


class _Timer:
    """CUDA-event stopwatch of the phases of one call; inert unless a `profile` dict was passed."""

    def __init__(self, profile, cuda):
        self.on = profile is not None and cuda
        self.profile = profile
        self.spans = []

    def span(self, name, stream):
        return _Span(self, name, stream) if self.on else _NULL

    def finish(self):
        if not self.on:
            return
        torch.cuda.synchronize()
        for name, e0, e1 in self.spans:
            self.profile[name] = self.profile.get(name, 0.0) + e0.elapsed_time(e1)


class _Span:
    def __init__(self, timer, name, stream):
        self.timer, self.name, self.stream = timer, name, stream

    def __enter__(self):
        self.e0 = torch.cuda.Event(enable_timing=True)
        self.e0.record(self.stream)

    def __exit__(self, *exc):
        e1 = torch.cuda.Event(enable_timing=True)
        e1.record(self.stream)
        self.timer.spans.append((self.name, self.e0, e1))
        return False


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NULL = _Null()


def _move(tensors, table, rows, world, n_loc, head0, heads, inverse=False, rope=None, thread_blocks=0):
    """mindiesd_ulysses_move on CUDA tensors.  `tensors`: [rows, N, D] views; `table`: [P, rows, k*heads, D]
    buffer whose chunk r is rank r's side.  Host tensors (the gloo tests of the host logic) take the
    same movement as torch indexing."""
    t0 = tensors[0]
    if t0.is_cuda:
        from .. import _cabi
        ptrs = [table[r].data_ptr() for r in range(world)]
        cos = sin = None
        mode = 0
        if rope is not None and not inverse:
            cos, sin, mode = rope
        _cabi.ulysses_move(tensors, ptrs, table.stride(1), rows, world, n_loc, head0, heads, inverse=inverse,
                           cos=cos, sin=sin, rope_mode=mode, thread_blocks=thread_blocks)
        return
    if rope is not None:
        raise ParametersInvalid("The rotary embedding inside the exchange needs CUDA tensors.")
    d = t0.shape[-1]
    if not inverse:
        for i, t in enumerate(tensors):
            src = t.reshape(rows, world, n_loc, d)[:, :, head0:head0 + heads]  # [rows, P, heads, D]
            table[:, :, i * heads:(i + 1) * heads].copy_(src.permute(1, 0, 2, 3))
    else:
        dst = t0.reshape(rows, world, n_loc, d)[:, :, head0:head0 + heads]
        dst.copy_(table.permute(1, 0, 2, 3))


def ulysses_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, group=None,
                      scale: Optional[float] = None, head_chunks: Union[None, int, Sequence[int]] = None,
                      attn_fn: Optional[Callable] = None, rope=None, profile: Optional[dict] = None,
                      transport: Optional[str] = None, _piece_ready: Optional[Callable] = None, _piece_done: Optional[Callable] = None,
                      _out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """query/key/value: this rank's [B, S/P, N, D] slice (BSND).  Returns this rank's [B, S/P, N, D]
    slice of the attention output over the full sequence.

    head_chunks: how the N/P local heads are cut into pieces for overlap: a count (equal pieces), a list of
    piece sizes, or None for `default_head_pieces`.
    attn_fn(q, k, v, scale) -> out on [B, S, h, D] BSND tensors replaces the local attention (sparse or
    FP8 variants); the default is the dense kernel.
    rope: (cos, sin, rotated_mode) -- fp32 tables [S/P, D] for this rank's tokens and "rotated_half" or
    "rotated_interleaved": q and k are rotated as `rotary_position_embedding` would, inside the kernel that
    re-shards them, so the rotated tensors are never written on this rank.
    transport: "nccl" (pack, all_to_all_single, unpack), "peer" (the re-shard kernels store to and load from
    the peers' buffers over NVLink; CUDA tensors, B = 1, default attention), or None: the environment variable
    MINDIESD_ULYSSES_TRANSPORT, else "peer" where the call and the group allow it (one host, every GPU can map
    the others' memory; the ranks decide together), else "nccl".
    profile: a dict that receives the summed CUDA-event milliseconds of the phases of this call
    ("pack", "exchange_in", "attention", "exchange_out", "unpack"); it synchronises the device.
    """
    if query.dim() != 4 or key.shape != query.shape or value.shape != query.shape:
        raise ParametersInvalid("ulysses_attention expects q, k, v of one shape [B, S/P, N, D].")
    world = dist.get_world_size(group)
    b, s_loc, n, d = query.shape
    if n % world:
        raise ParametersInvalid(f"The head number {n} must be divisible by the sequence-parallel size {world}.")
    if scale is None:
        scale = d ** -0.5
    rope_args = None
    if rope is not None:
        cos, sin, mode = rope
        if mode not in _ROPE_MODES:
            raise ParametersInvalid(f"Unsupported rotated_mode: {mode}.")
        if cos.shape != (b * s_loc, d) and cos.shape != (s_loc, d) or sin.shape != cos.shape or cos.dtype != torch.float32:
            raise ParametersInvalid("rope tables must be fp32 [S/P, D] for this rank's tokens.")
        if b > 1 and cos.shape[0] == s_loc:
            cos, sin = cos.repeat(b, 1), sin.repeat(b, 1)
        rope_args = (cos.contiguous(), sin.contiguous(), _ROPE_MODES[mode])
    if world == 1:
        if rope_args is not None:
            from ..layers.rope import rotary_position_embedding
            query, key = (rotary_position_embedding(x, rope[0], rope[1], rope[2], head_first=False) for x in (query, key))
        return attn_fn(query, key, value, scale) if attn_fn else _default_attention(query, key, value, scale)
    n_loc = n // world
    sizes = _piece_sizes(head_chunks, n_loc, s_loc * world, b)
    cuda = query.is_cuda
    device = query.device
    q, k, v = (x if x.is_contiguous() else x.contiguous() for x in (query, key, value))
    rows = b * s_loc
    qr, kr, vr = (x.view(rows, n, d) for x in (q, k, v))
    out = _out if _out is not None else torch.empty_like(q)
    outr = out.view(rows, n, d)

    if transport is None:
        transport = _default_transport(device, group, cuda and b == 1 and attn_fn is None)
    if transport not in ("nccl", "peer"):
        raise ParametersInvalid(f"transport must be 'nccl' or 'peer', but got {transport}.")
    if transport == "peer" and not (cuda and b == 1 and attn_fn is None):
        raise ParametersInvalid("transport='peer' needs CUDA tensors, batch 1 and the default attention.")
    key_ = (device, q.dtype, world, b, s_loc, n, d, tuple(sizes), id(group))
    if transport == "peer":
        return _ulysses_peer(qr, kr, vr, out, outr, sizes, world, dist.get_rank(group), rows, n_loc, d, scale, group,
                             rope_args, profile, key_, _piece_ready, _piece_done)
    # One set of buffers per piece: a piece's buffers are free again when the call returns.
    shapes = []
    for h in sizes:
        shapes += [(world, rows, 3 * h, d)] * 2 + [(world, rows, h, d)] * 2  # send, recv, o_send, o_recv
    bufs = _buffers(key_, shapes, q.dtype, device)

    compute = comm = ret = None
    attn_streams = [None, None]
    if cuda:
        compute = torch.cuda.current_stream(device)
        comm, ret, compute2 = _side_streams(device)
        attn_streams = [compute, compute2]
        for side in (comm, ret, compute2):
            side.wait_stream(compute)  # the inputs and the buffers' previous readers
    timer = _Timer(profile, cuda)

    def on(stream):
        return torch.cuda.stream(stream) if cuda else _NULL

    def record(stream):
        if not cuda:
            return None
        ev = torch.cuda.Event()
        ev.record(stream)
        return ev

    def exchange_in(c, head0):
        """Pack piece c for every destination and start its all-to-all (inbound stream)."""
        send, recv = bufs[4 * c], bufs[4 * c + 1]
        with on(comm):
            if _piece_ready is not None:
                _piece_ready(c, head0, sizes[c], comm)  # e.g. wait for the piece's heads to arrive from the host
            with timer.span("pack", comm):
                _move((qr, kr, vr), send, rows, world, n_loc, head0, sizes[c], rope=rope_args,
                      thread_blocks=0)
            with timer.span("exchange_in", comm):
                dist.all_to_all_single(recv, send, group=group)
            return record(comm)

    def local_attention(c, stream):
        h = sizes[c]
        recv, o_send = bufs[4 * c + 1], bufs[4 * c + 2]
        # recv[r] holds rank r's rows: with B == 1 the buffer already is [S, 3h, D].
        if b == 1:
            full = recv.view(1, world * s_loc, 3 * h, d)
            o_view = o_send.view(1, world * s_loc, h, d)
        else:
            full = recv.view(world, b, s_loc, 3 * h, d).permute(1, 0, 2, 3, 4).reshape(b, world * s_loc, 3 * h, d)
            o_view = None
        qq, kk, vv = full[:, :, 0:h], full[:, :, h:2 * h], full[:, :, 2 * h:3 * h]
        with on(stream), timer.span("attention", stream):
            if attn_fn is None and o_view is not None and cuda:
                _default_attention(qq, kk, vv, scale, out=o_view)  # straight into the return exchange's send buffer
            else:
                o = attn_fn(qq, kk, vv, scale) if attn_fn else _default_attention(qq, kk, vv, scale)  # [B, S, h, D]
                o_send.view(world, b, s_loc, h, d).copy_(o.reshape(b, world, s_loc, h, d).permute(1, 0, 2, 3, 4))
        return record(stream)

    def send_back(c, head0, done):
        """Return exchange of piece c and the scatter into the caller's output (outbound stream)."""
        o_send, o_recv = bufs[4 * c + 2], bufs[4 * c + 3]
        if cuda:
            ret.wait_event(done)
        with on(ret):
            with timer.span("exchange_out", ret):
                dist.all_to_all_single(o_recv, o_send, group=group)
            with timer.span("unpack", ret):
                _move((outr,), o_recv, rows, world, n_loc, head0, sizes[c], inverse=True)
            if _piece_done is not None:
                _piece_done(c, head0, sizes[c], ret)  # e.g. start the piece's copy back to the host

    head0 = [sum(sizes[:c]) for c in range(len(sizes))]
    arrived = exchange_in(0, head0[0])
    for c in range(len(sizes)):
        ready = arrived
        if c + 1 < len(sizes):
            arrived = exchange_in(c + 1, head0[c + 1])
        stream = attn_streams[c % 2]
        if cuda:
            stream.wait_event(ready)
        send_back(c, head0[c], local_attention(c, stream))
    if cuda:
        # The caller's stream continues behind everything this call started; the side streams' last readers of
        # q, k, v and of the buffers are then ordered before whatever the caller, or the next call, does.
        for side in (attn_streams[1], ret, comm):
            compute.wait_stream(side)
    timer.finish()
    return out


def _ulysses_peer(qr, kr, vr, out, outr, sizes, world, rank, rows, n_loc, d, scale, group, rope_args, profile, key_,
                  piece_ready, piece_done):
    """The exchange over peer memory.  Per piece c (communication stream): the re-shard kernel writes, for
    every rank r, that rank's heads of my rows into rows [rank * rows, ...) of r's receive buffer c; a
    one-element all-reduce then tells every rank that all blocks of piece c have been written.  Compute
    stream: attention on my receive buffer into my output buffer c; another one-element all-reduce; then
    the scatter kernel loads, from every rank r, the rows of r's output buffer c that are mine."""
    from .. import _cabi
    device = qr.device
    shapes = []
    for h in sizes:
        shapes += [(world * rows, 3 * h, d), (world * rows, h, d)]  # receive buffer [S, 3h, D], output buffer [S, h, D]
    pb = _peer_buffers(key_ + ("peer",), shapes, qr.dtype, device, group)
    compute = torch.cuda.current_stream(device)
    comm, ret, compute2 = _side_streams(device)
    attn_streams = [compute, compute2]
    for side in (comm, ret, compute2):
        side.wait_stream(compute)
    timer = _Timer(profile, True)
    esz = qr.element_size()
    head0 = [sum(sizes[:c]) for c in range(len(sizes))]

    def order_ranks():
        # Every rank reaches this point of the stream it is called under before any rank leaves it.
        dist.all_reduce(pb.flag, group=group)

    def send(c):
        h = sizes[c]
        with torch.cuda.stream(comm):
            if piece_ready is not None:
                piece_ready(c, head0[c], h, comm)
            with timer.span("pack", comm):
                ptrs = [pb.peer_ptr[r][2 * c] + rank * rows * 3 * h * d * esz for r in range(world)]
                cos = sin = None
                mode = 0
                if rope_args is not None:
                    cos, sin, mode = rope_args
                _cabi.ulysses_move((qr, kr, vr), ptrs, 3 * h * d, rows, world, n_loc, head0[c], h, cos=cos, sin=sin,
                                   rope_mode=mode, thread_blocks=0)
            with timer.span("exchange_in", comm):
                order_ranks()
            ev = torch.cuda.Event()
            ev.record(comm)
            return ev

    arrived = send(0)
    for c, h in enumerate(sizes):
        ready = arrived
        if c + 1 < len(sizes):
            arrived = send(c + 1)
        stream = attn_streams[c % 2]
        stream.wait_event(ready)
        recv, o_buf = pb.local[2 * c], pb.local[2 * c + 1]
        full = recv.view(1, world * rows, 3 * h, d)
        with torch.cuda.stream(stream), timer.span("attention", stream):
            _cabi.attention(full[:, :, 0:h], full[:, :, h:2 * h], full[:, :, 2 * h:3 * h], head_first=False, scale=scale,
                            out=o_buf.view(1, world * rows, h, d))
        done = torch.cuda.Event()
        done.record(stream)
        ret.wait_event(done)
        with torch.cuda.stream(ret):
            with timer.span("exchange_out", ret):
                order_ranks()
            with timer.span("unpack", ret):
                ptrs = [pb.peer_ptr[r][2 * c + 1] + rank * rows * h * d * esz for r in range(world)]
                _cabi.ulysses_move((outr,), ptrs, h * d, rows, world, n_loc, head0[c], h, inverse=True)
            if piece_done is not None:
                piece_done(c, head0[c], h, ret)
    # The next call writes into the peers' receive buffers and this rank's output buffers again: it may only
    # start once every rank has finished reading them, i.e. after everyone's last scatter kernel.
    with torch.cuda.stream(ret):
        order_ranks()
    for side in (attn_streams[1], ret, comm):
        compute.wait_stream(side)
    timer.finish()
    return out


_HOST_STAGING = {}


def ulysses_attention_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, out: Optional[torch.Tensor] = None,
                           group=None, scale: Optional[float] = None,
                           head_chunks: Union[None, int, Sequence[int]] = None, device=None) -> torch.Tensor:
    """`ulysses_attention` on operands that live in pinned host memory: this rank's [B, S/P, N, D] slices in,
    a pinned [B, S/P, N, D] slice out.  The copies are pipelined with the exchange and the attention piece
    by piece: the heads of piece c+1 cross PCIe (strided copies, one per tensor) while piece c is exchanged
    and computed, and piece c-1's output columns go back to the host behind them, so only the first piece's
    copy in and the last piece's copy out are exposed.  Returns after the last copy has landed."""
    from .. import _cabi
    for name, x in (("query", query), ("key", key), ("value", value)):
        if not isinstance(x, torch.Tensor) or x.dim() != 4 or x.is_cuda or not x.is_pinned() or not x.is_contiguous():
            raise ParametersInvalid(f"The input {name} must be a contiguous 4-D tensor in pinned host memory.")
    if key.shape != query.shape or value.shape != query.shape or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ParametersInvalid("query, key and value must share shape and dtype.")
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    world = dist.get_world_size(group)
    b, s_loc, n, d = query.shape
    if n % world:
        raise ParametersInvalid(f"The head number {n} must be divisible by the sequence-parallel size {world}.")
    if out is None:
        out = torch.empty(query.shape, dtype=query.dtype, pin_memory=True)
    n_loc = n // world
    if head_chunks is None:
        head_chunks = default_head_pieces(n_loc, s_loc * world, b, waves=8, split_small=True)
    sizes = _piece_sizes(head_chunks, n_loc, s_loc * world, b)
    skey = (device.index, tuple(query.shape), query.dtype)
    if skey not in _HOST_STAGING:
        _HOST_STAGING.clear()
        _HOST_STAGING[skey] = ([torch.empty(query.shape, dtype=query.dtype, device=device) for _ in range(4)],
                               torch.cuda.Stream(device), torch.cuda.Stream(device))
    (dq, dk, dv, do), copy_in, copy_out = _HOST_STAGING[skey]
    compute = torch.cuda.current_stream(device)
    copy_in.wait_stream(compute)
    copy_out.wait_stream(compute)
    esz = query.element_size()
    pitch = n_loc * d * esz          # one destination rank's head group of one token
    height = b * s_loc * world       # (token, destination rank) pairs

    def start_copy_in(head0, heads):
        off = head0 * d * esz
        for dst, src in ((dq, query), (dk, key), (dv, value)):
            _cabi.copy_2d(dst.data_ptr() + off, pitch, src.data_ptr() + off, pitch, heads * d * esz, height, copy_in)
        ev = torch.cuda.Event()
        ev.record(copy_in)
        return ev

    head0 = [sum(sizes[:c]) for c in range(len(sizes))]
    arrived = [start_copy_in(head0[c], sizes[c]) for c in range(len(sizes))]  # the copy engine takes them in order
    copied_out = []

    def piece_ready(c, h0, heads, stream):
        stream.wait_event(arrived[c])

    def piece_done(c, h0, heads, stream):
        ev = torch.cuda.Event()
        ev.record(stream)
        copy_out.wait_event(ev)
        off = h0 * d * esz
        _cabi.copy_2d(out.data_ptr() + off, pitch, do.data_ptr() + off, pitch, heads * d * esz, height, copy_out)
        done = torch.cuda.Event()
        done.record(copy_out)
        copied_out.append(done)

    ulysses_attention(dq, dk, dv, group=group, scale=scale, head_chunks=sizes, _piece_ready=piece_ready,
                      _piece_done=piece_done, _out=do)
    compute.wait_event(copied_out[-1])
    copied_out[-1].synchronize()
    raise_if_kernel_gave_up("ulysses_attention_host")  # the call has synchronised anyway
    return out
