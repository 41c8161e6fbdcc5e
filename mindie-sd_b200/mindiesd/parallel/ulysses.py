"""Ulysses sequence-parallel attention: every rank holds a slice of the sequence with all heads,
an all-to-all turns that into the full sequence with a slice of the heads, attention runs locally,
and a second all-to-all turns the result back.

MindIE-SD documents this pattern (docs/zh/features/parallelism.md:207-233) without shipping it;
this is the same tensor contract -- BSND in, BSND out, `N % world_size == 0` -- with two additions:
q, k and v travel in ONE all-to-all per head chunk (stacked along the head axis), and the local
heads are cut into chunks so that the exchange of chunk c+1 and the return of chunk c-1 run on a
communication stream while chunk c's attention runs on the compute stream.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from ..utils.exception import ParametersInvalid


def _default_attention(q, k, v, scale):
    # BSND views with a non-unit head-group stride: the kernel reads them through strides.
    return torch.ops.mindiesd.attention_fwd(q, k, v, float(scale), False)


class _Streams:
    """Compute/communication stream pair with event hand-over; on CPU every method is a no-op."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.compute = torch.cuda.current_stream(device)
            self.comm = _comm_stream(device)

    def comm_after_compute(self):
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self.compute)
            self.comm.wait_event(ev)

    def compute_after_comm(self):
        if self.cuda:
            ev = torch.cuda.Event()
            ev.record(self.comm)
            return ev
        return None

    def wait(self, ev):
        if self.cuda and ev is not None:
            self.compute.wait_event(ev)

    def on_comm(self):
        return torch.cuda.stream(self.comm) if self.cuda else _Null()


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_COMM_STREAMS = {}


def _comm_stream(device):
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = torch.cuda.Stream(device=device)
    return _COMM_STREAMS[key]


def default_head_chunks(local_heads: int, seq: int = 1 << 30, batch: int = 1, limit: int = 8) -> int:
    """Most pieces (a divisor of the local head count, at most `limit`) such that a piece still launches
    about eight full waves of attention thread blocks (one block per 256 query rows of a head, 148 SMs).
    A piece of one or two waves loses more to the exchange kernels that run beside it, which take SMs
    for a while, and to the partial last wave than its overlap wins back: at 75 600 tokens and 8 GPUs
    (5 local heads) one piece measured 13.8 ms per layer, five pieces 15.4 ms."""
    blocks_per_head = batch * ((seq + 255) // 256)
    min_heads = max(1, -(-8 * 148 // blocks_per_head))
    ok = [c for c in range(1, min(local_heads, limit) + 1) if local_heads % c == 0 and local_heads // c >= min_heads]
    return max(ok) if ok else 1


def ulysses_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, group=None,
                      scale: Optional[float] = None, head_chunks: Optional[int] = None,
                      attn_fn: Optional[Callable] = None) -> torch.Tensor:
    """query/key/value: this rank's [B, S/P, N, D] slice (BSND).  Returns this rank's [B, S/P, N, D]
    slice of the attention output over the full sequence.

    head_chunks: pieces the N/P local heads are cut into for overlap (default: default_head_chunks --
    as many as still leave every piece about eight waves of thread blocks, at most 8).  attn_fn(q, k, v, scale) -> out on [B, S, h, D] BSND tensors replaces the local
    attention (sparse or FP8 variants); the default is the dense kernel.
    """
    if query.dim() != 4 or key.shape != query.shape or value.shape != query.shape:
        raise ParametersInvalid("ulysses_attention expects q, k, v of one shape [B, S/P, N, D].")
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    b, s_loc, n, d = query.shape
    if n % world:
        raise ParametersInvalid(f"The head number {n} must be divisible by the sequence-parallel size {world}.")
    if scale is None:
        scale = d ** -0.5
    attn = attn_fn or _default_attention
    if world == 1:
        return attn(query, key, value, scale)
    n_loc = n // world
    if head_chunks is None:
        head_chunks = default_head_chunks(n_loc, s_loc * world, b)
    if head_chunks < 1 or n_loc % head_chunks:
        raise ParametersInvalid(f"head_chunks={head_chunks} must divide the {n_loc} local heads.")
    hc = n_loc // head_chunks
    st = _Streams(query.device)
    out = torch.empty_like(query)
    # [B, S/P, P, N/P, D]: axis 2 is the destination rank of a head group.
    qv, kv, vv = (x.view(b, s_loc, world, n_loc, d) for x in (query, key, value))
    ov = out.view(b, s_loc, world, n_loc, d)

    def exchange_in(c):
        """Pack chunk c of every destination's head group and start its all-to-all."""
        send = torch.empty(world, b, s_loc, 3 * hc, d, dtype=query.dtype, device=query.device)
        for i, x in enumerate((qv, kv, vv)):
            send[:, :, :, i * hc:(i + 1) * hc].copy_(x[:, :, :, c * hc:(c + 1) * hc].permute(2, 0, 1, 3, 4))
        recv = torch.empty_like(send)
        st.comm_after_compute()
        with st.on_comm():
            dist.all_to_all_single(recv, send, group=group)
        if st.cuda:
            send.record_stream(st.comm)
            recv.record_stream(st.comm)
        return recv, st.compute_after_comm()

    def local_attention(recv):
        # recv[r] holds rank r's rows: with B == 1 the buffer already is [S, 3*hc, D].
        if b == 1:
            full = recv.view(1, world * s_loc, 3 * hc, d)
        else:
            full = recv.permute(1, 0, 2, 3, 4).reshape(b, world * s_loc, 3 * hc, d)
        o = attn(full[:, :, 0:hc], full[:, :, hc:2 * hc], full[:, :, 2 * hc:3 * hc], scale)  # [B, S, hc, D]
        return o.reshape(b, world, s_loc, hc, d).permute(1, 0, 2, 3, 4).contiguous()  # [P, B, S/P, hc, D]

    def exchange_out(o_send):
        recv = torch.empty_like(o_send)
        st.comm_after_compute()
        with st.on_comm():
            dist.all_to_all_single(recv, o_send, group=group)
        if st.cuda:
            o_send.record_stream(st.comm)
            recv.record_stream(st.comm)
        return recv, st.compute_after_comm()

    def unpack(c, recv, ev):
        st.wait(ev)
        ov[:, :, :, c * hc:(c + 1) * hc].copy_(recv.permute(1, 2, 0, 3, 4))  # recv[p]: heads of rank p's group

    pending_in = exchange_in(0)
    pending_out = None
    for c in range(head_chunks):
        recv, ev = pending_in
        if c + 1 < head_chunks:
            pending_in = exchange_in(c + 1)
        st.wait(ev)
        o_send = local_attention(recv)
        if pending_out is not None:
            unpack(*pending_out)
        r, e = exchange_out(o_send)
        pending_out = (c, r, e)
    unpack(*pending_out)
    del rank
    return out
