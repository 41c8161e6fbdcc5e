"""Attention on operands that live in pinned host memory (weights-offload style callers).

`attention_forward_host` cuts the heads into chunks and runs a three-stage pipeline on three CUDA
streams -- host-to-device copy of chunk c+1, `attention_forward` on chunk c, device-to-host copy of
chunk c-1 -- so that for a long sequence the PCIe transfers hide behind the kernel instead of
adding to it.  It has no counterpart in MindIE-SD (whose offload module moves weights, not
activations).  The device side is two fixed sets of staging buffers ordered by events.
"""
from __future__ import annotations

import threading
from typing import Optional

import torch

from ...utils.exception import ParametersInvalid
from ...utils.status import raise_if_kernel_gave_up


_STAGING = {}  # device index -> (key, buffers, streams): one set of staging buffers per device, reused across calls
_LOCKS = {}    # device index -> lock: calls on one device take turns (they share the staging buffers)
_LOCKS_GUARD = threading.Lock()


def _staging(device, shape, dtype):
    """Two (q, k, v, o) sets of device buffers for one head chunk and the two copy streams.  They are kept between calls: taking
    them from the allocator per chunk makes it grow and call cudaMalloc in the middle of the pipeline,
    which stalls every stream."""
    key = (tuple(shape), dtype)
    cached = _STAGING.get(device.index)
    if cached is None or cached[0] != key:
        _STAGING.pop(device.index, None)
        bufs = [[torch.empty(shape, dtype=dtype, device=device) for _ in range(4)] for _ in range(2)]
        streams = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        _STAGING[device.index] = (key, bufs, streams)
    return _STAGING[device.index][1:]


def default_host_chunks(heads: int, seq: int = 1 << 30, batch: int = 1) -> int:
    """Most chunks (at most 40) such that a chunk still launches two full waves of thread blocks (one
    block per 256 query rows of a head, 148 SMs): the first copy in and the last copy out are the
    only ones that do not overlap the kernel, so they should be small."""
    blocks_per_head = batch * ((seq + 255) // 256)
    min_heads = max(1, -(-296 // blocks_per_head))
    ok = [c for c in range(1, min(heads, 40) + 1) if heads % c == 0 and heads // c >= min_heads]
    return max(ok) if ok else 1


def attention_forward_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, out: Optional[torch.Tensor] = None,
                           scale: Optional[float] = None, head_chunks: Optional[int] = None, device=None) -> torch.Tensor:
    """query/key/value: pinned host tensors [B, N, S, D] (head-first, so a head chunk is one contiguous
    range).  Returns (and, if given, fills) a pinned host tensor of the same shape.  The call returns
    after the last chunk has arrived in host memory.  head_chunks defaults to default_host_chunks(N, S, B)."""
    from ... import _cabi
    for name, x in (("query", query), ("key", key), ("value", value)):
        if not isinstance(x, torch.Tensor) or x.dim() != 4:
            raise ParametersInvalid(f"The input {name} must be a 4-D torch.Tensor.")
        if x.is_cuda or not x.is_pinned():
            raise ParametersInvalid(f"The input {name} must live in pinned host memory.")
    b, n, s, d = query.shape
    if key.shape != query.shape or value.shape != key.shape or key.dtype != query.dtype or value.dtype != query.dtype:
        raise ParametersInvalid("query, key and value must share shape and dtype.")
    if head_chunks is None:
        head_chunks = default_host_chunks(n, s, b)
    if head_chunks < 1 or n % head_chunks:
        raise ParametersInvalid(f"head_chunks={head_chunks} must divide the {n} heads.")
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    if out is None:
        out = torch.empty(query.shape, dtype=query.dtype, pin_memory=True)
    hc = n // head_chunks
    with _LOCKS_GUARD:
        lock = _LOCKS.setdefault(device.index, threading.Lock())
    with lock:
        return _run_pipeline(query, key, value, out, scale, head_chunks, hc, device)


def _run_pipeline(query, key, value, out, scale, head_chunks, hc, device):
    from ... import _cabi
    b, _, s, d = query.shape
    bufs, (copy_in, copy_out) = _staging(device, (b, hc, s, d), query.dtype)
    compute = torch.cuda.current_stream(device)
    copy_in.wait_stream(compute)
    copy_out.wait_stream(compute)
    computed, stored = {}, {}

    def fetch(c):
        slot = bufs[c % 2]
        with torch.cuda.stream(copy_in):
            if c - 2 in computed:  # the kernel that read this slot last
                copy_in.wait_event(computed[c - 2])
            for dst, src in zip(slot[:3], (query, key, value)):
                dst.copy_(src[:, c * hc:(c + 1) * hc], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_in)
        return ev

    fetched = fetch(0)
    for c in range(head_chunks):
        dq, dk, dv, do = bufs[c % 2]
        ready = fetched
        if c + 1 < head_chunks:
            fetched = fetch(c + 1)
        compute.wait_event(ready)
        if c - 2 in stored:  # the copy that drained this slot's output last
            compute.wait_event(stored[c - 2])
        _cabi.attention(dq, dk, dv, head_first=True, scale=scale, out=do)
        computed[c] = torch.cuda.Event()
        computed[c].record(compute)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(computed[c])
            out[:, c * hc:(c + 1) * hc].copy_(do, non_blocking=True)
            stored[c] = torch.cuda.Event()
            stored[c].record(copy_out)
    # The calling stream is ordered after the last copy out, and so is the host.
    compute.wait_event(stored[head_chunks - 1])
    stored[head_chunks - 1].synchronize()
    raise_if_kernel_gave_up("attention_forward_host")  # the call has synchronised anyway
    return out
