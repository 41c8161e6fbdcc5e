"""Attention on operands that live in pinned host memory (weights-offload style callers).

`attention_forward_host` cuts the heads into chunks and runs a three-stage pipeline on three CUDA
streams -- host-to-device copy of chunk c+1, `attention_forward` on chunk c, device-to-host copy of
chunk c-1 -- so that for a long sequence the PCIe transfers hide behind the kernel instead of
adding to it.  It has no counterpart in MindIE-SD (whose offload module moves weights, not
activations); it composes the public `attention_forward` and nothing else.
"""
from __future__ import annotations

from typing import Optional

import torch

from .attention_forward import attention_forward
from ...utils.exception import ParametersInvalid


def attention_forward_host(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, out: Optional[torch.Tensor] = None,
                           scale: Optional[float] = None, head_chunks: int = 5, device=None) -> torch.Tensor:
    """query/key/value: pinned host tensors [B, N, S, D] (head-first, so a head chunk is one contiguous
    range).  Returns (and, if given, fills) a pinned host tensor of the same shape.  The call returns
    after the last chunk has arrived in host memory."""
    for name, x in (("query", query), ("key", key), ("value", value)):
        if not isinstance(x, torch.Tensor) or x.dim() != 4:
            raise ParametersInvalid(f"The input {name} must be a 4-D torch.Tensor.")
        if x.is_cuda or not x.is_pinned():
            raise ParametersInvalid(f"The input {name} must live in pinned host memory.")
    b, n, s, d = query.shape
    if key.shape[0] != b or key.shape[1] != n or value.shape != key.shape:
        raise ParametersInvalid("query, key and value must share batch and head counts.")
    if head_chunks < 1 or n % head_chunks:
        raise ParametersInvalid(f"head_chunks={head_chunks} must divide the {n} heads.")
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    if out is None:
        out = torch.empty(query.shape, dtype=query.dtype, pin_memory=True)
    hc = n // head_chunks
    compute = torch.cuda.current_stream(device)
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    copy_in.wait_stream(compute)

    def fetch(c):
        with torch.cuda.stream(copy_in):
            dev = [x[:, c * hc:(c + 1) * hc].to(device, non_blocking=True) for x in (query, key, value)]
            ev = torch.cuda.Event()
            ev.record(copy_in)
        return dev, ev

    pending = fetch(0)
    last = None
    for c in range(head_chunks):
        (dq, dk, dv), ev = pending
        if c + 1 < head_chunks:
            pending = fetch(c + 1)
        compute.wait_event(ev)
        o = attention_forward(dq, dk, dv, scale=scale, head_first=True)
        for x in (dq, dk, dv):
            x.record_stream(compute)
        done = torch.cuda.Event()
        done.record(compute)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(done)
            out[:, c * hc:(c + 1) * hc].copy_(o, non_blocking=True)
            o.record_stream(copy_out)
            last = torch.cuda.Event()
            last.record(copy_out)
    if last is not None:
        last.synchronize()
    return out
