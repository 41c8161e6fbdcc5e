"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations (Wan2.1-shaped video-DiT self-attention).  No dataset is involved: the latent
grids stand in for Wan2.1 latents after 1x2x2 patchify.

    C1  B1 N12 S2048          fp32, N(0,1), k has a per-channel offset N(0,0.5)
    C2  B1 N12 S32760 21x30x52 bf16, 0.5*N(0,1), 3-D RoPE (44/42/42 channels, base 10000) on q, k
    C3  B1 N40 S75600 21x45x80 bf16, as C2 plus a per-head low-rank spatial/temporal bias
    C4  same shape             bf16 N(0,1), 1 % outlier channels scaled 8x
    C5  C3's dense tensors, sharded along the sequence across ranks

On CPU the normals come from numpy's RandomState (a frozen stream, so fixtures stay valid);
on a CUDA device from torch's generator of that device (fast at full size).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

HEAD_DIM = 128


@dataclass(frozen=True)
class Config:
    name: str
    batch: int
    heads: int
    grid: tuple | None  # (t, h, w) latent grid, None when the sequence has no grid
    seq: int
    dtype: torch.dtype

    @property
    def flops(self) -> float:
        """Dense attention FLOPs: 4 * B * N * S^2 * D."""
        return 4.0 * self.batch * self.heads * self.seq * self.seq * HEAD_DIM


C1 = Config("C1", 1, 12, None, 2048, torch.float32)
C2 = Config("C2", 1, 12, (21, 30, 52), 21 * 30 * 52, torch.bfloat16)
C3 = Config("C3", 1, 40, (21, 45, 80), 21 * 45 * 80, torch.bfloat16)
C4 = Config("C4", 1, 40, (21, 45, 80), 21 * 45 * 80, torch.bfloat16)


def _normal(shape, seed, device):
    device = torch.device(device)
    if device.type == "cuda":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        return torch.randn(shape, generator=g, device=device, dtype=torch.float32)
    rs = np.random.RandomState(seed)
    return torch.from_numpy(rs.standard_normal(size=shape).astype(np.float32))


def rope_tables(grid, device="cpu", base=10000.0, split=(44, 42, 42)):
    """cos/sin tables [S, 128] of a 3-D rotary embedding: the channel pairs are divided between
    the t, h and w axes as 22/21/21 pairs, pair i of an axis with d channels turning by
    pos * base^(-2i/d).  Laid out for the interleaved rotation (x_{2i}, x_{2i+1})."""
    t, h, w = grid
    pos = torch.stack(torch.meshgrid(torch.arange(t), torch.arange(h), torch.arange(w), indexing="ij"), -1)
    pos = pos.reshape(-1, 3).to(torch.float64)
    angles = []
    for axis, d in enumerate(split):
        inv = base ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
        angles.append(pos[:, axis:axis + 1] * inv[None, :])
    ang = torch.cat(angles, dim=1).repeat_interleave(2, dim=1)  # [S, 128]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def apply_rope(x, cos, sin):
    """x [B, N, S, D]; interleaved rotation x*cos + rot(x)*sin with rot(x) = (-x1, x0, -x3, x2, ...),
    the formula of mindiesd/layers/rope.py:104-108 of MindIE-SD."""
    xr = torch.stack([-x[..., 1::2], x[..., 0::2]], dim=-1).flatten(-2)
    return x * cos + xr * sin


def _structure_bias(cfg, seed, device, rank=3, strength=1.5):
    """Per-head low-rank term added to q and k so that block scores have spatial and temporal
    structure: sum_r u_r(head) * f_r(t, h, w) with smooth f_r."""
    t, h, w = cfg.grid
    tt, hh, ww = torch.meshgrid(torch.arange(t) / t, torch.arange(h) / h, torch.arange(w) / w, indexing="ij")
    feats = torch.stack([torch.cos(2 * math.pi * tt), torch.sin(2 * math.pi * hh) * torch.cos(math.pi * ww),
                         2 * tt - 1], dim=-1).reshape(-1, 3)[:, :rank].float().to(device)
    u = _normal((cfg.heads, rank, HEAD_DIM), seed, device) * (strength / math.sqrt(HEAD_DIM))
    return torch.einsum("sr,nrd->nsd", feats, u)[None]  # [1, N, S, D]


def make_qkv(cfg: Config, device="cpu", seed=0, heads=None, layout="BNSD"):
    """q, k, v of a configuration (optionally only the first `heads` heads), in `layout`."""
    n = heads or cfg.heads
    sub = Config(cfg.name, cfg.batch, n, cfg.grid, cfg.seq, cfg.dtype)
    shape = (cfg.batch, n, cfg.seq, HEAD_DIM)
    q, k, v = (_normal(shape, seed * 16 + i, device) for i in range(3))
    if cfg.name == "C1":
        k = k + 0.5 * _normal((HEAD_DIM,), seed * 16 + 3, device)
    elif cfg.name in ("C2", "C3"):
        q, k, v = 0.5 * q, 0.5 * k, 0.5 * v
        if cfg.name == "C3":
            bias = _structure_bias(sub, seed * 16 + 4, device)
            q, k = q + bias, k + bias
        cos, sin = rope_tables(cfg.grid, device)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    elif cfg.name == "C4":
        outl = _normal((n, HEAD_DIM), seed * 16 + 5, device).abs()
        # about 1 % of the channels (at least one per head) carry 8x larger values
        kth = max(1, round(0.01 * HEAD_DIM))
        thr = outl.topk(kth, dim=-1).values[:, -1:]
        gain = torch.where(outl >= thr, 8.0, 1.0)[None, :, None, :]
        q, k, v = q * gain, k * gain, v * gain
    q, k, v = (x.to(cfg.dtype) for x in (q, k, v))
    if layout == "BSND":
        q, k, v = (x.transpose(1, 2).contiguous() for x in (q, k, v))
    return q, k, v
