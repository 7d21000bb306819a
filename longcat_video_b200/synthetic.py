"""Seeded synthetic Q/K/V for the benchmark configurations and the parity tests.

No dataset or checkpoint is involved anywhere: activations are drawn from a CPU
``torch.Generator`` (portable across machines) with the shapes of the DiT's
self-attention inputs (``longcat_video/modules/attention.py:107-121`` hands
``flash_attn_bsa_3d`` tensors shaped ``[B, heads, T*H*W, head_dim]``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class Workload:
    name: str
    seed: int
    batch: int
    heads: int
    head_dim: int
    grid_q: Tuple[int, int, int]
    grid_k: Tuple[int, int, int]
    chunk: Tuple[int, int, int]
    sparsity: float
    dtype: torch.dtype
    recipe: str  # "normal" | "scaled_lowrank"

    @property
    def sq(self) -> int:
        return self.grid_q[0] * self.grid_q[1] * self.grid_q[2]

    @property
    def sk(self) -> int:
        return self.grid_k[0] * self.grid_k[1] * self.grid_k[2]


def _w(name, seed, heads, grid_q, grid_k=None, sparsity=0.9375, dtype=torch.bfloat16,
       recipe="scaled_lowrank", chunk=(4, 4, 4)):
    return Workload(name, seed, 1, heads, 128, tuple(grid_q), tuple(grid_k or grid_q), tuple(chunk),
                    sparsity, dtype, recipe)


# The named configurations.  "legal" grids divide by the 4x4x4 block and are the ones the
# reference accepts (bsa_interface.py:639-640); the literal 30/45-row grids are ragged.
WORKLOADS = {
    "cfg1_plumbing": _w("cfg1_plumbing", 1001, 4, (4, 8, 8), sparsity=0.5, dtype=torch.float32, recipe="normal"),
    "480p_legal": _w("480p_legal", 1002, 32, (24, 32, 52)),
    "480p_ragged": _w("480p_ragged", 1002, 32, (24, 30, 52)),
    "720p_legal": _w("720p_legal", 1003, 32, (24, 48, 80)),
    "720p_bucket": _w("720p_bucket", 1003, 32, (24, 44, 80)),
    "720p_ragged": _w("720p_ragged", 1003, 32, (24, 45, 80)),
    # the block shape flash_attn_bsa_3d takes when the caller passes none: [4, 4, 8], 128 tokens
    "480p_blocks128": _w("480p_blocks128", 1002, 32, (24, 32, 56), chunk=(4, 4, 8)),
    "720p_blocks128": _w("720p_blocks128", 1003, 32, (24, 48, 80), chunk=(4, 4, 8)),
    # every parameter of the entry point left at its default: [4, 4, 8] blocks and sparsity 0.875 (90 of 720 blocks)
    "720p_defaults": _w("720p_defaults", 1003, 32, (24, 48, 80), chunk=(4, 4, 8), sparsity=0.875),
    "vc_legal": _w("vc_legal", 1005, 32, (12, 48, 80), (24, 48, 80), recipe="normal"),
    "vc_ragged": _w("vc_ragged", 1005, 32, (11, 45, 80), (24, 45, 80), recipe="normal"),
}


def _positions(grid):
    T, H, W = grid
    t = torch.arange(T, dtype=torch.float32).view(T, 1, 1).expand(T, H, W).reshape(-1) / T
    h = torch.arange(H, dtype=torch.float32).view(1, H, 1).expand(T, H, W).reshape(-1) / H
    w = torch.arange(W, dtype=torch.float32).view(1, 1, W).expand(T, H, W).reshape(-1) / W
    return t, h, w


def make_qkv(wl: Workload, heads: Optional[int] = None, head_offset: int = 0, device="cpu"):
    """Draw ``q [B,h,Sq,D]``, ``k, v [B,h,Sk,D]`` for heads ``head_offset .. head_offset+heads``.

    Every head has its own generator stream (seed, head) so that a rank holding a subset
    of the heads draws exactly the values the full tensor would have there.
    """
    heads = wl.heads if heads is None else heads
    D = wl.head_dim
    qs, ks, vs = [], [], []
    for hh in range(head_offset, head_offset + heads):
        g = torch.Generator().manual_seed(wl.seed * 1000 + hh)
        q = torch.randn(wl.batch, 1, wl.sq, D, generator=g)
        k = torch.randn(wl.batch, 1, wl.sk, D, generator=g)
        v = torch.randn(wl.batch, 1, wl.sk, D, generator=g)
        if wl.recipe == "scaled_lowrank":
            s = D ** -0.5
            q, k, v = q * s, k * s, v * s
            r = 4
            freq = torch.randint(0, 4, (3, r), generator=g).to(torch.float32)
            phase = torch.rand(r, generator=g) * (2 * math.pi)
            wmat = torch.randn(D, r, generator=g) * 0.5
            t, h, w = _positions(wl.grid_k)
            arg = 2 * math.pi * (t[:, None] * freq[0] + h[:, None] * freq[1] + w[:, None] * freq[2]) + phase
            u = torch.cos(arg)  # [Sk, r]
            k = k + (u @ wmat.t()).view(1, 1, wl.sk, D)
        elif wl.recipe != "normal":
            raise ValueError(wl.recipe)
        qs.append(q.to(wl.dtype))
        ks.append(k.to(wl.dtype))
        vs.append(v.to(wl.dtype))
    q, k, v = torch.cat(qs, 1), torch.cat(ks, 1), torch.cat(vs, 1)
    if device != "cpu":
        q, k, v = q.to(device), k.to(device), v.to(device)
    return q, k, v
