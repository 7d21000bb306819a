"""q/k RMSNorm + 3-D rotary embedding in one CUDA pass: the step in front of the block-sparse attention.

Stands in for these lines of ``Attention.forward`` (``longcat_video/modules/attention.py:113-121``)::

    q, k = self.q_norm(q), self.k_norm(k)          # RMSNorm_FP32, longcat_video/modules/blocks.py:42-53
    q, k = self.rope_3d(q, k, grid_size=shape)     # longcat_video/modules/rope_3d.py:99-120

which run as six elementwise passes with fp32 temporaries.  ``qk_norm_rope`` reads the strided q and k views of the
fused qkv projection once and writes ``[B, H, S, D]`` outputs once.  All arithmetic is in liblcbsa.so
(``lcbsa_norm_rope``); PyTorch builds the small angle table and allocates the outputs.  There is no CPU path.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from .. import _lib as L

_TABLES = {}


def _angles(n: int, part: int, base: float) -> torch.Tensor:
    """Angles of one axis, ``[n, part]``: pair i of the part turns by ``pos / base**(2i/part)`` (rope_3d.py:62-84),
    repeated for both elements of the pair (rope_3d.py:113-115)."""
    inv = 1.0 / (base ** (torch.arange(0, part, 2)[: part // 2].float() / part))
    pos = torch.arange(n, dtype=torch.float32)
    return torch.repeat_interleave(pos[:, None] * inv[None, :], 2, dim=1)


def rope_table(grid_size: Sequence[int], head_dim: int, device, base: float = 10000.0) -> torch.Tensor:
    """The packed separable fp32 table ``lcbsa_norm_rope`` reads, cached per (grid, head_dim, base, device):
    ``cos_t [T, dt] sin_t [T, dt] cos_h [H, dh] sin_h [H, dh] cos_w [W, dh] sin_w [W, dh]`` with
    ``dh = 2 * (D // 6)`` and ``dt = D - 2 * dh`` -- the split of rope_3d.py:62-66.  The reference caches its
    ``[S, D]`` tables per grid the same way (rope_3d.py:86-97)."""
    T, H, W = (int(v) for v in grid_size)
    device = torch.device(device)
    key = (T, H, W, int(head_dim), float(base), device)
    tab = _TABLES.get(key)
    if tab is None:
        dh = 2 * (head_dim // 6)
        dt = head_dim - 2 * dh
        parts = []
        for n, part in ((T, dt), (H, dh), (W, dh)):
            a = _angles(n, part, base)
            parts += [a.cos().reshape(-1), a.sin().reshape(-1)]
        tab = torch.cat(parts).contiguous()
        g = L.grid_desc((T, H, W), (1, 1, 1))
        want = L.lib().lcbsa_rope_table_floats(ctypes.byref(g), int(head_dim))
        if want != tab.numel():
            raise ValueError(f"rope table for grid {(T, H, W)}, head_dim {head_dim}: {tab.numel()} floats built, library expects {want}")
        tab = tab.to(device)
        _TABLES[key] = tab
    return tab


def norm_rope(x: torch.Tensor, weight: torch.Tensor, grid_size: Sequence[int], eps: float = 1e-6, base: float = 10000.0,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm(x) * weight, then the 3-D rotary embedding, for one ``[B, H, S, D]`` tensor (any B/H/S strides)."""
    if x.dim() != 4:
        raise ValueError("expected a [B, H, S, D] tensor")
    if not L.abi_ok(x):
        x = x.contiguous()
    B, H, S, D = x.shape
    if out is None:
        out = torch.empty(B, H, S, D, dtype=x.dtype, device=x.device)
    w = weight.to(device=x.device, dtype=x.dtype).contiguous()
    if w.numel() != D:
        raise ValueError(f"weight has {w.numel()} elements, head_dim is {D}")
    tab = rope_table(grid_size, D, x.device, base)
    xd, od, g = L.tensor_desc(x), L.tensor_desc(out), L.grid_desc(grid_size, (1, 1, 1))
    with torch.cuda.device(x.device):
        L.check(L.lib().lcbsa_norm_rope(ctypes.byref(xd), ctypes.c_void_p(w.data_ptr()), ctypes.byref(g),
                                        ctypes.c_void_p(tab.data_ptr()), ctypes.c_float(eps), ctypes.byref(od),
                                        L.current_stream(x.device)))
    return out


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, grid_size: Sequence[int],
                 eps: float = 1e-6, base: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``rope_3d(q_norm(q), k_norm(k), grid_size)`` of attention.py:113-121: two launches, one per tensor."""
    return norm_rope(q, q_weight, grid_size, eps, base), norm_rope(k, k_weight, grid_size, eps, base)
