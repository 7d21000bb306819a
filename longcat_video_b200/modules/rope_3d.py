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


def _angles(n: int, part: int, base: float, start: int = 0) -> torch.Tensor:
    """Angles of one axis for positions ``start .. start + n - 1``, ``[n, part]``: pair i of the part turns by
    ``pos / base**(2i/part)`` (rope_3d.py:62-84), repeated for both elements of the pair (rope_3d.py:113-115)."""
    inv = 1.0 / (base ** (torch.arange(0, part, 2)[: part // 2].float() / part))
    pos = torch.arange(start, start + n, dtype=torch.float32)
    return torch.repeat_interleave(pos[:, None] * inv[None, :], 2, dim=1)


def rope_table(grid_size: Sequence[int], head_dim: int, device, base: float = 10000.0,
               pos_offset: Sequence[int] = (0, 0, 0)) -> torch.Tensor:
    """The packed separable fp32 table ``lcbsa_norm_rope`` reads, cached per (grid, head_dim, base, offset, device).
    ``pos_offset`` is the (t, h, w) position of the grid's first token: a context-parallel rank that holds rows
    ``h0 ..`` and columns ``w0 ..`` of the frame (the split of rope_3d.py:91-95) passes ``(0, h0, w0)``.  Layout:
    ``cos_t [T, dt] sin_t [T, dt] cos_h [H, dh] sin_h [H, dh] cos_w [W, dh] sin_w [W, dh]`` with
    ``dh = 2 * (D // 6)`` and ``dt = D - 2 * dh`` -- the split of rope_3d.py:62-66.  The reference caches its
    ``[S, D]`` tables per grid the same way (rope_3d.py:86-97)."""
    T, H, W = (int(v) for v in grid_size)
    device = torch.device(device)
    off = tuple(int(v) for v in pos_offset)
    key = (T, H, W, int(head_dim), float(base), off, device)
    tab = _TABLES.get(key)
    if tab is None:
        dh = 2 * (head_dim // 6)
        dt = head_dim - 2 * dh
        parts = []
        for n, part, start in ((T, dt, off[0]), (H, dh, off[1]), (W, dh, off[2])):
            a = _angles(n, part, base, start)
            parts += [a.cos().reshape(-1), a.sin().reshape(-1)]
        tab = torch.cat(parts).contiguous()
        g = L.grid_desc((T, H, W), (1, 1, 1))
        want = L.lib().lcbsa_rope_table_floats(ctypes.byref(g), int(head_dim))
        if want != tab.numel():
            raise ValueError(f"rope table for grid {(T, H, W)}, head_dim {head_dim}: {tab.numel()} floats built, library expects {want}")
        tab = tab.to(device)
        _TABLES[key] = tab
    return tab


def norm_rope(x: torch.Tensor, weight: Optional[torch.Tensor], grid_size: Sequence[int], eps: float = 1e-6, base: float = 10000.0,
              out: Optional[torch.Tensor] = None, rope: bool = True, t_offset: int = 0, table_frames: Optional[int] = None,
              pos_offset: Sequence[int] = (0, 0, 0)) -> torch.Tensor:
    """RMSNorm(x) * weight, then the 3-D rotary embedding, for one ``[B, H, S, D]`` tensor (any B/H/S strides).

    ``weight=None`` skips the normalisation and ``rope=False`` the embedding.  ``t_offset`` places the tensor's first
    frame at frame ``t_offset`` of a table of ``table_frames`` frames (default ``T + t_offset``): the new tokens behind
    cached frames (attention.py:165-169)."""
    if x.dim() != 4:
        raise ValueError("expected a [B, H, S, D] tensor")
    if weight is None and not rope:
        raise ValueError("neither normalisation nor rotary embedding requested")
    if not L.abi_ok(x):
        x = x.contiguous()
    B, H, S, D = x.shape
    if out is None:
        out = torch.empty(B, H, S, D, dtype=x.dtype, device=x.device)
    w_ptr = None
    if weight is not None:
        w = weight.to(device=x.device, dtype=x.dtype).contiguous()
        if w.numel() != D:
            raise ValueError(f"weight has {w.numel()} elements, head_dim is {D}")
        w_ptr = ctypes.c_void_p(w.data_ptr())
    T = int(grid_size[0])
    frames = T + int(t_offset) if table_frames is None else int(table_frames)
    tab_ptr = None
    if rope:
        tab = rope_table((frames, grid_size[1], grid_size[2]), D, x.device, base, pos_offset)
        tab_ptr = ctypes.c_void_p(tab.data_ptr())
    xd, od, g = L.tensor_desc(x), L.tensor_desc(out), L.grid_desc(grid_size, (1, 1, 1))
    with torch.cuda.device(x.device):
        L.check(L.lib().lcbsa_norm_rope_ex(ctypes.byref(xd), w_ptr, ctypes.byref(g), tab_ptr, frames, int(t_offset),
                                           ctypes.c_float(eps), ctypes.byref(od), L.current_stream(x.device)))
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``RMSNorm_FP32`` alone (blocks.py:42-53) on ``[B, H, S, D]``: what ``return_kv`` caches (attention.py:118-119)."""
    return norm_rope(x, weight, (x.shape[2], 1, 1), eps, out=out, rope=False)


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, grid_size: Sequence[int],
                 eps: float = 1e-6, base: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``rope_3d(q_norm(q), k_norm(k), grid_size)`` of attention.py:113-121: two launches, one per tensor."""
    return norm_rope(q, q_weight, grid_size, eps, base), norm_rope(k, k_weight, grid_size, eps, base)


def qk_norm_rope_with_kv_cache(q: torch.Tensor, k: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, k_cache: torch.Tensor,
                               grid_size: Sequence[int], num_cond_latents: int, eps: float = 1e-6, base: float = 10000.0
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The q / k part of ``forward_with_kv_cache`` (attention.py:156-171): returns q ``[B,H,N,D]`` and
    ``k_full [B,H,(NC+T)HW,D]``.  The reference concatenates the cache and the new keys, pads q in front with an empty
    tensor of the cache's size, embeds both over ``(T + NC, H, W)`` and cuts q's tail off again; here the cached keys
    are embedded into the head of ``k_full``, the new keys are normalised and embedded into its tail, and q is
    normalised and embedded at frame offset NC: three launches, no padding and no concatenation."""
    T, Hh, W = (int(v) for v in grid_size)
    nc = int(num_cond_latents)
    B, H, N, D = q.shape
    sc = nc * Hh * W
    if k_cache.shape[0] == 1 and B > 1:  # attention.py:160-162
        k_cache = k_cache.expand(B, -1, -1, -1)
    assert k_cache.shape[2] == sc and N == T * Hh * W
    k_full = torch.empty(B, H, sc + N, D, dtype=k.dtype, device=k.device)
    norm_rope(k_cache, None, (nc, Hh, W), eps, base, out=k_full[:, :, :sc], table_frames=T + nc)
    norm_rope(k, k_weight, grid_size, eps, base, out=k_full[:, :, sc:], t_offset=nc)
    q_out = norm_rope(q, q_weight, grid_size, eps, base, t_offset=nc)
    return q_out, k_full
