"""The self-attention layer between its two linear projections, as single calls on this library's ops.

Stands in for the body of ``Attention.forward`` and ``Attention.forward_with_kv_cache``
(``longcat_video/modules/attention.py:107-147`` and ``149-181``) from the point where q, k, v are the ``[B, H, N, D]``
views of the fused qkv projection (``qkv.view(B, N, 3, H, D).permute(2, 0, 3, 1, 4).unbind(0)``, attention.py:113-115)
up to the ``[B, H, N, D]`` attention result the layer transposes and projects (attention.py:139-142).  The views go in
as they are: the RMSNorm + rotary producer and the block-sparse attention read strided tensors, so nothing is made
contiguous, padded or concatenated except v behind its cache.  All arithmetic is in liblcbsa.so; there is no CPU path.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from ..block_sparse_attention.bsa_interface import flash_attn_bsa_3d, flash_attn_bsa_3d_cond
from .rope_3d import norm_rope, qk_norm_rope_with_kv_cache, rms_norm


def self_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                   shape: Sequence[int], bsa_params: dict, num_cond_latents: Optional[int] = None, return_kv: bool = False,
                   eps: float = 1e-6):
    """``Attention.forward`` between the projections (attention.py:116-137): q/k RMSNorm, 3-D rotary embedding over
    ``shape`` = (T, H, W), then the block-sparse attention -- with ``num_cond_latents`` the first that many frames attend
    among themselves and the rest to everything (attention.py:124-135), as one op on views.  ``return_kv`` also returns
    what the layer caches for video continuation: the normalised, not yet embedded k and a copy of v
    (attention.py:118-119).  Returns ``x [B, H, N, D]`` or ``(x, (k_cache, v_cache))``."""
    shape = tuple(int(s) for s in shape)
    kv = None
    if return_kv:
        kv = (rms_norm(k, k_weight, eps), v.clone())
    q_e = norm_rope(q, q_weight, shape, eps)
    k_e = norm_rope(k, k_weight, shape, eps)
    if num_cond_latents is not None and num_cond_latents > 0:
        x = flash_attn_bsa_3d_cond(q_e, k_e, v, shape, num_cond_latents, **bsa_params)
    else:
        x = flash_attn_bsa_3d(q_e, k_e, v, shape, shape, **bsa_params)
    return (x, kv) if return_kv else x


def self_attention_with_kv_cache(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                                 shape: Sequence[int], kv_cache: Tuple[torch.Tensor, torch.Tensor], bsa_params: dict,
                                 num_cond_latents: int, eps: float = 1e-6) -> torch.Tensor:
    """``Attention.forward_with_kv_cache`` between the projections (attention.py:156-173): the ``T`` new frames of
    ``shape`` = (T, H, W) attend to the ``num_cond_latents`` cached frames and to themselves.  The cached keys (stored
    normalised, attention.py:118-119) are embedded at frames ``0 .. NC-1`` into the head of one key buffer, the new keys
    are normalised and embedded at frames ``NC ..`` into its tail, q is embedded at ``NC ..`` without the padding the
    reference puts in front of it (attention.py:166-169), and the attention runs with ``Tq = T`` query frames against
    ``Tk = T + NC`` key frames.  A cache of batch 1 serves every batch entry (attention.py:159-162).  The reference
    defines the concatenated k, v only when ``num_cond_latents > 0`` (attention.py:164-169); any other value is refused
    here.  Returns ``x [B, H, N, D]``."""
    T, Hh, W = (int(s) for s in shape)
    nc = int(num_cond_latents or 0)
    if nc <= 0:
        raise ValueError("forward_with_kv_cache needs num_cond_latents > 0 (the cached frames)")
    k_cache, v_cache = kv_cache
    B, H, N, D = q.shape
    sc = nc * Hh * W
    if k_cache.shape[0] != v_cache.shape[0] or k_cache.shape[0] not in (1, B):
        raise ValueError(f"cache batch {k_cache.shape[0]} / {v_cache.shape[0]} against batch {B}")
    if N != T * Hh * W or k_cache.shape[2] != sc or v_cache.shape[2] != sc:
        raise ValueError(f"{N} new tokens and {k_cache.shape[2]} cached ones do not match shape {(T, Hh, W)} with {nc} cached frames")
    q_e, k_full = qk_norm_rope_with_kv_cache(q, k, q_weight, k_weight, k_cache, (T, Hh, W), nc, eps)
    v_full = torch.empty(B, H, sc + N, D, dtype=v.dtype, device=v.device)
    v_full[:, :, :sc].copy_(v_cache if v_cache.shape[0] == B else v_cache.expand(B, -1, -1, -1))
    v_full[:, :, sc:].copy_(v)
    return flash_attn_bsa_3d(q_e, k_full, v_full, (T, Hh, W), (T + nc, Hh, W), **bsa_params)
