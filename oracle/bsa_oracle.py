"""ctypes front end of the CPU oracle (``bsa_oracle.c``).

TEST INFRASTRUCTURE ONLY: the shipped package never imports this module.  It is used by
the tests, by the smoke check and by the CPU-baseline leg of the benchmark.

The C file restates the reference's block-select and block-sparse attention forward
(``longcat_video/block_sparse_attention/bsa_interface.py:168-224, 600-660`` and
``flash_attn_bsa_varlen_mask.py:172-285``); this module only marshals tensors.

All tensors are torch CPU tensors shaped ``[B, H, S, D]`` in the latent grid's T,H,W
token order, dtype bfloat16, float16 or float32.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence, Tuple

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "bsa_oracle.c")
_OUT_DIR = os.path.join(_HERE, "_build")
_SO = os.path.join(_OUT_DIR, "libbsa_oracle.so")

_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


class _Grid(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("T", "H", "W", "ct", "ch", "cw")]


def build(force: bool = False) -> str:
    """Compile ``bsa_oracle.c`` into ``oracle/_build/libbsa_oracle.so`` with gcc."""
    if not force and os.path.exists(_SO) and os.path.getmtime(_SO) >= os.path.getmtime(_SRC):
        return _SO
    os.makedirs(_OUT_DIR, exist_ok=True)
    cmd = ["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
           "-o", _SO, _SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.lco_num_blocks.restype = ctypes.c_int
        _lib.lco_token_of.restype = ctypes.c_int64
    return _lib


def _grid(latent_shape: Sequence[int], chunk: Sequence[int]) -> _Grid:
    return _Grid(int(latent_shape[0]), int(latent_shape[1]), int(latent_shape[2]),
                 int(chunk[0]), int(chunk[1]), int(chunk[2]))


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    assert t.device.type == "cpu" and t.is_contiguous()
    return ctypes.c_void_p(t.data_ptr())


def num_blocks(latent_shape, chunk) -> int:
    g = _grid(latent_shape, chunk)
    return int(lib().lco_num_blocks(ctypes.byref(g)))


def num_selected(sparsity: float, n_k_blocks: int) -> int:
    """``int((1 - sparsity) * Nk)`` in Python floats (bsa_interface.py:214)."""
    return int((1 - sparsity) * n_k_blocks)


def token_map(latent_shape, chunk) -> torch.Tensor:
    """int64 ``[Nblk, block_size]``: T,H,W-order token of each block slot, -1 where absent."""
    g = _grid(latent_shape, chunk)
    nb = num_blocks(latent_shape, chunk)
    bs = int(chunk[0]) * int(chunk[1]) * int(chunk[2])
    out = torch.empty(nb, bs, dtype=torch.int64)
    L = lib()
    for b in range(nb):
        for r in range(bs):
            out[b, r] = L.lco_token_of(ctypes.byref(g), b, r)
    return out


def pool(x: torch.Tensor, latent_shape, chunk) -> torch.Tensor:
    """Mean-pool every 3-D block: ``[B,H,S,D] -> [B,H,Nblk,D]`` in the dtype of ``x``."""
    B, H, S, D = x.shape
    assert S == latent_shape[0] * latent_shape[1] * latent_shape[2] and D <= 512
    x = x.contiguous()
    g = _grid(latent_shape, chunk)
    nb = num_blocks(latent_shape, chunk)
    out = torch.empty(B, H, nb, D, dtype=x.dtype)
    lib().lco_pool(_ptr(x), _DTYPE_CODE[x.dtype], B * H, ctypes.byref(g), D, _ptr(out))
    return out


def score(q_cmp: torch.Tensor, k_cmp: torch.Tensor) -> torch.Tensor:
    """Block scores ``q_cmp @ k_cmp^T``: ``[B,H,Nq,D],[B,H,Nk,D] -> [B,H,Nq,Nk]`` (input dtype)."""
    B, H, Nq, D = q_cmp.shape
    Nk = k_cmp.shape[2]
    q_cmp, k_cmp = q_cmp.contiguous(), k_cmp.contiguous()
    out = torch.empty(B, H, Nq, Nk, dtype=q_cmp.dtype)
    lib().lco_score(_ptr(q_cmp), _ptr(k_cmp), _DTYPE_CODE[q_cmp.dtype], B * H, Nq, Nk, D, _ptr(out))
    return out


def topk(score_: torch.Tensor, nsel: int, cap: Optional[int] = None
         ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-row top-``nsel``: returns (idx int32 ``[B,H,Nq,cap]`` ascending, -1 padded;
    cnt int32 ``[B,H,Nq]``; boundary_ties int32 ``[B,H,Nq]``)."""
    B, H, Nq, Nk = score_.shape
    cap = max(nsel, 1) if cap is None else cap
    assert 0 <= nsel <= Nk and cap >= nsel
    score_ = score_.contiguous()
    idx = torch.empty(B, H, Nq, cap, dtype=torch.int32)
    cnt = torch.empty(B, H, Nq, dtype=torch.int32)
    ties = torch.empty(B, H, Nq, dtype=torch.int32)
    lib().lco_topk(_ptr(score_), _DTYPE_CODE[score_.dtype], B * H, Nq, Nk, nsel, cap,
                   _ptr(idx), _ptr(cnt), _ptr(ties))
    return idx, cnt, ties


def cdf_select(score_: torch.Tensor, cdf_threshold: float, sm_scale: float, nsel_min: int = 0
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The cdf_threshold selectors of bsa_interface.py:234-266 on bf16 / fp16 scores ``[B,H,Nq,Nk]``: returns the whole
    index row sorted by descending softmax weight (int32 ``[B,H,Nq,Nk]``; ties by ascending index) and the number of
    leading entries to use (int32 ``[B,H,Nq]``), at least ``nsel_min`` (the combined "max(cdf, topk)" selector)."""
    B, H, Nq, Nk = score_.shape
    assert score_.dtype in (torch.bfloat16, torch.float16) and 0 < Nk <= 4096
    score_ = score_.contiguous()
    idx = torch.empty(B, H, Nq, Nk, dtype=torch.int32)
    cnt = torch.empty(B, H, Nq, dtype=torch.int32)
    lib().lco_cdf_select(_ptr(score_), _DTYPE_CODE[score_.dtype], ctypes.c_int64(B * H * Nq), Nk, ctypes.c_float(sm_scale),
                         ctypes.c_float(cdf_threshold), int(nsel_min), _ptr(idx), _ptr(cnt))
    return idx, cnt


def block_select(q, k, latent_shape_q, latent_shape_k, sparsity, chunk_q, chunk_k, cap=None):
    """pool -> score -> top-k (the ``sparsity``-only branch of bsa_interface.py:268-277)."""
    qc = pool(q, latent_shape_q, chunk_q)
    kc = pool(k, latent_shape_k, chunk_k)
    sc = score(qc, kc)
    nsel = num_selected(sparsity, kc.shape[2])
    idx, cnt, ties = topk(sc, nsel, cap)
    return idx, cnt, ties, sc


def attention(q, k, v, latent_shape_q, latent_shape_k, chunk_q, chunk_k, idx, cnt,
              sm_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact-softmax attention over the listed K/V blocks; fp32 ``out [B,H,Sq,D]`` and
    natural-log ``lse [B,H,Sq]``."""
    B, H, Sq, D = q.shape
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    idx, cnt = idx.contiguous(), cnt.contiguous()
    assert idx.dtype == torch.int32 and cnt.dtype == torch.int32
    if sm_scale is None:
        sm_scale = 1.0 / D ** 0.5
    gq, gk = _grid(latent_shape_q, chunk_q), _grid(latent_shape_k, chunk_k)
    out = torch.zeros(B, H, Sq, D, dtype=torch.float32)
    lse = torch.zeros(B, H, Sq, dtype=torch.float32)
    lib().lco_attn(_ptr(q), _ptr(k), _ptr(v), _DTYPE_CODE[q.dtype], B * H, ctypes.byref(gq),
                   ctypes.byref(gk), D, _ptr(idx), _ptr(cnt), idx.shape[-1],
                   ctypes.c_float(sm_scale), _ptr(out), _ptr(lse))
    return out, lse


def flash_attn_bsa_3d(q, k, v, latent_shape_q, latent_shape_k, sparsity=0.875, cdf_threshold=None,
                      chunk_3d_shape_q=(4, 4, 8), chunk_3d_shape_k=(4, 4, 8)):
    """Whole forward with the reference's signature (bsa_interface.py:612-623); fp32 result."""
    if sparsity is None and cdf_threshold is None:
        raise ValueError
    if cdf_threshold is not None:  # bsa_interface.py:271-274
        qc, kc = pool(q, latent_shape_q, chunk_3d_shape_q), pool(k, latent_shape_k, chunk_3d_shape_k)
        nsel_min = 0 if sparsity is None else num_selected(sparsity, kc.shape[2])
        idx, cnt = cdf_select(score(qc, kc), cdf_threshold, 1 / q.shape[-1] ** 0.5, nsel_min)
        out, _ = attention(q, k, v, latent_shape_q, latent_shape_k, chunk_3d_shape_q, chunk_3d_shape_k, idx, cnt)
        return out
    idx, cnt, _, _ = block_select(q, k, latent_shape_q, latent_shape_k, sparsity,
                                  chunk_3d_shape_q, chunk_3d_shape_k)
    out, _ = attention(q, k, v, latent_shape_q, latent_shape_k, chunk_3d_shape_q, chunk_3d_shape_k,
                       idx, cnt)
    return out


if __name__ == "__main__":
    print(build(force=True))


def rope_tables(grid_size, head_dim: int, base: float = 10000.0):
    """fp32 ``cos, sin [T*H*W, head_dim]`` of the reference's 3-D rotary embedding
    (``longcat_video/modules/rope_3d.py:60-97, 113-115``): the head dimension is split into a T part of
    ``D - 4*(D//6)`` and H and W parts of ``2*(D//6)`` elements; within a part, pair i of the elements turns by
    ``position / base**(2i/part)``; every angle is repeated for the two elements of its pair."""
    T, H, W = grid_size
    d_h = d_w = 2 * (head_dim // 6)
    d_t = head_dim - d_h - d_w

    def angles(n, part):
        inv = 1.0 / (base ** (torch.arange(0, part, 2)[: part // 2].float() / part))
        pos = torch.arange(n, dtype=torch.float32)
        return torch.repeat_interleave(pos[:, None] * inv[None, :], 2, dim=1)  # [n, part]

    at, ah, aw = angles(T, d_t), angles(H, d_h), angles(W, d_w)
    full = torch.cat([at[:, None, None, :].expand(T, H, W, d_t), ah[None, :, None, :].expand(T, H, W, d_h),
                      aw[None, None, :, :].expand(T, H, W, d_w)], dim=-1).reshape(T * H * W, head_dim)
    return full.cos().contiguous(), full.sin().contiguous()


def norm_rope(x: torch.Tensor, weight: Optional[torch.Tensor], cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
              eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm (fp32) + weight + 3-D rotary embedding of ``x [B, H, S, D]`` (any strides, D contiguous); dense result.
    ``weight=None`` skips the normalisation, ``cos=sin=None`` the embedding (the halves the KV-cache path uses)."""
    B, H, S, D = x.shape
    assert D % 16 == 0 and x.stride(3) == 1 and (weight is not None or cos is not None)
    xc = x.contiguous()
    out = torch.empty(B, H, S, D, dtype=x.dtype)
    w = None if weight is None else weight.to(x.dtype).contiguous()
    if cos is not None:
        assert cos.shape == (S, D) and sin.shape == (S, D)
        cos, sin = cos.float().contiguous(), sin.float().contiguous()
    null = ctypes.c_void_p(None)
    lib().lco_norm_rope(ctypes.c_void_p(xc.data_ptr()), ctypes.c_int64(D), _DTYPE_CODE[x.dtype], ctypes.c_int64(B * H * S), D,
                        ctypes.c_int64(S), null if w is None else ctypes.c_void_p(w.data_ptr()),
                        null if cos is None else ctypes.c_void_p(cos.data_ptr()), null if cos is None else ctypes.c_void_p(sin.data_ptr()),
                        ctypes.c_float(eps), ctypes.c_void_p(out.data_ptr()))
    return out
