"""Host side of the B200 block-sparse attention: the reference's operator interface over liblcbsa.so.

``flash_attn_bsa_3d`` keeps the name, arguments, defaults and error behaviour of
``longcat_video/block_sparse_attention/bsa_interface.py:612-660`` so that
``longcat_video/modules/attention.py:67`` can call it unchanged.  The stages underneath are
exposed too, named after the reference functions they replace:

  ``mean_pooling_compression_3d``  rearrange_THW_to_3d_block + mean_pooling_compression (:600, :168)
  ``get_select_indices``           cal_score + get_select_indices_topk_from_score (:180, :212, :268)
  ``attn_fwd_bsa_varlen``          attn_fwd_bsa_varlen_triton and the Triton kernels (:290)

All computation happens in the CUDA kernels; PyTorch only allocates outputs and workspaces and
provides the stream.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence, Tuple

import torch

from .. import _lib as L


# A callable that ``flash_attn_bsa_3d`` invokes between its two stages (block-select done, attention not yet
# launched); a profiler or a benchmark sets it to record a CUDA event there.  None: nothing happens.
STAGE_HOOK = None


def _prod(x: Sequence[int]) -> int:
    return int(x[0]) * int(x[1]) * int(x[2])


def num_blocks(latent_shape: Sequence[int], chunk: Sequence[int]) -> int:
    g = L.grid_desc(latent_shape, chunk)
    n = L.lib().lcbsa_num_blocks(ctypes.byref(g))
    if n < 0:
        L.check(n)
    return n


def num_selected(sparsity: float, n_k_blocks: int) -> int:
    """``int((1 - sparsity) * Nk)`` -- bsa_interface.py:214, evaluated in double precision."""
    return int(L.lib().lcbsa_num_selected(float(sparsity), int(n_k_blocks)))


def _as_abi(t: torch.Tensor) -> torch.Tensor:
    return t if L.abi_ok(t) else t.contiguous()


def mean_pooling_compression_3d(x: torch.Tensor, latent_shape, chunk_3d_shape) -> torch.Tensor:
    """Mean over every 3-D block of a T,H,W-ordered ``[B,H,S,D]`` tensor -> ``[B,H,Nblk,D]`` (dtype of x)."""
    x = _as_abi(x)
    B, H, S, D = x.shape
    nb = num_blocks(latent_shape, chunk_3d_shape)
    out = torch.empty(B, H, nb, D, dtype=x.dtype, device=x.device)
    xd, g = L.tensor_desc(x), L.grid_desc(latent_shape, chunk_3d_shape)
    with torch.cuda.device(x.device):
        L.check(L.lib().lcbsa_pool(ctypes.byref(xd), ctypes.byref(g), ctypes.c_void_p(out.data_ptr()),
                                   L.current_stream(x.device)))
    return out


def get_select_indices_from_pooled(q_cmp: torch.Tensor, k_cmp: torch.Tensor, sparsity: float,
                                   cdf_threshold: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block lists from pooled tensors, the three branches of ``get_select_indices`` (bsa_interface.py:268-277):
    ``sparsity`` only: int32 ``idx [B,H,Nq,nsel]`` (ascending) and ``lens [B,H,Nq]``; with ``cdf_threshold``: the whole
    index row sorted by descending softmax weight, ``idx [B,H,Nq,Nk]``, and the number of leading entries to use."""
    if sparsity is None and cdf_threshold is None:
        raise ValueError
    q_cmp, k_cmp = q_cmp.contiguous(), k_cmp.contiguous()
    B, H, Nq, D = q_cmp.shape
    Nk = k_cmp.shape[2]
    if cdf_threshold is not None:
        return _select_cdf(q_cmp, k_cmp, float(cdf_threshold), 0 if sparsity is None else num_selected(sparsity, Nk))
    nsel = num_selected(sparsity, Nk)
    cap = max(nsel, 1)
    idx = torch.empty(B, H, Nq, cap, dtype=torch.int32, device=q_cmp.device)
    cnt = torch.empty(B, H, Nq, dtype=torch.int32, device=q_cmp.device)
    dt = L.dtype_code(q_cmp.dtype)
    keys_bytes = L.lib().lcbsa_score_keys_bytes(dt, B * H, Nq, Nk, D)  # 0: only the fused kernel applies
    ws = torch.empty(max(keys_bytes, 16), dtype=torch.uint8, device=q_cmp.device)
    with torch.cuda.device(q_cmp.device):
        L.check(L.lib().lcbsa_score_topk_ws(q_cmp.data_ptr(), k_cmp.data_ptr(), dt, B * H, Nq, Nk, D, nsel, cap,
                                            idx.data_ptr(), cnt.data_ptr(), ws.data_ptr(), keys_bytes,
                                            L.current_stream(q_cmp.device)))
    return idx, cnt


def get_select_indices_from_pooled_split(q_cmp: torch.Tensor, k_cmp: torch.Tensor, sparsity: float, hw_q: int, period_q: int, split_q: int,
                                         hw_k: int, period_k: int, split_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``get_select_indices_from_pooled`` for a grid with a first part (the conditioning frames; see ``LcbsaSplit`` in
    ``include/lcbsa.h``): query blocks of the first part select among the key blocks of the first part, with the number
    of blocks the reference's separate call on the conditioning tokens would select; all others select among all."""
    q_cmp, k_cmp = q_cmp.contiguous(), k_cmp.contiguous()
    B, H, Nq, D = q_cmp.shape
    Nk = k_cmp.shape[2]
    nk_first = Nk // hw_k // period_k * split_k * hw_k
    nsel, nsel_first = num_selected(sparsity, Nk), num_selected(sparsity, nk_first)
    cap = max(nsel, nsel_first, 1)
    idx = torch.empty(B, H, Nq, cap, dtype=torch.int32, device=q_cmp.device)
    cnt = torch.empty(B, H, Nq, dtype=torch.int32, device=q_cmp.device)
    dt = L.dtype_code(q_cmp.dtype)
    keys_bytes = L.lib().lcbsa_score_keys_bytes(dt, B * H, Nq, Nk, D)
    ws = torch.empty(max(keys_bytes, 16), dtype=torch.uint8, device=q_cmp.device)
    sp = L.LcbsaSplit(hw_q, period_q, split_q, hw_k, period_k, split_k, nsel_first)
    with torch.cuda.device(q_cmp.device):
        L.check(L.lib().lcbsa_score_topk_split(q_cmp.data_ptr(), k_cmp.data_ptr(), dt, B * H, Nq, Nk, D, ctypes.byref(sp), nsel, cap,
                                               idx.data_ptr(), cnt.data_ptr(), ws.data_ptr(), keys_bytes, L.current_stream(q_cmp.device)))
    return idx, cnt


def get_select_indices_split(q, k, latent_shape_q, latent_shape_k, sparsity, chunk_3d_shape_q, chunk_3d_shape_k, period_tq, split_tq,
                             period_tk, split_tk) -> Tuple[torch.Tensor, torch.Tensor]:
    """The whole block-select stage (pool, score, top-k: three launches) for a grid with a first part; periods and
    splits in frame blocks."""
    q, k = _as_abi(q), _as_abi(k)
    B, H, _, D = q.shape
    gq, gk = L.grid_desc(latent_shape_q, chunk_3d_shape_q), L.grid_desc(latent_shape_k, chunk_3d_shape_k)
    nq, nk = num_blocks(latent_shape_q, chunk_3d_shape_q), num_blocks(latent_shape_k, chunk_3d_shape_k)
    hw_k = nk // (-(-int(latent_shape_k[0]) // int(chunk_3d_shape_k[0])))
    nk_first = nk // hw_k // period_tk * split_tk * hw_k
    nsel, nsel_first = num_selected(sparsity, nk), num_selected(sparsity, nk_first)
    cap = max(nsel, nsel_first, 1)
    qd, kd = L.tensor_desc(q), L.tensor_desc(k)
    ws_bytes = L.lib().lcbsa_select_workspace_bytes_fast(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(gq), ctypes.byref(gk))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=q.device)
    idx = torch.empty(B, H, nq, cap, dtype=torch.int32, device=q.device)
    cnt = torch.empty(B, H, nq, dtype=torch.int32, device=q.device)
    with torch.cuda.device(q.device):
        L.check(L.lib().lcbsa_block_select_split(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(gq), ctypes.byref(gk), int(period_tq),
                                                 int(split_tq), int(period_tk), int(split_tk), nsel_first, nsel, cap, idx.data_ptr(),
                                                 cnt.data_ptr(), ws.data_ptr(), ws_bytes, L.current_stream(q.device)))
    return idx, cnt


def _select_cdf(q_cmp: torch.Tensor, k_cmp: torch.Tensor, cdf_threshold: float, nsel_min: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """get_select_indices_cdf / get_select_indices_cdf_topk (bsa_interface.py:226-266) in two launches: scores, then one
    CTA per row for softmax, sort, running sum and count."""
    B, H, Nq, D = q_cmp.shape
    Nk = k_cmp.shape[2]
    dt = L.dtype_code(q_cmp.dtype)
    idx = torch.empty(B, H, Nq, Nk, dtype=torch.int32, device=q_cmp.device)
    cnt = torch.empty(B, H, Nq, dtype=torch.int32, device=q_cmp.device)
    keys_bytes = L.lib().lcbsa_score_keys_bytes(dt, B * H, Nq, Nk, D)
    ws = torch.empty(max(keys_bytes, 16), dtype=torch.uint8, device=q_cmp.device)
    with torch.cuda.device(q_cmp.device):
        L.check(L.lib().lcbsa_score_cdf(q_cmp.data_ptr(), k_cmp.data_ptr(), dt, B * H, Nq, Nk, D, ctypes.c_float(1 / D ** 0.5),
                                        ctypes.c_float(cdf_threshold), int(nsel_min), idx.data_ptr(), cnt.data_ptr(),
                                        ws.data_ptr(), keys_bytes, L.current_stream(q_cmp.device)))
    return idx, cnt


def get_select_indices(q: torch.Tensor, k: torch.Tensor, latent_shape_q, latent_shape_k, sparsity,
                       cdf_threshold=None, chunk_3d_shape_q=(4, 4, 8), chunk_3d_shape_k=(4, 4, 8)
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The whole block-select stage on T,H,W-ordered q and k (pool, score, top-k) in one call."""
    if sparsity is None and cdf_threshold is None:
        raise ValueError
    if cdf_threshold is not None:
        return get_select_indices_from_pooled(mean_pooling_compression_3d(q, latent_shape_q, chunk_3d_shape_q),
                                              mean_pooling_compression_3d(k, latent_shape_k, chunk_3d_shape_k), sparsity, cdf_threshold)
    q, k = _as_abi(q), _as_abi(k)
    B, H, _, D = q.shape
    gq, gk = L.grid_desc(latent_shape_q, chunk_3d_shape_q), L.grid_desc(latent_shape_k, chunk_3d_shape_k)
    nq, nk = num_blocks(latent_shape_q, chunk_3d_shape_q), num_blocks(latent_shape_k, chunk_3d_shape_k)
    nsel = num_selected(sparsity, nk)
    cap = max(nsel, 1)
    qd, kd = L.tensor_desc(q), L.tensor_desc(k)
    ws_bytes = L.lib().lcbsa_select_workspace_bytes_fast(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(gq), ctypes.byref(gk))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=q.device)
    idx = torch.empty(B, H, nq, cap, dtype=torch.int32, device=q.device)
    cnt = torch.empty(B, H, nq, dtype=torch.int32, device=q.device)
    with torch.cuda.device(q.device):
        L.check(L.lib().lcbsa_block_select(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(gq), ctypes.byref(gk), nsel, cap,
                                           idx.data_ptr(), cnt.data_ptr(), ws.data_ptr(), ws_bytes,
                                           L.current_stream(q.device)))
    return idx, cnt


def attn_fwd_bsa_varlen(q, k, v, sm_scale, block_indices, block_indices_lens, latent_shape_q, latent_shape_k,
                        chunk_3d_shape_q, chunk_3d_shape_k, return_lse: bool = False, impl: int = L.ATTN_AUTO, out=None):
    """Block-sparse attention forward over the listed K/V blocks; q/k/v and the result in T,H,W order.  ``out`` may be a
    ``[B,H,Sq,D]`` view (head_dim contiguous, 16-byte strides) to write into."""
    q, k, v = _as_abi(q), _as_abi(k), _as_abi(v)
    B, H, Sq, D = q.shape
    if out is None:
        out = torch.empty(B, H, Sq, D, dtype=q.dtype, device=q.device)
    elif tuple(out.shape) != (B, H, Sq, D) or out.dtype != q.dtype or not L.abi_ok(out):
        raise ValueError("out must be a [B, H, Sq, D] view of the input dtype with 16-byte aligned strides")
    lse = torch.empty(B, H, Sq, dtype=torch.float32, device=q.device) if return_lse else None
    idx = block_indices.to(torch.int32).contiguous()
    cnt = block_indices_lens.to(torch.int32).contiguous()
    gq, gk = L.grid_desc(latent_shape_q, chunk_3d_shape_q), L.grid_desc(latent_shape_k, chunk_3d_shape_k)
    qd, kd, vd, od = L.tensor_desc(q), L.tensor_desc(k), L.tensor_desc(v), L.tensor_desc(out)
    with torch.cuda.device(q.device):
        L.check(L.lib().lcbsa_attn_fwd(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(vd), ctypes.byref(gq), ctypes.byref(gk),
                                       idx.data_ptr(), cnt.data_ptr(), idx.shape[-1], float(sm_scale), ctypes.byref(od),
                                       lse.data_ptr() if lse is not None else None, int(impl),
                                       L.current_stream(q.device)))
    return (out, lse) if return_lse else out


def attn_bwd_bsa_varlen(do, q, k, v, o, lse, sm_scale, block_indices, block_indices_lens, latent_shape_q, latent_shape_k,
                        chunk_3d_shape_q, chunk_3d_shape_k):
    """dq, dk, dv of the block-sparse attention for fixed block lists (``attn_bwd_bsa_varlen_triton`` of the reference,
    longcat_video/block_sparse_attention/bsa_interface.py:343-461).  ``o`` and ``lse`` are what the forward returned."""
    q, k, v, o, do = _as_abi(q), _as_abi(k), _as_abi(v), _as_abi(o), _as_abi(do)
    dq, dk, dv = torch.empty_like(q, memory_format=torch.contiguous_format), torch.empty_like(k, memory_format=torch.contiguous_format), \
        torch.empty_like(v, memory_format=torch.contiguous_format)
    idx = block_indices.to(torch.int32).contiguous()
    cnt = block_indices_lens.to(torch.int32).contiguous()
    lse = lse.to(torch.float32).contiguous()
    gq, gk = L.grid_desc(latent_shape_q, chunk_3d_shape_q), L.grid_desc(latent_shape_k, chunk_3d_shape_k)
    d = {n: L.tensor_desc(t) for n, t in dict(q=q, k=k, v=v, o=o, do=do, dq=dq, dk=dk, dv=dv).items()}
    with torch.cuda.device(q.device):
        need = L.lib().lcbsa_attn_bwd_workspace_bytes(ctypes.byref(d["q"]), ctypes.byref(gq), ctypes.byref(gk), idx.shape[-1])
        ws = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
        L.check(L.lib().lcbsa_attn_bwd(ctypes.byref(d["q"]), ctypes.byref(d["k"]), ctypes.byref(d["v"]), ctypes.byref(d["o"]),
                                       ctypes.byref(d["do"]), ctypes.byref(gq), ctypes.byref(gk), idx.data_ptr(), cnt.data_ptr(),
                                       idx.shape[-1], float(sm_scale), lse.data_ptr(), ctypes.byref(d["dq"]), ctypes.byref(d["dk"]),
                                       ctypes.byref(d["dv"]), ws.data_ptr(), ws.numel(), L.current_stream(q.device)))
    return dq, dk, dv


class _AttentionBSA(torch.autograd.Function):
    """The autograd contract of the reference's ``_attention_bsa`` (bsa_interface.py:535-596): the forward selects the
    blocks and attends to them, the backward differentiates the attention with the lists held fixed."""

    @staticmethod
    def forward(ctx, q, k, v, latent_shape_q, latent_shape_k, sparsity, cdf_threshold, chunk_q, chunk_k, sm_scale):
        idx, cnt = get_select_indices(q, k, latent_shape_q, latent_shape_k, sparsity, cdf_threshold, chunk_q, chunk_k)
        o, lse = attn_fwd_bsa_varlen(q, k, v, sm_scale, idx, cnt, latent_shape_q, latent_shape_k, chunk_q, chunk_k, return_lse=True)
        ctx.save_for_backward(q, k, v, o, lse, idx, cnt)
        ctx.geom = (tuple(latent_shape_q), tuple(latent_shape_k), tuple(chunk_q), tuple(chunk_k), float(sm_scale))
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, idx, cnt = ctx.saved_tensors
        sq, sk, cq, ck, sm_scale = ctx.geom
        dq, dk, dv = attn_bwd_bsa_varlen(do, q, k, v, o, lse, sm_scale, idx, cnt, sq, sk, cq, ck)
        return dq, dk, dv, None, None, None, None, None, None, None


@torch.compiler.disable
def flash_attn_bsa_3d(
    q: torch.Tensor,  # [B, H, Sq, D]
    k: torch.Tensor,  # [B, H, Skv, D]
    v: torch.Tensor,  # [B, H, Skv, D]
    latent_shape_q,
    latent_shape_k,
    # bsa_params
    sparsity=0.875,
    cdf_threshold=None,
    chunk_3d_shape_q=[4, 4, 8],
    chunk_3d_shape_k=[4, 4, 8],
    allow_ragged: bool = False,
) -> torch.Tensor:
    """Drop-in for the reference's ``flash_attn_bsa_3d`` (same positional and keyword arguments).

    ``allow_ragged=True`` (an extension; the reference asserts divisibility) lets T, H, W be any
    size: edge blocks are partial, a partial block is pooled as (sum of present tokens) / block
    size, absent keys take no part in the softmax and absent query rows are not written.
    """
    _, _, Sq, head_dim_q = q.shape
    _, _, Sk, head_dim_k = k.shape
    assert head_dim_q == head_dim_k
    head_dim = head_dim_q
    assert head_dim == v.shape[-1]
    assert head_dim in {16, 32, 64, 128, 256}

    Tq, Hq, Wq = latent_shape_q
    Tk, Hk, Wk = latent_shape_k
    assert Tq * Hq * Wq == Sq
    assert Tk * Hk * Wk == Sk

    tq, hq, wq = chunk_3d_shape_q
    tk, hk, wk = chunk_3d_shape_k
    if not allow_ragged:
        assert Tq % tq == 0 and Hq % hq == 0 and Wq % wq == 0
        assert Tk % tk == 0 and Hk % hk == 0 and Wk % wk == 0

    if sparsity is None and cdf_threshold is None:
        raise ValueError
    if not q.is_cuda:
        raise RuntimeError("flash_attn_bsa_3d (B200) needs CUDA tensors; there is no CPU path")

    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _AttentionBSA.apply(q, k, v, latent_shape_q, latent_shape_k, sparsity, cdf_threshold, chunk_3d_shape_q,
                                   chunk_3d_shape_k, 1 / head_dim ** 0.5)
    idx, cnt = get_select_indices(q, k, latent_shape_q, latent_shape_k, sparsity, cdf_threshold,
                                  chunk_3d_shape_q, chunk_3d_shape_k)
    if STAGE_HOOK is not None:
        STAGE_HOOK()
    return attn_fwd_bsa_varlen(q, k, v, 1 / head_dim ** 0.5, idx, cnt, latent_shape_q, latent_shape_k,
                               chunk_3d_shape_q, chunk_3d_shape_k)


@torch.compiler.disable
def flash_attn_bsa_3d_cond(q, k, v, latent_shape, num_cond_latents, **bsa_params) -> torch.Tensor:
    """The cond / noise split of ``Attention.forward`` (longcat_video/modules/attention.py:124-137) as one op: the first
    ``num_cond_latents`` frames attend among themselves, the remaining frames attend to everything, and the two results
    are one ``[B,H,S,D]`` tensor.  The reference makes contiguous copies of q_cond, k_cond, v_cond and q_noise, calls
    the attention twice and concatenates; here both calls work on views of q, k, v and write into their part of one
    output, so nothing is copied; when the cond frames are whole blocks, q and k are pooled and scored once, one
    selection launch serves both kinds of rows and a single attention launch serves both parts (four launches in all;
    with ``cdf_threshold`` the two selections stay separate).  Bit-identical to the two separate calls.
    ``latent_shape`` is the (T, H, W) of q."""
    T, Hh, W = (int(x) for x in latent_shape)
    B_, H_, S, D = q.shape
    nc = int(num_cond_latents or 0)
    if nc <= 0:
        return flash_attn_bsa_3d(q, k, v, latent_shape, latent_shape, **bsa_params)
    if not 0 < nc < T:
        raise ValueError(f"num_cond_latents {nc} outside (0, {T})")
    assert T * Hh * W == S and k.shape[2] == S and v.shape[2] == S
    sc = nc * Hh * W
    out = torch.empty(B_, H_, S, D, dtype=q.dtype, device=q.device)
    chunk_q = bsa_params.get("chunk_3d_shape_q", [4, 4, 8])
    chunk_k = bsa_params.get("chunk_3d_shape_k", [4, 4, 8])
    sparsity, cdf = bsa_params.get("sparsity", 0.875), bsa_params.get("cdf_threshold", None)
    if not bsa_params.get("allow_ragged", False):
        assert nc % chunk_q[0] == 0 and (T - nc) % chunk_q[0] == 0 and nc % chunk_k[0] == 0 and T % chunk_k[0] == 0
        assert Hh % chunk_q[1] == 0 and W % chunk_q[2] == 0 and Hh % chunk_k[1] == 0 and W % chunk_k[2] == 0
    aligned = nc % chunk_q[0] == 0 and nc % chunk_k[0] == 0 and T % chunk_q[0] == 0 and T % chunk_k[0] == 0
    if (aligned and cdf is None and sparsity is not None and q.dtype in (torch.bfloat16, torch.float16) and D in (64, 128)
            and num_blocks((T, Hh, W), chunk_k) <= 1536):
        # One pass over the whole q and k: pooled once, scored once, and a selection whose rows know which part they
        # belong to (lcbsa_block_select_split); then one attention launch.  Four launches for both parts together.
        idx, cnt = get_select_indices_split(q, k, (T, Hh, W), (T, Hh, W), sparsity, chunk_q, chunk_k, T // chunk_q[0], nc // chunk_q[0],
                                            T // chunk_k[0], nc // chunk_k[0])
        attn_fwd_bsa_varlen(q, k, v, 1 / D ** 0.5, idx, cnt, (T, Hh, W), (T, Hh, W), chunk_q, chunk_k, out=out)
        return out
    parts = ((q[:, :, :sc], sc, out[:, :, :sc], (nc, Hh, W), (nc, Hh, W)),
             (q[:, :, sc:], S, out[:, :, sc:], (T - nc, Hh, W), (T, Hh, W)))
    lists = [get_select_indices(qp, k[:, :, :n], gq, gk, sparsity, cdf, chunk_q, chunk_k) for qp, n, _, gq, gk in parts]
    if nc % chunk_q[0] == 0 and nc % chunk_k[0] == 0:
        # Blocks are numbered frame-major, so the cond blocks are the first blocks of the whole grid on both sides and
        # their lists hold the same numbers there: both parts go through one attention launch over the whole q.
        (idx_c, cnt_c), (idx_n, cnt_n) = lists
        cap = max(idx_c.shape[-1], idx_n.shape[-1])
        nq_c = idx_c.shape[2]
        idx = torch.full((B_, H_, nq_c + idx_n.shape[2], cap), -1, dtype=torch.int32, device=q.device)
        idx[:, :, :nq_c, :idx_c.shape[-1]] = idx_c
        idx[:, :, nq_c:, :idx_n.shape[-1]] = idx_n
        attn_fwd_bsa_varlen(q, k, v, 1 / D ** 0.5, idx, torch.cat([cnt_c, cnt_n], dim=2), (T, Hh, W), (T, Hh, W), chunk_q, chunk_k,
                            out=out)
        return out
    for (qp, n, op, gq, gk), (idx, cnt) in zip(parts, lists):  # ragged split: two launches on views
        attn_fwd_bsa_varlen(qp, k[:, :, :n], v[:, :, :n], 1 / D ** 0.5, idx, cnt, gq, gk, chunk_q, chunk_k, out=op)
    return out


_HOST_STATE = {}


def flash_attn_bsa_3d_host(q, k, v, latent_shape_q, latent_shape_k, out=None, heads_per_chunk=2, device=None, **bsa_params):
    """``flash_attn_bsa_3d`` for tensors that live in (pinned) host memory: q, k, v ``[B, H, S, D]`` on the host in,
    the result on the host out (``out`` is filled and returned if given, else a pinned tensor is allocated).

    An extension without counterpart in the reference (whose op only takes device tensors).  The heads are
    independent, so the call is pipelined by chunks of ``heads_per_chunk`` heads over three streams: while the
    kernels work on chunk c, the copy engines bring in chunk c+1 and take the result of chunk c-1 back, through two
    device staging buffers per tensor.  End to end the call then costs about what moving the bytes over PCIe costs.
    The call returns when the result is complete in ``out``: no further synchronisation is needed to read it.
    """
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise RuntimeError("flash_attn_bsa_3d_host takes host tensors; use flash_attn_bsa_3d for device tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B_, H, Sq, D = q.shape
    Sk = k.shape[2]
    hc = max(1, min(int(heads_per_chunk), H))
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    key = (dev.index, B_, hc, Sq, Sk, D, q.dtype)
    st = _HOST_STATE.get(key)
    if st is None:
        _HOST_STATE.clear()  # one shape at a time: the staging buffers of another shape are dropped
        st = {"q": [torch.empty(B_, hc, Sq, D, dtype=q.dtype, device=dev) for _ in range(2)],
              "k": [torch.empty(B_, hc, Sk, D, dtype=q.dtype, device=dev) for _ in range(2)],
              "v": [torch.empty(B_, hc, Sk, D, dtype=q.dtype, device=dev) for _ in range(2)],
              "h2d": torch.cuda.Stream(device=dev), "d2h": torch.cuda.Stream(device=dev)}
        _HOST_STATE[key] = st
    main = torch.cuda.current_stream(dev)
    h2d, d2h = st["h2d"], st["d2h"]
    h2d.wait_stream(main)
    d2h.wait_stream(main)
    chunks = [(lo, min(lo + hc, H)) for lo in range(0, H, hc)]
    done = []

    def bring(c):
        lo, hi = chunks[c]
        slot = c & 1
        with torch.cuda.stream(h2d):
            if c >= 2:
                h2d.wait_event(done[c - 2])  # the kernels of chunk c-2 are through with this staging buffer
            for name, src in (("q", q), ("k", k), ("v", v)):
                st[name][slot][:, :hi - lo].copy_(src[:, lo:hi], non_blocking=True)
            return h2d.record_event()

    arrived = [bring(0)]
    for c, (lo, hi) in enumerate(chunks):
        if c + 1 < len(chunks):
            # chunk c-1's kernels are already queued, so its `done` event exists when chunk c+1 wants its buffer
            arrived.append(bring(c + 1))
        slot = c & 1
        main.wait_event(arrived[c])
        o = flash_attn_bsa_3d(st["q"][slot][:, :hi - lo], st["k"][slot][:, :hi - lo], st["v"][slot][:, :hi - lo],
                              latent_shape_q, latent_shape_k, **bsa_params)
        done.append(main.record_event())
        o.record_stream(d2h)
        with torch.cuda.stream(d2h):
            d2h.wait_event(done[c])
            out[:, lo:hi].copy_(o, non_blocking=True)
    main.wait_stream(d2h)
    main.wait_stream(h2d)
    # The result is host memory: the caller may read it (and reuse q, k, v) as soon as this returns, so the host
    # itself waits for the copies here; ordering the streams alone would not cover a CPU reader.
    d2h.synchronize()
    h2d.synchronize()
    return out
