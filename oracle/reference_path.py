"""CPU timing port of the reference's "PyTorch block-select + masked SDPA" path.

TEST / BENCHMARK INFRASTRUCTURE ONLY (the shipped package never imports it).  It is what the
benchmark's ``cpu_baseline`` leg and ``bench.py --impl reference`` time on the host cores.

It follows ``longcat_video/block_sparse_attention/bsa_interface.py``:
``rearrange_THW_to_3d_block`` (:600), ``mean_pooling_compression`` (:168), ``cal_score`` (:180),
``get_select_indices_topk_from_score`` (:212) and, for the attention itself, the dense-masked
``scaled_dot_product_attention`` that config 1 of the benchmark names.  An S x S token mask does not
fit in memory at the benchmark's sizes (7.5 GB of bool per head at 720p), so the mask is applied in
its mathematically identical per-query-block form: gather the selected K/V blocks of a query block
and run SDPA on ``[block, nsel*block]``.  fp32 throughout, every host thread torch can use.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def _to_blocks(x, grid, chunk):
    B, H, S, D = x.shape
    T, Hh, W = grid
    t, h, w = chunk
    x = x.view(B, H, T // t, t, Hh // h, h, W // w, w, D).permute(0, 1, 2, 4, 6, 3, 5, 7, 8)
    return x.reshape(B, H, (T // t) * (Hh // h) * (W // w), t * h * w, D)


def _from_blocks(x, grid, chunk):
    B, H, _, _, D = x.shape
    T, Hh, W = grid
    t, h, w = chunk
    x = x.view(B, H, T // t, Hh // h, W // w, t, h, w, D).permute(0, 1, 2, 5, 3, 6, 4, 7, 8)
    return x.reshape(B, H, T * Hh * W, D)


@torch.no_grad()
def bsa_forward_cpu(q, k, v, grid_q, grid_k, sparsity, chunk, q_blocks_per_call: int = 64):
    """q,k,v: CPU ``[B,H,S,D]`` (any float dtype; computed in fp32). Returns fp32 ``[B,H,Sq,D]``."""
    q, k, v = q.float(), k.float(), v.float()
    D = q.shape[-1]
    qb, kb, vb = _to_blocks(q, grid_q, chunk), _to_blocks(k, grid_k, chunk), _to_blocks(v, grid_k, chunk)
    q_cmp, k_cmp = qb.mean(dim=3), kb.mean(dim=3)
    score = torch.matmul(q_cmp, k_cmp.transpose(-1, -2))
    nsel = int((1 - sparsity) * score.shape[-1])
    idx = torch.topk(score, nsel)[1]                       # [B,H,Nq,nsel]
    B, H, Nq, bs, _ = qb.shape
    out = torch.empty_like(qb)
    for b in range(B):
        for h in range(H):
            for i0 in range(0, Nq, q_blocks_per_call):
                sel = idx[b, h, i0:i0 + q_blocks_per_call]               # [n, nsel]
                kg = kb[b, h][sel].reshape(sel.shape[0], nsel * bs, D)   # gathered keys
                vg = vb[b, h][sel].reshape(sel.shape[0], nsel * bs, D)
                out[b, h, i0:i0 + q_blocks_per_call] = F.scaled_dot_product_attention(
                    qb[b, h, i0:i0 + q_blocks_per_call], kg, vg, scale=1.0 / math.sqrt(D))
    return _from_blocks(out, grid_q, chunk)


def algorithmic_flops(heads: int, sq: int, nsel: int, block: int, head_dim: int, batch: int = 1) -> float:
    """QK^T and PV on the selected blocks only: 4 * B * H * Sq * (nsel * block) * D."""
    return 4.0 * batch * heads * sq * nsel * block * head_dim
