"""CPU oracle for the backward of the block-sparse attention.  Test infrastructure only: nothing in the product path
imports it.

What it restates: ``_attention_bsa.backward`` of the reference (longcat_video/block_sparse_attention/
bsa_interface.py:570-596) differentiates the attention of the forward with the block lists held fixed
(``attn_bwd_bsa_varlen_triton``, bsa_interface.py:343-461).  Mathematically that is the gradient of

    o[i] = softmax_j( q[i] . k[j] * sm_scale  over the keys j of the key blocks that query block(i) selected ) v[j]

so the oracle builds the token-level mask from the lists (as ``create_mask_from_indices_varlen``,
bsa_interface.py:131-149, expanded to tokens) and lets autograd differentiate a float64 masked softmax attention.

Pinned on fixtures made from the reference: its backward exists only as Triton kernels, which need a GPU, but the forward
it differentiates has a CPU formulation made of the reference's own functions (block rearrangement, pooling, selection,
``create_mask_from_indices_varlen``) around a masked fp32 ``scaled_dot_product_attention``.  tests/golden/
make_golden_backward.py runs that and lets torch autograd take the gradients; tests/test_oracle_backward.py holds this
oracle to them (rel-L2 3e-7 to 4e-7 on the three fixtures: fp32 against float64 arithmetic).  On a machine with a GPU and
the reference's modules at hand, tests/test_gpu_reference_triton.py also compares this library's gradients with those of
the reference's Triton kernels.
"""
from __future__ import annotations

import torch

from . import bsa_oracle as O


def token_mask(idx: torch.Tensor, cnt: torch.Tensor, grid_q, grid_k, chunk_q, chunk_k) -> torch.Tensor:
    """[B, H, Sq, Sk] bool: query token s may attend to key token t.  ``idx`` [B,H,Nq,cap], ``cnt`` [B,H,Nq]."""
    tq, tk = O.token_map(grid_q, chunk_q), O.token_map(grid_k, chunk_k)  # [Nq, bsq], [Nk, bsk]; -1 = absent
    B, H, Nq, _ = idx.shape
    Sq = grid_q[0] * grid_q[1] * grid_q[2]
    Sk = grid_k[0] * grid_k[1] * grid_k[2]
    mask = torch.zeros(B, H, Sq, Sk, dtype=torch.bool)
    for b in range(B):
        for h in range(H):
            for i in range(Nq):
                rows = tq[i][tq[i] >= 0]
                n = int(cnt[b, h, i])
                if n == 0 or rows.numel() == 0:
                    continue
                keys = tk[idx[b, h, i, :n].long()].reshape(-1)
                keys = keys[keys >= 0]
                mask[b, h, rows[:, None], keys[None, :]] = True
    return mask


def attention_backward(q, k, v, do, idx, cnt, grid_q, grid_k, chunk_q, chunk_k, sm_scale=None):
    """(o, dq, dk, dv) in float64 for inputs of any float dtype (their values are taken as they are)."""
    qd, kd, vd = (t.detach().double().requires_grad_(True) for t in (q, k, v))
    sm_scale = qd.shape[-1] ** -0.5 if sm_scale is None else sm_scale
    mask = token_mask(idx, cnt, grid_q, grid_k, chunk_q, chunk_k)
    s = torch.einsum("bhqd,bhkd->bhqk", qd, kd) * sm_scale
    s = s.masked_fill(~mask, float("-inf"))
    has = mask.any(dim=-1, keepdim=True)
    p = torch.where(has, torch.softmax(torch.where(has, s, torch.zeros_like(s)), dim=-1), torch.zeros_like(s))
    p = torch.where(mask, p, torch.zeros_like(p))  # rows without any key: all zeros, as in the forward
    o = torch.einsum("bhqk,bhkd->bhqd", p, vd)
    (o * do.detach().double()).sum().backward()
    return o.detach(), qd.grad, kd.grad, vd.grad
