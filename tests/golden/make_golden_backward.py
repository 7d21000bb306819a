"""Generate the backward fixtures by differentiating the REFERENCE's own PyTorch path on CPU.

Run once, in a container that has the reference checkout:

    PYTHONPATH=<reference checkout> TORCH_COMPILE_DISABLE=1 PYTHONDONTWRITEBYTECODE=1 \
        python tests/golden/make_golden_backward.py

The reference's backward exists only as Triton kernels, which need a GPU.  What it computes is the gradient of its
forward with the block lists held fixed (``_attention_bsa.backward``, longcat_video/block_sparse_attention/
bsa_interface.py:570-596), and that forward has a CPU formulation made of the reference's own functions: seeded inputs
go through ``rearrange_THW_to_3d_block`` (:600), ``mean_pooling_compression`` (:168), ``get_select_indices`` (:268) and
``create_mask_from_indices_varlen`` (:131); the block mask, expanded to tokens, masks
``torch.nn.functional.scaled_dot_product_attention`` in fp32, and torch autograd differentiates that call with respect to
q, k and v (the mask is a constant: no gradient flows through the selection).  The gradients go back to T,H,W order
through ``rearrange_3d_block_to_THW`` (:606) and are stored in fp32 beside the lists they were computed for.
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from longcat_video_b200.synthetic import make_qkv  # noqa: E402
from tests.golden.cases import BWD_CASES, make_dout  # noqa: E402
from longcat_video.block_sparse_attention import bsa_interface as R  # noqa: E402  (the reference)


def run_reference(wl):
    q, k, v = make_qkv(wl)
    do = make_dout(wl)
    D = wl.head_dim
    (Tq, Hq, Wq), (Tk, Hk, Wk), (ct, ch, cw) = wl.grid_q, wl.grid_k, wl.chunk
    bs = ct * ch * cw
    nq3, nk3 = (Tq // ct, Hq // ch, Wq // cw), (Tk // ct, Hk // ch, Wk // cw)
    qb = R.rearrange_THW_to_3d_block(q, *nq3, ct, ch, cw, D)
    kb = R.rearrange_THW_to_3d_block(k, *nk3, ct, ch, cw, D)
    vb = R.rearrange_THW_to_3d_block(v, *nk3, ct, ch, cw, D)
    dob = R.rearrange_THW_to_3d_block(do, *nq3, ct, ch, cw, D)
    q_cmp, k_cmp = R.mean_pooling_compression(qb, bs), R.mean_pooling_compression(kb, bs)
    idx, lens = R.get_select_indices(q_cmp, k_cmp, wl.sparsity, None)
    bmask = R.create_mask_from_indices_varlen(idx, k_cmp.shape[2])
    tmask = bmask.repeat_interleave(bs, dim=2).repeat_interleave(bs, dim=3)
    qf, kf, vf = (t.float().detach().requires_grad_(True) for t in (qb, kb, vb))
    o = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=tmask, scale=1.0 / D ** 0.5)
    o.backward(dob.float())
    dq = R.rearrange_3d_block_to_THW(qf.grad, *nq3, ct, ch, cw, D)
    dk = R.rearrange_3d_block_to_THW(kf.grad, *nk3, ct, ch, cw, D)
    dv = R.rearrange_3d_block_to_THW(vf.grad, *nk3, ct, ch, cw, D)
    return {
        "checksum": np.array([q.double().sum().item(), k.double().sum().item(), v.double().sum().item(), do.double().sum().item()]),
        "idx": idx.numpy().astype(np.int16), "lens": lens.numpy().astype(np.int32),
        "dq": dq.numpy().astype(np.float32), "dk": dk.numpy().astype(np.float32), "dv": dv.numpy().astype(np.float32),
    }


def main():
    torch.manual_seed(0)
    for name, wl in BWD_CASES.items():
        res = run_reference(wl)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **res)
        print(name, {k_: v_.shape for k_, v_ in res.items()}, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
