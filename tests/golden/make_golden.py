"""Generate the golden fixtures in this folder by running the REFERENCE's own PyTorch code on CPU.

Run once, in a container that has the reference checkout (it cannot travel to the GPU box):

    PYTHONPATH=<reference checkout> TORCH_COMPILE_DISABLE=1 PYTHONDONTWRITEBYTECODE=1 \
        python tests/golden/make_golden.py

For every case the script draws seeded inputs (``longcat_video_b200.synthetic``), pushes
them through the reference's functions
(``longcat_video/block_sparse_attention/bsa_interface.py``: ``rearrange_THW_to_3d_block``
:600, ``mean_pooling_compression`` :168, ``cal_score`` :180, ``get_select_indices`` :268,
``create_mask_from_indices_varlen`` :131, ``rearrange_3d_block_to_THW`` :606) and, for the
attention result, through ``torch.nn.functional.scaled_dot_product_attention`` in fp32 with
the block mask expanded to tokens -- the "PyTorch block-select + masked SDPA" path.  The
reference's Triton kernels need a GPU and are not run.

Outputs are stored as ``.npz`` (bf16 values as their uint16 bit patterns).
"""
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from longcat_video_b200.synthetic import Workload, make_qkv  # noqa: E402,F401
from tests.golden.cases import CASES  # noqa: E402
from longcat_video.block_sparse_attention import bsa_interface as R  # noqa: E402  (the reference)



def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def run_reference(wl: Workload, store_attention: bool):
    q, k, v = make_qkv(wl)
    D = wl.head_dim
    (Tq, Hq, Wq), (Tk, Hk, Wk), (ct, ch, cw) = wl.grid_q, wl.grid_k, wl.chunk
    bs = ct * ch * cw
    qb = R.rearrange_THW_to_3d_block(q, Tq // ct, Hq // ch, Wq // cw, ct, ch, cw, D)
    kb = R.rearrange_THW_to_3d_block(k, Tk // ct, Hk // ch, Wk // cw, ct, ch, cw, D)
    vb = R.rearrange_THW_to_3d_block(v, Tk // ct, Hk // ch, Wk // cw, ct, ch, cw, D)
    q_cmp = R.mean_pooling_compression(qb, bs)
    k_cmp = R.mean_pooling_compression(kb, bs)
    score = R.cal_score(q_cmp, k_cmp)
    idx, lens = R.get_select_indices(q_cmp, k_cmp, wl.sparsity, None)
    out = {
        "checksum": np.array([q.double().sum().item(), k.double().sum().item(), v.double().sum().item()]),
        "q_cmp": bits(q_cmp), "k_cmp": bits(k_cmp), "score": bits(score),
        "idx": idx.numpy().astype(np.int16), "lens": lens.numpy().astype(np.int32),
    }
    if not store_attention:
        del out["score"]  # 1320 x 1320: too large to commit; the index lists carry the tie information
    if store_attention:
        nk = k_cmp.shape[2]
        bmask = R.create_mask_from_indices_varlen(idx, nk)  # [B,H,Nq,Nk] bool
        tmask = bmask.repeat_interleave(bs, dim=2).repeat_interleave(bs, dim=3)
        o = F.scaled_dot_product_attention(qb.float(), kb.float(), vb.float(), attn_mask=tmask,
                                           scale=1.0 / D ** 0.5)
        o = R.rearrange_3d_block_to_THW(o, Tq // ct, Hq // ch, Wq // cw, ct, ch, cw, D)
        out["attn"] = o.numpy().astype(np.float32)
    return out


def main():
    torch.manual_seed(0)
    for name, (wl, store_attention) in CASES.items():
        res = run_reference(wl, store_attention)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **res)
        print(name, {k_: v_.shape for k_, v_ in res.items()}, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
