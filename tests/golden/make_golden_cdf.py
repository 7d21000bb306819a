"""Fixtures for the cdf_threshold selectors, produced by the reference's own functions on CPU.

Run in a container that has the reference checked out (it is not needed to run the tests):

    PYTHONPATH=<reference checkout>:<this repo> python tests/golden/make_golden_cdf.py

For every case: seeded pooled q/k rows -> ``cal_score`` -> ``get_select_indices_cdf_from_score`` or
``get_select_indices_cdf_topk_from_score`` (longcat_video/block_sparse_attention/bsa_interface.py:180-184, 234-266;
the functions under their ``torch.compile`` decorators, called eagerly).  Stored: the score bits, the softmax
weights the reference sorted (bits), its sorted index rows and its counts.  torch.sort leaves the order of equal
weights open, so the tests compare counts exactly and index rows through the weights they point at.
"""
import os

import numpy as np
import torch

from longcat_video.block_sparse_attention import bsa_interface as R  # the reference

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (seed, heads, Nq, Nk, D, amplitude, dtype, cdf_threshold, sparsity or None)
CASES = {
    "cdf_nk360": (3, 2, 64, 360, 128, 0.6, torch.bfloat16, 0.9, None),
    "cdf_nk360_peaked": (4, 2, 64, 360, 128, 1.2, torch.bfloat16, 0.703, None),
    "cdf_topk_nk1440": (5, 2, 32, 1440, 128, 0.9, torch.bfloat16, 0.5, 0.9375),
    "cdf_nk100_d64_fp16": (6, 3, 48, 100, 64, 1.5, torch.float16, 0.95, None),
    "cdf_topk_nk24": (7, 2, 16, 24, 128, 2.0, torch.bfloat16, 0.3, 0.75),
}


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    for name, (seed, H, Nq, Nk, D, amp, dtype, thr, sparsity) in CASES.items():
        g = torch.Generator().manual_seed(seed)
        q = (torch.randn(1, H, Nq, D, generator=g) * amp).to(dtype)
        k = (torch.randn(1, H, Nk, D, generator=g) * amp).to(dtype)
        score = R.cal_score(q, k)
        scale = 1 / D ** 0.5
        if sparsity is None:
            idx, lens = R.get_select_indices_cdf_from_score.__wrapped__(score, thr, scale)
        else:
            idx, lens = R.get_select_indices_cdf_topk_from_score.__wrapped__(score, sparsity, thr, scale)
        w = torch.softmax(score * scale, dim=-1)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, q=bits(q), k=bits(k), score=bits(score), weights=bits(w), idx=idx.numpy().astype(np.int16),
                            lens=lens.numpy().astype(np.int32), meta=np.array([H, Nq, Nk, D, int(dtype == torch.float16)]),
                            params=np.array([thr, -1.0 if sparsity is None else sparsity, scale]))
        print(name, int(lens.min()), int(lens.max()), os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    main()
