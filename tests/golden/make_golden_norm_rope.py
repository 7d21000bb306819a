"""Generate ``norm_rope_*.npz`` by running the REFERENCE's own modules on CPU.

    PYTHONPATH=<reference checkout> PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_norm_rope.py

Seeded qkv activations (bf16, the ``[B, N, 3, H, D]`` output layout of the fused qkv projection) and seeded norm
weights go through ``RMSNorm_FP32`` (``longcat_video/modules/blocks.py:42-53``, eps 1e-6 as in
``longcat_video/modules/attention.py:40-41``) and ``RotaryPositionalEmbedding`` (``longcat_video/modules/rope_3d.py``)
exactly as ``Attention.forward`` chains them (``attention.py:113-121``).  Stored: the inputs' bit patterns, the weights,
the reference's q and k (bf16 bit patterns), the normalised q and k before the embedding (what ``return_kv`` caches,
``attention.py:118-119``), and the KV-cache flow of ``forward_with_kv_cache`` (``attention.py:156-171``) with ``NC``
cached frames: cached keys (normalised, not embedded), then ``rope_3d`` over ``(T + NC, H, W)`` on
``cat([k_cache, k_norm(k)])`` and on q padded in front, of which the last N tokens are kept.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from longcat_video.modules.blocks import RMSNorm_FP32  # noqa: E402  (the reference)
from longcat_video.modules.rope_3d import RotaryPositionalEmbedding  # noqa: E402  (the reference)

NC = 2  # cached frames in the KV-cache flow

CASES = {
    # name: (seed, B, heads, head_dim, grid)
    "norm_rope_d128": (501, 1, 3, 128, (4, 6, 10)),
    "norm_rope_d64_b2": (502, 2, 2, 64, (3, 4, 8)),
}


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    for name, (seed, B, H, D, grid) in CASES.items():
        g = torch.Generator().manual_seed(seed)
        N = grid[0] * grid[1] * grid[2]
        qkv = (torch.randn(B, N, 3, H, D, generator=g) * 1.5).to(torch.bfloat16)
        wq = (1.0 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16)
        wk = (1.0 + 0.2 * torch.randn(D, generator=g)).to(torch.bfloat16)
        q, k, _ = qkv.permute(2, 0, 3, 1, 4).unbind(0)  # [B, H, N, D] views, as attention.py:113-115
        qn, kn = RMSNorm_FP32(D, eps=1e-6), RMSNorm_FP32(D, eps=1e-6)
        with torch.no_grad():
            qn.weight.data = wq.clone()
            kn.weight.data = wk.clone()
            rope = RotaryPositionalEmbedding(D, cp_split_hw=(1, 1))
            q1, k1 = qn(q), kn(k)
            q2, k2 = rope(q1, k1, grid)
            # forward_with_kv_cache: keys of NC earlier frames, cached after k_norm and before rope_3d
            kc_raw = (torch.randn(B, H, NC * grid[1] * grid[2], D, generator=g) * 1.5).to(torch.bfloat16)
            k_cache = kn(kc_raw)
            k_full = torch.cat([k_cache, k1], dim=2).contiguous()
            q_padding = torch.cat([torch.zeros_like(k_cache), q1], dim=2).contiguous()
            q_padding, k_full = rope(q_padding, k_full, (grid[0] + NC, grid[1], grid[2]))
            q_kv = q_padding[:, :, -N:].contiguous()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), qkv=bits(qkv), wq=bits(wq), wk=bits(wk), q=bits(q2), k=bits(k2),
                            q_normed=bits(q1), k_normed=bits(k1), k_cache=bits(k_cache), q_kv=bits(q_kv), k_full=bits(k_full),
                            grid=np.array(grid), meta=np.array([seed, B, H, D]))
        print(name, tuple(q2.shape), q2.dtype)


if __name__ == "__main__":
    main()
