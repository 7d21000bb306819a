"""Times the cdf_threshold selector (score_gemm_kernel + cdf_rows kernel) on one GPU and prints one JSON line.

    python bench_select_cdf.py [--blocks 1440] [--heads 32] [--threshold 0.5]

A step is the selection of one attention layer from pooled rows ([1, H, N, 128] bf16, seeded random): N x N block
scores per head, then per row softmax, sort, running sum and count.  Algorithmic bytes of the row kernel: 2 read +
4 written per score.  It is not HBM-bound (a sorting network per row); the roofline entry says how far it is from
the HBM rate.  Timed with CUDA events on the launching stream; scores and index rows are larger than the L2.
"""
from __future__ import annotations

import argparse
import json
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from longcat_video_b200.block_sparse_attention import bsa_interface as B  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", type=int, default=1440)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--threshold", type=float, default=0.5)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(5)
    H, N, D = a.heads, a.blocks, 128
    q = (torch.randn(1, H, N, D, generator=g, device=dev) * 0.8).bfloat16()
    k = (torch.randn(1, H, N, D, generator=g, device=dev) * 0.8).bfloat16()
    for _ in range(max(a.warmup, 3)):
        idx, cnt = B.get_select_indices_from_pooled(q, k, None, a.threshold)
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(a.steps):
        idx, cnt = B.get_select_indices_from_pooled(q, k, None, a.threshold)
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / a.steps
    scores = float(H) * N * N
    here = os.path.dirname(os.path.abspath(__file__))
    try:
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            peak, which = float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        peak, which = 6650.0, "fallback"
    achieved = (2 + 2 + 4) * scores / (ms * 1e-3) / 1e9  # keys written, keys read, index rows written
    print(json.dumps({
        "kernels": ["score_gemm_kernel", "cdf_rows_fast_kernel"], "ms_per_step": ms, "launches_per_step": 2,
        "gpu_launches": 2 * a.steps, "dtype": "bf16", "rows_per_s": H * N / (ms * 1e-3),
        "config": {"workload": f"{H} heads x {N} x {N} block scores, threshold {a.threshold}", "mean_selected": float(cnt.float().mean()),
                   "l2": "scores and index rows larger than L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "peak_source": which, "unit": "GB/s", "frac": achieved / peak,
                     "note": "both kernels together; the row kernel is bound by its sorting network, not by HBM"},
    }))


if __name__ == "__main__":
    main()
