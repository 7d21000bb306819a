"""Times the fused q/k RMSNorm + 3-D rotary kernel on one GPU and prints one JSON line with its HBM roofline.

    python bench_norm_rope.py [--grid 24 48 80] [--heads 32] [--head-dim 128] [--steps 20] [--warmup 3]

A step is the producer of one attention layer: q and k of the fused qkv projection ([B, S, 3, H, D], read through
their strided views) -> two dense [B, H, S, D] outputs, two launches.  Algorithmic bytes per element: 2 read +
2 written (bf16); the angle table and the weights stay in cache.  The inputs (2 x 0.75 GB at the default size) are
larger than the L2, so no flush is needed between steps.  Timed with CUDA events on the launching stream.
"""
from __future__ import annotations

import argparse
import json
import os

import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from longcat_video_b200.modules import rope_3d as R  # noqa: E402

# DRAM bytes per algorithmic byte of one launch, from the ncu capture of this kernel at 8 heads of the same grid
# (188.9 MB read + 142.3 MB written for 377.5 MB); both grow in proportion to the number of heads.
NCU_DRAM_PER_IO_BYTE = 331.2 / 377.5


def _peak_gbs():
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--grid", type=int, nargs=3, default=[24, 48, 80])
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    S, H, D = a.grid[0] * a.grid[1] * a.grid[2], a.heads, a.head_dim
    g = torch.Generator(device=dev).manual_seed(0)
    qkv = torch.randn(1, S, 3, H, D, generator=g, device=dev, dtype=torch.bfloat16)
    q, k, _ = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    wq = torch.ones(D, device=dev, dtype=torch.bfloat16)
    wk = torch.ones(D, device=dev, dtype=torch.bfloat16)
    oq, ok = torch.empty(1, H, S, D, device=dev, dtype=torch.bfloat16), torch.empty(1, H, S, D, device=dev, dtype=torch.bfloat16)

    def step():
        R.norm_rope(q, wq, a.grid, out=oq)
        R.norm_rope(k, wk, a.grid, out=ok)

    for _ in range(max(a.warmup, 3)):
        step()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(a.steps):
        step()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / a.steps
    bytes_per_launch = 4.0 * S * H * D  # 2 B read + 2 B written per element
    achieved = bytes_per_launch / (ms / 2 * 1e-3) / 1e9
    peak, which = _peak_gbs()
    print(json.dumps({
        "kernel": "norm_rope_kernel", "ms_per_step": ms, "launches_per_step": 2, "gpu_launches": 2 * a.steps, "dtype": "bf16",
        "config": {"workload": f"grid {a.grid[0]}x{a.grid[1]}x{a.grid[2]}, {H} heads x {D}", "tokens": S,
                   "l2": "inputs larger than L2"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "peak_source": which, "unit": "GB/s",
                     "frac": achieved / peak, "algorithmic_bytes_per_launch": bytes_per_launch, "traffic": bytes_per_launch * NCU_DRAM_PER_IO_BYTE,
                     "traffic_source": "ncu capture at 8 heads, scaled by bytes"},
    }))


if __name__ == "__main__":
    main()
