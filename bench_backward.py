"""Timing of the backward of the block-sparse attention (``lcbsa_attn_bwd``) on synthetic tensors of a named workload.

    python bench_backward.py [--workload 480p_legal] [--heads 8] [--steps 5] [--warmup 2] [--skip-gpu-reference]

Prints one JSON line: ms of the forward and of the backward of this library (CUDA events), the effective TFLOP/s of the
backward on the selected blocks (five contractions per (query block, key block) pair: 10 * B * H * Sq * nsel * block * D
flop), and -- when the reference's modules are under ``baseline/_ref`` -- the same through the reference's autograd
function and Triton kernels on the same tensors.  Side benchmark: the headline of this repository is ``bench.py``.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from longcat_video_b200.synthetic import WORKLOADS, make_qkv  # noqa: E402


def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="480p_legal", choices=sorted(WORKLOADS))
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--skip-gpu-reference", action="store_true")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_backward.py needs a CUDA device")
    from longcat_video_b200 import _lib as L
    from longcat_video_b200.block_sparse_attention import bsa_interface as B

    wl = WORKLOADS[args.workload]
    q, k, v = (t.cuda() for t in make_qkv(wl, heads=args.heads))
    g = torch.Generator().manual_seed(11)
    do = (torch.randn(q.shape, generator=g) * 0.5).to(q.dtype).cuda()
    scale = wl.head_dim ** -0.5
    idx, cnt = B.get_select_indices(q, k, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    nsel = int(cnt.flatten()[0])
    bs = wl.chunk[0] * wl.chunk[1] * wl.chunk[2]
    fwd_flops = 4.0 * wl.batch * args.heads * wl.sq * nsel * bs * wl.head_dim
    o, lse = B.attn_fwd_bsa_varlen(q, k, v, scale, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, return_lse=True)
    ms_fwd = _time(lambda: B.attn_fwd_bsa_varlen(q, k, v, scale, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, return_lse=True),
                   args.steps, args.warmup)
    ms_bwd = _time(lambda: B.attn_bwd_bsa_varlen(do, q, k, v, o, lse, scale, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk),
                   args.steps, args.warmup)
    L.check(L.lib().lcbsa_check_device_status())
    # delta, four list-transposition kernels, two passes; the tcgen05 passes add the per-block lse/delta layout and, for
    # blocks above 64 tokens, the rewriting of the lists per 64-token unit
    tc = wl.head_dim == 128 and os.environ.get("LCBSA_BWD_IMPL") != "mma"
    launches = 7 + (1 if tc else 0) + ((2 if bs == 128 else 1) if tc and bs > 64 else 0)  # 128-token blocks: one rewriting per pass
    line = {"bench": "bsa_backward", "workload": wl.name, "heads": args.heads, "block": list(wl.chunk), "selected_blocks": nsel,
            "dtype": "bf16", "data": "synthetic", "steps": args.steps, "warmup": args.warmup,
            "ms_forward_attention": ms_fwd, "ms_backward": ms_bwd, "backward_tflops": 2.5 * fwd_flops / ms_bwd / 1e9,
            "forward_tflops": fwd_flops / ms_fwd / 1e9, "gpu_launches_per_backward": launches}
    if not args.skip_gpu_reference:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_gpu as R
        with contextlib.redirect_stdout(sys.stderr):
            m = R.load()
        if m is None:
            line["gpu_reference"] = {"unavailable": R.why()}
        else:
            try:
                params = dict(sparsity=wl.sparsity, cdf_threshold=None, chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
                qr, kr, vr = (t.detach().clone().requires_grad_(True) for t in (q, k, v))

                def ref_step():
                    with contextlib.redirect_stdout(sys.stderr):
                        out = m.flash_attn_bsa_3d(qr, kr, vr, wl.grid_q, wl.grid_k, **params)
                        out.backward(do)
                    qr.grad = kr.grad = vr.grad = None

                def ref_fwd():
                    with contextlib.redirect_stdout(sys.stderr), torch.no_grad():
                        m.flash_attn_bsa_3d(qr, kr, vr, wl.grid_q, wl.grid_k, **params)

                ms_both = _time(ref_step, args.steps, args.warmup)
                ms_f = _time(ref_fwd, args.steps, args.warmup)
                line["gpu_reference"] = {"ms_forward_and_backward": ms_both, "ms_forward": ms_f, "ms_backward": ms_both - ms_f,
                                         "what": "reference flash_attn_bsa_3d + autograd (Triton), same inputs", **R.versions()}
            except Exception as e:  # noqa: BLE001
                torch.cuda.synchronize()
                line["gpu_reference"] = {"unavailable": f"the reference failed on this box: {e!r}"[:400]}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
