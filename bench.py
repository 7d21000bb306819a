"""Benchmark of the BSA forward (block-select + block-sparse attention, plus the Ulysses all-to-all
on more than one GPU) on synthetic tensors of the named workload.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--heads H] [--impl ours|reference]

One step = one attention layer's BSA forward over one batch of inputs.  Rank 0 prints ONE JSON line.
  value      effective TFLOP/s of the whole job (algorithmic flops of the selected blocks / step time) of the public
             entry point ``flash_attn_bsa_3d`` called eagerly on inputs resident in HBM; ms_per_step is ms/layer.
             ``config.ms_per_step_cuda_graph`` is the same call replayed from a CUDA graph (side figure).
  e2e        the same metric through ``flash_attn_bsa_3d_host`` with HOST (pinned) inputs and output: the
             host->device copies of q,k,v and the device->host copy of the result are inside the timing
             (pipelined with the kernels by chunks of two heads).
  N > 1      ``flash_attn_bsa_3d_ulysses`` on every rank's [1, H, S/N, D] slices (bench_multi_gpu.py).
  roofline   the attention kernel against the measured bf16 tensor peak (events around that launch, inside the
             timed region); roofline_select does the same for the block-select stage against the measured HBM rate.
  literal_720p   a short leg on BASELINE's literal 24x45x80 grid (ragged: through ``allow_ragged=True``).
  default_blocks_720p  two short legs on the same tensors with the entry point's default [4, 4, 8] blocks (128 tokens):
             at the headline's sparsity and with every parameter left at its default (sparsity 0.875).
  backward_720p_8heads  side figure: dq, dk, dv of the first 8 heads of the same tensors (lcbsa_attn_bwd), with the headline's
             blocks and with every parameter at its default; bench_backward.py is the benchmark of the backward proper.
  gpu_reference  the reference's own Triton BSA (baseline/_ref, see baseline/install_reference.py) timed on the
             same GPU and inputs, outside the timed region of this library; absent checkout -> "unavailable".
  cpu_baseline  the reference's PyTorch block-select + masked-SDPA path (oracle/reference_path.py) on the
             host cores, on a bounded sample of the same workload.
``--impl reference`` times that CPU path alone (rank 0 only).
Inputs (2.8 GB at 720p) are far larger than the 126 MB L2, so no flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import statistics
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from longcat_video_b200.clocks import ClockSampler  # noqa: E402
from longcat_video_b200.synthetic import WORKLOADS, make_qkv  # noqa: E402

METRIC = "bsa_fwd_effective_tflops"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one attn_tc_kernel launch over the bytes of q, k, v and out, from
# the ncu capture summarised in profiles/attn_tc_kernel_480p_16heads.md (454.0 MB read + 150.7 MB written against
# 654.3 MB).  K and V of a head are re-read from L2, so the traffic of a launch grows with the tensors, not with the
# selected blocks.
NCU_ATTN_DRAM_PER_IO_BYTE = (454.0 + 150.7) / 654.3
# the same for the block-select stage at 720p / 32 heads (profiles/select_kernels_720p_32heads.md): the pool launch
# reads q and k once (1524 MB read, 65 MB written against 1415.6 MB of q and k), the score launch adds 23.6 + 76 MB
# and the top-k launch 135.7 + 8.6 MB (its 16-bit keys no longer fit in L2 at this size).
NCU_SELECT_DRAM_PER_IO_BYTE = (1524.0 + 65.0 + 23.6 + 76.0 + 135.7 + 8.6) / 1415.6

def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def n_selected(sparsity, nk):
    return int((1 - sparsity) * nk)


def is_ragged(wl):
    return any(g % c for grid in (wl.grid_q, wl.grid_k) for g, c in zip(grid, wl.chunk))


def algorithmic_flops(wl, heads, nsel):
    """4 * B * H * Sq * (nsel * block) * D on legal grids; present rows / keys only on ragged ones."""
    ct, ch, cw = wl.chunk
    bs = ct * ch * cw
    if not is_ragged(wl):
        return 4.0 * wl.batch * heads * wl.sq * nsel * bs * wl.head_dim
    return None  # counted from the lists at run time


def _present_per_block(grid, chunk):
    """Number of present tokens of every 3-D block (blocks numbered t-major, then h, then w), as a float64 vector."""
    def axis(n, c):
        nb = -(-n // c)
        return torch.tensor([min(c, n - i * c) for i in range(nb)], dtype=torch.float64)
    t, h, w = (axis(n, c) for n, c in zip(grid, chunk))
    return (t[:, None, None] * h[None, :, None] * w[None, None, :]).reshape(-1)


def flops_from_lists(wl, idx, cnt):
    """Exact count for ragged grids: rows(i) * sum of present keys of the listed blocks."""
    present_q, present_k = _present_per_block(wl.grid_q, wl.chunk), _present_per_block(wl.grid_k, wl.chunk)
    idx_c, cnt_c = idx.cpu().long(), cnt.cpu()
    valid = torch.arange(idx_c.shape[-1])[None, None, None, :] < cnt_c[..., None]
    keys = (present_k[idx_c.clamp_min(0)] * valid).sum(-1)  # [B,H,Nq]
    return float(4.0 * wl.head_dim * (keys * present_q[None, None, :]).sum())


def cpu_reference_arm(wl, steps, warmup, heads_per_step=1):
    """Times the CPU port of the reference path; each step is `heads_per_step` heads of the workload."""
    from oracle.reference_path import bsa_forward_cpu
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v = make_qkv(wl, heads=heads_per_step)
    nsel = n_selected(wl.sparsity, (wl.grid_k[0] // wl.chunk[0]) * (wl.grid_k[1] // wl.chunk[1]) * (wl.grid_k[2] // wl.chunk[2]))
    fl = algorithmic_flops(wl, heads_per_step, nsel)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        bsa_forward_cpu(q, k, v, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return {"value": fl / t / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{heads_per_step} of {wl.heads} heads of {wl.name}, fp32, median of {len(times)} runs ({t * 1e3:.0f} ms each)"}, t


def legal_twin(wl):
    return WORKLOADS["720p_legal"] if is_ragged(wl) else wl


class StepTimer:
    """Times K eager calls of ``flash_attn_bsa_3d`` with an event between its two stages (bsa_interface.STAGE_HOOK)."""

    def __init__(self, B, q, k, v, wl, params):
        self.B, self.q, self.k, self.v, self.wl, self.params = B, q, k, v, wl, params
        self.mids = []

    def call(self):
        return self.B.flash_attn_bsa_3d(self.q, self.k, self.v, self.wl.grid_q, self.wl.grid_k, **self.params)

    def _hook(self):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.mids.append(ev)

    def run(self, steps):
        """-> (ms per step, ms of the block-select stage, ms of the attention launch), means over the steps."""
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        self.mids = []
        self.B.STAGE_HOOK = self._hook
        try:
            torch.cuda.synchronize()
            marks[0].record()
            for i in range(steps):
                self.call()
                marks[i + 1].record()
            torch.cuda.synchronize()
        finally:
            self.B.STAGE_HOOK = None
        ms = marks[0].elapsed_time(marks[steps]) / steps
        ms_sel = statistics.mean(marks[i].elapsed_time(self.mids[i]) for i in range(steps))
        ms_att = statistics.mean(self.mids[i].elapsed_time(marks[i + 1]) for i in range(steps))
        return ms, ms_sel, ms_att

    def run_graph(self, steps):
        """The same call captured once in a CUDA graph and replayed; None if capture is not possible."""
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=cap):
                self.call()
            torch.cuda.current_stream().wait_stream(cap)
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / steps
        except Exception:  # noqa: BLE001 - a side figure only
            torch.cuda.synchronize()
            return None


def gpu_reference_leg(wl, q, k, v, params, flops, steps=5, warmup=2):
    """The reference's Triton BSA on this GPU, same inputs: ms per layer of its ``flash_attn_bsa_3d`` (gating,
    rearranges and kernel, as the DiT calls it).  Its prints are sent to stderr so that stdout stays one JSON line."""
    if is_ragged(wl):
        return {"unavailable": "the reference asserts on grids that do not divide by the block (bsa_interface.py:639-640)"}
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import reference_gpu as R
    except Exception as e:  # noqa: BLE001
        return {"unavailable": f"baseline/reference_gpu.py: {e!r}"[:200]}
    with contextlib.redirect_stdout(sys.stderr):
        if R.load() is None:
            return {"unavailable": R.why(), **R.versions()}
        try:
            for _ in range(warmup):
                out = R.flash_attn_bsa_3d(q, k, v, wl.grid_q, wl.grid_k, **params)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                out = R.flash_attn_bsa_3d(q, k, v, wl.grid_q, wl.grid_k, **params)
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / steps
            del out
        except Exception as e:  # noqa: BLE001 - e.g. a Triton construct this Triton version no longer compiles
            torch.cuda.synchronize()
            return {"unavailable": f"the reference failed on this box: {e!r}"[:400], **R.versions()}
    return {"ms_per_step": ms, "tflops": flops / ms / 1e9, "steps": steps, "what": "reference flash_attn_bsa_3d (Triton), same inputs",
            **R.versions()}


def backward_leg(B, L, q, k, v, wl, heads=8, steps=3, warmup=2):
    """Side figure: the backward (lcbsa_attn_bwd) of the first ``heads`` heads of the tensors on the device, for the lists the
    forward selects; same call sequence as bench_backward.py.  Returns a record, or the reason why there is none."""
    try:
        qs, ks, vs = (t[:, :heads].contiguous() for t in (q, k, v))
        g = torch.Generator().manual_seed(11)
        do = (torch.randn(qs.shape, generator=g) * 0.5).to(qs.dtype).to(qs.device)
        scale = wl.head_dim ** -0.5
        idx, cnt = B.get_select_indices(qs, ks, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
        nsel = int(cnt.flatten()[0])
        o, lse = B.attn_fwd_bsa_varlen(qs, ks, vs, scale, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, return_lse=True)

        def step():
            return B.attn_bwd_bsa_varlen(do, qs, ks, vs, o, lse, scale, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)

        for _ in range(warmup):
            step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        L.check(L.lib().lcbsa_check_device_status())
        ms = a.elapsed_time(b) / steps
        flops = 2.5 * algorithmic_flops(wl, heads, nsel)  # five contractions per (query block, key block) against the forward's two
        return {"workload": wl.name, "heads": heads, "block": list(wl.chunk), "selected_blocks": nsel, "steps": steps, "ms_backward": ms,
                "algorithmic_tflop": flops / 1e12, "backward_tflops": flops / ms / 1e9,
                "what": "dq, dk, dv for the lists of the forward (lcbsa_attn_bwd); bench_backward.py times the reference's Triton backward beside it"}
    except Exception as e:  # noqa: BLE001  (a side figure must not take the headline down)
        return {"unavailable": f"{e!r}"[:300]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="720p_legal", choices=sorted(WORKLOADS))
    ap.add_argument("--heads", type=int, default=None, help="total heads (default: the workload's 32)")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-literal", action="store_true", help="no extra leg on the literal 24x45x80 grid")
    ap.add_argument("--skip-blocks128", action="store_true", help="no extra leg with the default [4, 4, 8] blocks")
    ap.add_argument("--skip-gpu-reference", action="store_true", help="do not time the reference's Triton kernels")
    ap.add_argument("--skip-backward", action="store_true", help="no side figure for the backward")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[args.workload]
    heads = args.heads or wl.heads

    if args.impl == "reference":
        if rank != 0:
            return
        cpu_wl = legal_twin(wl)  # the reference asserts divisibility (bsa_interface.py:639-640)
        base, t = cpu_reference_arm(cpu_wl, args.steps, args.warmup)
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": cpu_wl.name, "grid": list(cpu_wl.grid_k), "heads": 1, "sparsity": cpu_wl.sparsity,
                           "block": list(cpu_wl.chunk), "note": "CPU port of the reference's PyTorch block-select + masked SDPA"},
                "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    from longcat_video_b200 import _lib as L
    from longcat_video_b200.block_sparse_attention import bsa_interface as B

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    peaks, peak_src = load_peaks()

    if world > 1:
        import bench_multi_gpu
        return bench_multi_gpu.run_multi_gpu(args, wl, heads, world, rank, local_rank, peaks, peak_src)

    # ------------------------------------------------------------------ single GPU
    q_h, k_h, v_h = (t.pin_memory() for t in make_qkv(wl, heads=heads))
    q, k, v = (t.to(dev, non_blocking=True) for t in (q_h, k_h, v_h))
    params = dict(sparsity=wl.sparsity, cdf_threshold=None, chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    ragged = is_ragged(wl)
    timer = StepTimer(B, q, k, v, wl, dict(params, allow_ragged=ragged))
    launches_per_step = 4  # pool (q and k in one launch), score GEMM, top-k, attention

    sampler = ClockSampler(local_rank)
    sampler.start()  # nvidia-smi needs a moment to start: long before the timed region
    for _ in range(args.warmup):
        timer.call()
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    idx, cnt = B.get_select_indices(q, k, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    nsel = int(cnt.flatten()[0])
    flops = algorithmic_flops(wl, heads, nsel)
    if flops is None:
        flops = flops_from_lists(wl, idx, cnt)
    del idx, cnt

    sampler.mark_begin()
    ms, ms_select, ms_attn = timer.run(args.steps)
    sampler.mark_end()
    clocks = sampler.stop()
    L.check(L.lib().lcbsa_check_device_status())
    gpu_launches = launches_per_step * args.steps
    ms_graph = timer.run_graph(args.steps)

    es = q.element_size()
    select_bytes = es * wl.batch * heads * (wl.sq + wl.sk) * wl.head_dim  # read Q and K once
    attn_io_bytes = es * wl.batch * heads * (2 * wl.sq + 2 * wl.sk) * wl.head_dim  # q, out, k, v once
    attn_tf = flops / ms_attn / 1e9
    block_tokens = wl.chunk[0] * wl.chunk[1] * wl.chunk[2]
    roofline = {"bound": "tensor", "kernel": "attn_tc128_kernel" if block_tokens == 128 else "attn_tc_kernel",
                "achieved": attn_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": attn_tf / peaks["bf16_tflops"],
                "frac_of_sustained_peak": attn_tf / peaks["bf16_tflops_sustained"],
                "peak_source": f"{peak_src} (burst cuBLAS bf16); sustained {peaks['bf16_tflops_sustained']}",
                "ms_per_launch": ms_attn,
                "traffic": NCU_ATTN_DRAM_PER_IO_BYTE * attn_io_bytes,
                "traffic_source": "ncu capture of 480p_legal/16 heads scaled by the bytes of q,k,v,out"}
    sel_gbs = select_bytes / ms_select / 1e6
    roofline_select = {"bound": "hbm", "kernel": "pool_kernel + score_gemm_kernel + topk_rows_kernel", "achieved": sel_gbs, "peak": peaks["hbm_gbs"],
                       "unit": "GB/s", "frac": sel_gbs / peaks["hbm_gbs"], "peak_source": peak_src, "ms_per_stage": ms_select,
                       "traffic": NCU_SELECT_DRAM_PER_IO_BYTE * select_bytes,
                       "traffic_source": "ncu capture of 720p_legal/32 heads scaled by the bytes of q and k"}

    # ------------------------------------------------------------------ BASELINE's literal 720p grid (ragged), short leg
    literal = None
    if wl.name == "720p_legal" and not args.skip_literal:
        lw = WORKLOADS["720p_ragged"]
        lq, lk, lv = (t.to(dev) for t in make_qkv(lw, heads=heads))
        lt = StepTimer(B, lq, lk, lv, lw, dict(params, allow_ragged=True))
        for _ in range(3):
            lt.call()
        li, lc = B.get_select_indices(lq, lk, lw.grid_q, lw.grid_k, lw.sparsity, None, lw.chunk, lw.chunk)
        lflops = flops_from_lists(lw, li, lc)
        lms, lms_sel, lms_att = lt.run(5)
        L.check(L.lib().lcbsa_check_device_status())
        literal = {"workload": lw.name, "grid": list(lw.grid_k), "steps": 5, "ms_per_step": lms, "ms_select": lms_sel, "ms_attention": lms_att,
                   "algorithmic_tflop": lflops / 1e12, "value": lflops / lms / 1e9, "attention_tflops": lflops / lms_att / 1e9,
                   "attention_frac_of_peak": lflops / lms_att / 1e9 / peaks["bf16_tflops"],
                   "note": "extension: ragged grid through allow_ragged=True, flops counted on present rows and keys only"}
        del lq, lk, lv, lt, li, lc

    # ------------------------------------------------------------------ the entry point's default parameters, short legs
    blocks128 = None
    if wl.name == "720p_legal" and not args.skip_blocks128:
        blocks128 = {}
        # "same_sparsity": only the block shape changes ([4, 4, 8], 45 of 720 blocks: the same keys per query as the
        # headline); "all_defaults": flash_attn_bsa_3d(q, k, v, shape, shape) with nothing else passed (sparsity 0.875)
        for key, wname in (("same_sparsity", "720p_blocks128"), ("all_defaults", "720p_defaults")):
            bw = WORKLOADS[wname]
            bparams = dict(sparsity=bw.sparsity, cdf_threshold=None, chunk_3d_shape_q=list(bw.chunk), chunk_3d_shape_k=list(bw.chunk))
            bt = StepTimer(B, q, k, v, bw, dict(bparams, allow_ragged=False))
            for _ in range(3):
                bt.call()
            bi, bc = B.get_select_indices(q, k, bw.grid_q, bw.grid_k, bw.sparsity, None, bw.chunk, bw.chunk)
            bflops = algorithmic_flops(bw, heads, int(bc.flatten()[0]))
            bms, bms_sel, bms_att = bt.run(5)
            L.check(L.lib().lcbsa_check_device_status())
            leg = {"workload": bw.name, "block": list(bw.chunk), "sparsity": bw.sparsity, "selected_blocks": int(bc.flatten()[0]), "steps": 5,
                   "ms_per_step": bms, "ms_select": bms_sel, "ms_attention": bms_att, "algorithmic_tflop": bflops / 1e12,
                   "value": bflops / bms / 1e9, "attention_tflops": bflops / bms_att / 1e9,
                   "attention_frac_of_peak": bflops / bms_att / 1e9 / peaks["bf16_tflops"], "kernel": "attn_tc128_kernel"}
            if not args.skip_gpu_reference:  # the reference's Triton kernel with BLOCK_M = BLOCK_N = 128 on the same tensors
                bref = gpu_reference_leg(bw, q, k, v, bparams, bflops, steps=3, warmup=2)
                leg["gpu_reference"] = bref
                if "ms_per_step" in bref:
                    leg["speedup_of_this_library"] = bref["ms_per_step"] / bms
            blocks128[key] = leg
            del bt, bi, bc
        blocks128["note"] = "the headline stays on BASELINE's 4x4x4 blocks; these legs run the same tensors with the entry point's default block shape"

    # ------------------------------------------------------------------ backward of 8 heads, side figure
    backward = None
    if wl.name == "720p_legal" and not args.skip_backward:
        backward = {"blocks_4x4x4": backward_leg(B, L, q, k, v, wl), "all_defaults": backward_leg(B, L, q, k, v, WORKLOADS["720p_defaults"])}

    # ------------------------------------------------------------------ the reference's Triton kernels on this GPU
    gpu_reference = None
    if not args.skip_gpu_reference:
        gpu_reference = gpu_reference_leg(wl, q, k, v, params, flops)
        if "ms_per_step" in gpu_reference:
            gpu_reference["speedup_of_this_library"] = gpu_reference["ms_per_step"] / ms

    # ------------------------------------------------------------------ end to end from host buffers
    e2e = None
    if not args.skip_e2e:
        out_h = torch.empty(q_h.shape, dtype=q_h.dtype).pin_memory()

        def e2e_step():
            # host tensors in, host tensor out: copies and kernels pipelined by chunks of two heads
            B.flash_attn_bsa_3d_host(q_h, k_h, v_h, wl.grid_q, wl.grid_k, out=out_h, heads_per_chunk=2,
                                     allow_ragged=ragged, **params)

        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_e2e = max(3, min(args.steps, 10))
        s2.record()
        for _ in range(n_e2e):
            e2e_step()
        e2.record()
        torch.cuda.synchronize()
        ms_e2e = s2.elapsed_time(e2) / n_e2e
        e2e = {"value": flops / ms_e2e / 1e9, "unit": UNIT, "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": int(q_h.numel() + k_h.numel() + v_h.numel()) * es,
               "d2h_bytes_per_step": int(out_h.numel()) * es}

    cpu_baseline = None
    if not args.skip_cpu_baseline:
        cpu_baseline, _ = cpu_reference_arm(legal_twin(wl), steps=3, warmup=1)

    line = {"metric": METRIC, "value": flops / ms / 1e9, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": wl.name, "grid_q": list(wl.grid_q), "grid_k": list(wl.grid_k), "heads": heads,
                       "head_dim": wl.head_dim, "block": list(wl.chunk), "sparsity": wl.sparsity, "selected_blocks": nsel,
                       "algorithmic_tflop": flops / 1e12, "ms_select": ms_select, "ms_attention": ms_attn,
                       "timed_call": "flash_attn_bsa_3d, eager", "ms_per_step_cuda_graph": ms_graph,
                       "l2": "inputs (q,k,v,out) exceed the 126 MB L2; no flush between iterations", "parallelism": "1 GPU",
                       "literal_720p": literal, "default_blocks_720p": blocks128, "backward_720p_8heads": backward},
            "roofline": roofline, "roofline_select": roofline_select, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_reference": gpu_reference, "clocks": clocks, "gpu_launches": gpu_launches}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
