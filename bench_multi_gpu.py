"""Multi-GPU leg of ``bench.py``: one attention layer's BSA forward with Ulysses head sharding.

One process per GPU (torchrun), NCCL.  Every rank starts with its ``[1, H, S/N, D]`` slice of q, k, v
(the layout the DiT has under context parallelism), the decorated attention function trades them for
``[1, H/N, S, D]`` with the all-to-all, runs block-select + block-sparse attention on its heads over the
rank-major grid ``(N*T, H/sh, W/sw)`` (``longcat_video/modules/attention.py:60-66``), and trades the result
back.  The total work is that of one layer whatever N is ("strong" scaling).
"""
from __future__ import annotations

import json
import os
import statistics

import torch
import torch.distributed as dist

from ..synthetic import Workload, make_qkv


def run_multi_gpu(args, wl, heads, world, rank, local_rank, peaks, peak_src, attn_impl):
    from .. import _lib as L
    from ..block_sparse_attention import bsa_interface as B
    from . import context_parallel_util as cpu_
    from .ulysses_wrapper import ulysses_wrapper

    dev = torch.device("cuda", local_rank)
    # The attention kernel fills every SM it is given; the exchange runs on the copy engines, but its barrier is a
    # one-CTA kernel that must be able to start beside the attention: keep two SMs free.
    reserve = int(os.environ.get("LCBSA_ATTN_SM_RESERVE", "2"))
    dist.init_process_group("nccl", device_id=dev)
    if L.lib().lcbsa_set_attn_sm_reserve(reserve) < 0:
        L.check(-1)
    cpu_.init_context_parallel(world, rank, world)
    if heads % world:
        raise SystemExit(f"{heads} heads do not split over {world} ranks")
    sh, sw = cpu_.get_optimal_split(world)
    T, Hh, W = wl.grid_k
    if wl.grid_q != wl.grid_k or Hh % sh or W % sw or (Hh // sh) % wl.chunk[1] or (W // sw) % wl.chunk[2]:
        raise SystemExit(f"grid {wl.grid_k} does not split {sh}x{sw} into block-aligned parts; use 720p_legal or 480p_legal")
    local_grid = (T, Hh // sh, W // sw)
    bsa_grid = (world * T, Hh // sh, W // sw)
    local = Workload(wl.name + f"_rank{rank}", wl.seed + 17 * rank, 1, heads, wl.head_dim, local_grid, local_grid, wl.chunk,
                     wl.sparsity, wl.dtype, wl.recipe)
    q_h, k_h, v_h = (t.pin_memory() for t in make_qkv(local))
    q, k, v = (t.to(dev, non_blocking=True) for t in (q_h, k_h, v_h))
    params = dict(sparsity=wl.sparsity, cdf_threshold=None, chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    scale = wl.head_dim ** -0.5
    launches = {"n": 0}

    from .bsa_context_parallel import flash_attn_bsa_3d_ulysses

    class Layer:
        # the context-parallel op: local pooling, pooled rows exchanged first, block-select of all local heads while
        # the first slabs travel, attention by head group with the exchange on the copy engines
        def attn(self, q_, k_, v_, shape):
            launches["n"] += 2 + 2 + len(_stage_list)  # two pool launches, score GEMM, top-k, one attention per stage
            return flash_attn_bsa_3d_ulysses(q_, k_, v_, shape, **params)

    from . import ulysses_wrapper as U
    _stage_list = U._stages(heads // world, U._heads_per_group(heads // world))
    layer = Layer()

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        out = layer.attn(q, k, v, bsa_grid)
    sync()
    L.check(L.lib().lcbsa_check_device_status())
    assert out.shape == q.shape

    nsel = int((1 - wl.sparsity) * ((bsa_grid[0] // wl.chunk[0]) * (bsa_grid[1] // wl.chunk[1]) * (bsa_grid[2] // wl.chunk[2])))
    flops = 4.0 * heads * (wl.sq) * nsel * (wl.chunk[0] * wl.chunk[1] * wl.chunk[2]) * wl.head_dim  # whole job

    # One layer of a fixed shape is what a DiT repeats dozens of times per step: the whole call (pooling, copies,
    # barriers, block-select, attention stages) is captured once in a CUDA graph and replayed, which takes the host out
    # of the loop (at 8 GPUs the eager call costs the host about as much time as it costs the GPU).
    # LCBSA_BENCH_CUDA_GRAPH=0 times the eager call instead.
    graph, graph_note = None, "off"
    if os.environ.get("LCBSA_BENCH_CUDA_GRAPH", "1") == "1":
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=cap):
                out_graph = layer.attn(q, k, v, bsa_grid)
            torch.cuda.current_stream().wait_stream(cap)
            g_.replay()
            sync()
            if not torch.equal(out_graph, out):
                raise RuntimeError("the replayed graph does not reproduce the eager result")
            graph, graph_note = g_, "on"
        except Exception as e:  # noqa: BLE001 - capture is an optimisation: fall back to the eager call
            graph_note = f"capture failed, eager: {e!r}"[:200]
            torch.cuda.synchronize()
    ok_all = torch.tensor([1 if graph is not None else 0], device=dev)
    dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)  # every rank replays, or every rank runs eagerly
    if int(ok_all) == 0:
        graph = None
    stage_launches = 2 + 2 + len(_stage_list)

    sampler = None
    if rank == 0:
        from ..clocks import ClockSampler
        sampler = ClockSampler(local_rank)
        sampler.start()
    launches["n"] = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    start.record()
    for _ in range(args.steps):
        if graph is not None:
            graph.replay()
            launches["n"] += stage_launches
        else:
            layer.attn(q, k, v, bsa_grid)
    end.record()
    sync()
    clocks = sampler.stop() if sampler else None
    timed_launches = launches["n"]
    L.check(L.lib().lcbsa_check_device_status())
    ms_local = start.elapsed_time(end) / args.steps
    # the attention kernel by itself, on this rank's heads of the gathered tensors (not part of the timed region)
    qg, kg, vg = U.ulysses_a2a_in(q, k, v)
    idx, cnt = B.get_select_indices(qg, kg, bsa_grid, bsa_grid, wl.sparsity, None, wl.chunk, wl.chunk)
    for _ in range(2):
        B.attn_fwd_bsa_varlen(qg, kg, vg, scale, idx, cnt, bsa_grid, bsa_grid, wl.chunk, wl.chunk, impl=attn_impl)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    a0.record()
    for _ in range(args.steps):
        B.attn_fwd_bsa_varlen(qg, kg, vg, scale, idx, cnt, bsa_grid, bsa_grid, wl.chunk, wl.chunk, impl=attn_impl)
    a1.record()
    sync()
    ms_attn_local = a0.elapsed_time(a1) / args.steps
    del qg, kg, vg
    t = torch.tensor([ms_local, ms_attn_local], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_attn = float(t[0]), float(t[1])

    # end to end: host-resident shards in, host-resident result out, every step
    e2e = None
    if not args.skip_e2e:
        out_h = torch.empty(q_h.shape, dtype=q_h.dtype).pin_memory()
        qd, kd, vd = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

        def e2e_step():
            qd.copy_(q_h, non_blocking=True)
            kd.copy_(k_h, non_blocking=True)
            vd.copy_(v_h, non_blocking=True)
            out_h.copy_(layer.attn(qd, kd, vd, bsa_grid), non_blocking=True)

        e2e_step()
        n_e2e = max(3, min(args.steps, 10))
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        s2.record()
        for _ in range(n_e2e):
            e2e_step()
        e2.record()
        sync()
        t2 = torch.tensor([s2.elapsed_time(e2) / n_e2e], device=dev)
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        es = q.element_size()
        e2e = {"value": flops / float(t2[0]) / 1e9, "unit": "TFLOP/s", "ms_per_step": float(t2[0]),
               "h2d_bytes_per_step": int(q_h.numel() * 3 * es * world), "d2h_bytes_per_step": int(out_h.numel() * es * world)}

    if rank == 0:
        attn_tf = flops / ms_attn / 1e9
        peak = peaks["bf16_tflops"] * world
        line = {"metric": "bsa_fwd_effective_tflops", "value": flops / ms / 1e9, "unit": "TFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": wl.name, "grid": list(wl.grid_k), "rank_major_grid": list(bsa_grid), "heads": heads,
                           "heads_per_gpu": heads // world, "head_dim": wl.head_dim, "block": list(wl.chunk),
                           "sparsity": wl.sparsity, "selected_blocks": nsel, "algorithmic_tflop": flops / 1e12,
                           "ms_attention_kernels": ms_attn, "cp_split_hw": [sh, sw], "attn_sm_reserve": reserve, "cuda_graph": graph_note if graph is None else "on",
                           "l2": "inputs exceed the 126 MB L2; no flush between iterations",
                           "parallelism": f"ulysses{world} (flash_attn_bsa_3d_ulysses: pooled rows exchanged first, all-to-all in/out by peer DMA copies over NVLink, pipelined by head group)"},
                "roofline": {"bound": "tensor", "kernel": "attn_tc_kernel", "achieved": attn_tf, "peak": peak, "unit": "TFLOP/s",
                             "frac": attn_tf / peak, "peak_source": f"{peak_src} (burst cuBLAS bf16 x {world} GPUs)",
                             "ms_per_step_in_kernel": ms_attn, "traffic": None},
                "cpu_baseline": None, "e2e": e2e, "clocks": clocks, "gpu_launches": timed_launches}
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
