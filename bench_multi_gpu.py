"""Multi-GPU leg of ``bench.py``: one attention layer's BSA forward with Ulysses head sharding.

One process per GPU (torchrun), NCCL.  The workload is the SAME seeded tensor at every N: rank r holds the
``[1, H, S/N, D]`` slice of it that the DiT's context-parallel split gives that rank (its part of the H x W plane, all
frames, all heads: ``longcat_video/context_parallel/context_parallel_util.py:84-131``).  The context-parallel op trades
the slices for ``[1, H/N, S, D]`` (all tokens of the rank's heads, sequence rank-major), runs block-select and
block-sparse attention over the rank-major grid ``(N*T, H/sh, W/sw)`` (``longcat_video/modules/attention.py:60-66``) and
trades the result back.  The total work is that of one layer whatever N is ("strong" scaling).

``value`` is timed exactly like the single-GPU leg: eager calls of the public op, CUDA events, barrier and device
synchronisation on both sides, max over ranks; the same call replayed from a CUDA graph is a side figure.  After the
timed region rank 0 checks one head of the result against the CPU oracle run on the gathered rank-major tensors
(``parity`` in the JSON line): the oracle is used as the checker only, never on the timed path.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from longcat_video_b200.synthetic import make_qkv


def rank_shard(x: torch.Tensor, grid, sh: int, sw: int, rank: int) -> torch.Tensor:
    """The tokens of ``x [1, h, T*H*W, D]`` (T,H,W order) that context-parallel rank ``rank`` of an ``sh x sw`` split of
    the H x W plane holds, in its local T,H,W order: ``[1, h, T*(H/sh)*(W/sw), D]``."""
    T, Hh, W = grid
    Hl, Wl = Hh // sh, W // sw
    rh, rw = rank // sw, rank % sw
    _, h, _, D = x.shape
    return x.view(1, h, T, Hh, W, D)[:, :, :, rh * Hl:(rh + 1) * Hl, rw * Wl:(rw + 1) * Wl].reshape(1, h, T * Hl * Wl, D)


def build_shards(wl, heads, sh, sw, rank, keep_head=None):
    """This rank's slices of the seeded full tensors, head by head; also returns the full tensors of ``keep_head``."""
    qs, ks, vs, kept = [], [], [], None
    for hh in range(heads):
        q, k, v = make_qkv(wl, heads=1, head_offset=hh)
        qs.append(rank_shard(q, wl.grid_q, sh, sw, rank))
        ks.append(rank_shard(k, wl.grid_k, sh, sw, rank))
        vs.append(rank_shard(v, wl.grid_k, sh, sw, rank))
        if hh == keep_head:
            kept = (q, k, v)
    return torch.cat(qs, 1).contiguous(), torch.cat(ks, 1).contiguous(), torch.cat(vs, 1).contiguous(), kept


def oracle_parity(wl, kept, sh, sw, world, bsa_grid, out_head, dev, B):
    """Rank 0: head 0 of the N-GPU result against the CPU oracle on the gathered rank-major tensors of the same seed.
    Block lists over the whole head (bit-exact expected), attention on a spread-out sample of query blocks."""
    from oracle import bsa_oracle as O  # checker only; outside every timed region
    try:  # torchrun pins OMP_NUM_THREADS to 1; the oracle's OpenMP loops may use this rank's share of the cores here
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(max(1, (os.cpu_count() or 1) // 2))
    except OSError:
        pass
    q, k, v = (torch.cat([rank_shard(x, wl.grid_k, sh, sw, r) for r in range(world)], dim=2).contiguous() for x in kept)
    ref_idx, ref_cnt, _, _ = O.block_select(q, k, bsa_grid, bsa_grid, wl.sparsity, wl.chunk, wl.chunk)
    idx, cnt = B.get_select_indices(q.to(dev), k.to(dev), bsa_grid, bsa_grid, wl.sparsity, None, wl.chunk, wl.chunk)
    nsel = int(ref_cnt.flatten()[0])
    lists_equal = bool(torch.equal(cnt.cpu(), ref_cnt) and torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel]))
    nq = O.num_blocks(bsa_grid, wl.chunk)
    picks = sorted(set(range(0, nq, max(1, nq // 48))) | {nq - 1})
    masked = torch.zeros_like(ref_cnt)
    masked[..., picks] = ref_cnt[..., picks]
    ref, _ = O.attention(q, k, v, bsa_grid, bsa_grid, wl.chunk, wl.chunk, ref_idx, masked)
    tok = O.token_map(bsa_grid, wl.chunk)[picks].reshape(-1)
    got, want = out_head.float().cpu()[:, :, tok].double(), ref[:, :, tok].double()
    return {"head": 0, "lists_equal": lists_equal, "rel_l2": float((got - want).norm() / want.norm()),
            "max_abs": float((got - want).abs().max()), "query_blocks_checked": len(picks), "against": "CPU oracle on the gathered rank-major grid"}


def run_multi_gpu(args, wl, heads, world, rank, local_rank, peaks, peak_src):
    from longcat_video_b200 import _lib as L
    from longcat_video_b200.block_sparse_attention import bsa_interface as B
    from longcat_video_b200.context_parallel import context_parallel_util as cpu_
    from longcat_video_b200.context_parallel import ulysses_wrapper as U
    from longcat_video_b200.context_parallel.bsa_context_parallel import flash_attn_bsa_3d_ulysses, flash_attn_bsa_3d_ulysses_host

    dev = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=dev)
    cpu_.init_context_parallel(world, rank, world)  # also keeps two SMs free of the attention kernel for the exchange's barrier kernel
    reserve = int(os.environ.get("LCBSA_ATTN_SM_RESERVE", "2"))
    if heads % world:
        raise SystemExit(f"{heads} heads do not split over {world} ranks")
    sh, sw = cpu_.get_optimal_split(world)
    T, Hh, W = wl.grid_k
    if wl.grid_q != wl.grid_k or Hh % sh or W % sw or (Hh // sh) % wl.chunk[1] or (W // sw) % wl.chunk[2]:
        raise SystemExit(f"grid {wl.grid_k} does not split {sh}x{sw} into block-aligned parts; use 720p_legal or 480p_legal")
    bsa_grid = (world * T, Hh // sh, W // sw)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))  # torchrun pins it to 1; the seeded draw is CPU work
    q_c, k_c, v_c, kept = build_shards(wl, heads, sh, sw, rank, keep_head=0 if rank == 0 else None)
    q_h, k_h, v_h = (t.pin_memory() for t in (q_c, k_c, v_c))
    del q_c, k_c, v_c
    q, k, v = (t.to(dev, non_blocking=True) for t in (q_h, k_h, v_h))
    params = dict(sparsity=wl.sparsity, cdf_threshold=None, chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    from longcat_video_b200.context_parallel import bsa_context_parallel as CP
    stages = CP._stages_scattered(heads // world, world) if CP._SCATTER_OUT else U._stages(heads // world, U._heads_per_group(heads // world))
    launches_per_step = 1 + 2 + len(stages)  # pooling (q and k in one launch), score GEMM, top-k, one attention per stage

    def call():
        return flash_attn_bsa_3d_ulysses(q, k, v, bsa_grid, **params)

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    sampler = None
    if rank == 0:
        from longcat_video_b200.clocks import ClockSampler
        sampler = ClockSampler(local_rank)
        sampler.start()
    for _ in range(args.warmup):
        out = call()
    sync()
    L.check(L.lib().lcbsa_check_device_status())
    assert out.shape == q.shape

    nsel = int((1 - wl.sparsity) * ((bsa_grid[0] // wl.chunk[0]) * (bsa_grid[1] // wl.chunk[1]) * (bsa_grid[2] // wl.chunk[2])))
    flops = 4.0 * heads * wl.sq * nsel * (wl.chunk[0] * wl.chunk[1] * wl.chunk[2]) * wl.head_dim  # whole job

    # ---- timed region: K eager calls
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    if sampler:
        sampler.mark_begin()
    start.record()
    for _ in range(args.steps):
        call()
    end.record()
    sync()
    if sampler:
        sampler.mark_end()
    clocks = sampler.stop() if sampler else None
    L.check(L.lib().lcbsa_check_device_status())
    ms_local = start.elapsed_time(end) / args.steps

    # ---- side figure: the same call replayed from a CUDA graph (every rank replays, or none)
    ms_graph_local, graph_note = float("nan"), "off"
    if os.environ.get("LCBSA_BENCH_CUDA_GRAPH", "1") == "1":
        graph = None
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=cap):
                out_graph = call()
            torch.cuda.current_stream().wait_stream(cap)
            g_.replay()
            sync()
            if not torch.equal(out_graph, out):
                raise RuntimeError("the replayed graph does not reproduce the eager result")
            graph, graph_note = g_, "on"
        except Exception as e:  # noqa: BLE001 - a side figure only
            graph_note = f"capture failed: {e!r}"[:200]
            torch.cuda.synchronize()
        ok_all = torch.tensor([1 if graph is not None else 0], device=dev)
        dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
        if int(ok_all) == 1:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            sync()
            a.record()
            for _ in range(args.steps):
                graph.replay()
            b.record()
            sync()
            ms_graph_local = a.elapsed_time(b) / args.steps
        elif graph is not None:
            graph_note = "capture failed on another rank"

    # ---- the attention kernel by itself, on this rank's heads of the gathered tensors (not part of the timed region)
    out = call()
    qg, kg, vg = U.ulysses_a2a_in(q, k, v)
    idx, cnt = B.get_select_indices(qg, kg, bsa_grid, bsa_grid, wl.sparsity, None, wl.chunk, wl.chunk)
    scale = wl.head_dim ** -0.5
    for _ in range(2):
        B.attn_fwd_bsa_varlen(qg, kg, vg, scale, idx, cnt, bsa_grid, bsa_grid, wl.chunk, wl.chunk)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    a0.record()
    for _ in range(args.steps):
        B.attn_fwd_bsa_varlen(qg, kg, vg, scale, idx, cnt, bsa_grid, bsa_grid, wl.chunk, wl.chunk)
    a1.record()
    sync()
    ms_attn_local = a0.elapsed_time(a1) / args.steps
    del qg, kg, vg, idx, cnt
    t = torch.tensor([ms_local, ms_attn_local, ms_graph_local], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_attn, ms_graph = float(t[0]), float(t[1]), float(t[2])

    # ---- parity: head 0 of every rank's result, gathered rank-major on rank 0, against the oracle
    pieces = [torch.empty_like(out[:, 0]) for _ in range(world)] if rank == 0 else None
    dist.gather(out[:, 0].contiguous(), pieces, dst=0)
    parity = None
    if rank == 0 and not args.skip_cpu_baseline:
        out_head = torch.cat(pieces, dim=1).unsqueeze(1)  # [1, 1, N * S/N, D], rank-major
        parity = oracle_parity(wl, kept, sh, sw, world, bsa_grid, out_head, dev, B)

    # ---- end to end: host-resident shards in, host-resident result out, every step, pipelined by head chunk
    e2e = None
    if not args.skip_e2e:
        out_h = torch.empty(q_h.shape, dtype=q_h.dtype).pin_memory()
        hpc = world * max(1, (heads // world) // 4)

        def e2e_step():
            flash_attn_bsa_3d_ulysses_host(q_h, k_h, v_h, bsa_grid, out=out_h, heads_per_chunk=hpc, **params)

        for _ in range(2):
            e2e_step()
        n_e2e = max(3, min(args.steps, 10))
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        s2.record()
        for _ in range(n_e2e):
            e2e_step()
        e2.record()
        sync()
        same = torch.tensor([1 if torch.equal(out_h, out.cpu()) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        t2 = torch.tensor([s2.elapsed_time(e2) / n_e2e], device=dev)
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        es = q.element_size()
        e2e = {"value": flops / float(t2[0]) / 1e9, "unit": "TFLOP/s", "ms_per_step": float(t2[0]),
               "h2d_bytes_per_step": int(q_h.numel() * 3 * es * world), "d2h_bytes_per_step": int(out_h.numel() * es * world),
               "heads_per_chunk": hpc, "equals_device_result": bool(int(same))}

    if rank == 0:
        attn_tf = flops / ms_attn / 1e9
        peak = peaks["bf16_tflops"] * world
        line = {"metric": "bsa_fwd_effective_tflops", "value": flops / ms / 1e9, "unit": "TFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": wl.name, "grid": list(wl.grid_k), "rank_major_grid": list(bsa_grid), "heads": heads,
                           "heads_per_gpu": heads // world, "head_dim": wl.head_dim, "block": list(wl.chunk),
                           "sparsity": wl.sparsity, "selected_blocks": nsel, "algorithmic_tflop": flops / 1e12,
                           "ms_attention_kernels": ms_attn, "cp_split_hw": [sh, sw], "attn_sm_reserve": reserve,
                           "timed_call": "flash_attn_bsa_3d_ulysses, eager", "ms_per_step_cuda_graph": ms_graph if ms_graph == ms_graph else None,
                           "cuda_graph": graph_note, "stages_heads": [hi - lo for lo, hi in stages],
                           "inputs": "every rank holds its context-parallel slice of the one seeded tensor the single-GPU leg uses",
                           "l2": "inputs exceed the 126 MB L2; no flush between iterations",
                           "parallelism": f"ulysses{world} (flash_attn_bsa_3d_ulysses: pooled rows stored straight into their owners' memory, all-to-all in/out by peer DMA copies over NVLink, pipelined by head group)"},
                "roofline": {"bound": "tensor", "kernel": "attn_tc_kernel", "achieved": attn_tf, "peak": peak, "unit": "TFLOP/s",
                             "frac": attn_tf / peak, "peak_source": f"{peak_src} (burst cuBLAS bf16 x {world} GPUs)",
                             "ms_per_step_in_kernel": ms_attn, "traffic": None},
                "parity": parity, "cpu_baseline": None, "e2e": e2e, "clocks": clocks, "gpu_launches": launches_per_step * args.steps}
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()
