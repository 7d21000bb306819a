"""Block-sparse attention under Ulysses context parallelism as ONE op.

``Attention._process_attn`` of the reference (``longcat_video/modules/attention.py:49-67``) is
``ulysses_wrapper(flash_attn_bsa_3d)``: all-to-all, then pool + score + top-k + attention on the gathered tensors,
then all-to-all back.  ``flash_attn_bsa_3d_ulysses`` computes the same result (bit for bit) in a different order:

  1. every rank mean-pools the 3-D blocks of ITS tokens for all heads (blocks never straddle ranks: the gathered
     sequence is rank-major and the grid is split along T); the pooling kernel stores each head's rows -- 1/64 of
     the bytes -- straight into the memory of the rank that owns the head (``lcbsa_pool_scatter``), so the pooled
     tensors of the gathered sequence exist after one kernel and one barrier, while the first q, k, v slabs travel;
  2. the block lists of all the rank's heads are selected in one launch while the first q, k, v slabs are still on
     their way;
  3. the attention runs stage by stage over head groups, each stage's q, k, v arriving by peer DMA during the stage
     before and its result leaving during the stage after (``peer_exchange``).

Against the generic wrapper this takes the block-select off the critical path and out of the small per-stage
launches.  It falls back to ``ulysses_wrapper(flash_attn_bsa_3d)`` whenever its preconditions do not hold.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..block_sparse_attention import bsa_interface as B
from . import context_parallel_util, peer_exchange
from . import ulysses_wrapper as U


_PHASES = os.environ.get("LCBSA_CP_PHASES", "0") == "1"
_SCATTER_OUT = os.environ.get("LCBSA_CP_SCATTER_OUT", "1") == "1"


class _PhaseTimer:
    """CUDA events between the phases of a call on the main stream (LCBSA_CP_PHASES=1, for profiling).  Nothing is
    synchronised while calls run; ``phase_report()`` reads the events of all calls made so far."""
    calls = []

    def __init__(self, stream):
        self.stream, self.names, self.events = stream, [], [stream.record_event(torch.cuda.Event(enable_timing=True))]
        _PhaseTimer.calls.append(self)

    def mark(self, name):
        self.names.append(name)
        self.events.append(self.stream.record_event(torch.cuda.Event(enable_timing=True)))


def phase_report(skip: int = 0) -> str:
    """Mean milliseconds per phase over the recorded calls (the first ``skip`` left out), plus the mean distance between
    the starts of consecutive calls; clears the record."""
    torch.cuda.synchronize()
    calls = _PhaseTimer.calls[skip:]
    _PhaseTimer.calls = []
    if not calls:
        return "no calls recorded"
    names = calls[0].names
    means = [sum(c.events[i].elapsed_time(c.events[i + 1]) for c in calls) / len(calls) for i in range(len(names))]
    total = sum(c.events[0].elapsed_time(c.events[-1]) for c in calls) / len(calls)
    period = (calls[0].events[0].elapsed_time(calls[-1].events[0]) / (len(calls) - 1)) if len(calls) > 1 else float("nan")
    return ", ".join(f"{n} {m:.3f}" for n, m in zip(names, means)) + f", total {total:.3f}, period {period:.3f} ms over {len(calls)} calls"


def _stages_scattered(hn: int, n: int = 2):
    """Head ranges of the attention stages when the result leaves through the kernel's own stores: only the FIRST stage
    has to be small (its q, k, v slabs are the ones nothing can hide); every further launch costs a pipeline fill and a
    tail.  On two or four GPUs a head's slabs arrive two to three times faster than its attention runs, so the rest goes
    in at most two large stages.  On eight the slabs are eight times smaller (3 MB copies reach about half the link rate)
    and a head's slabs take three quarters of its attention time: a stage of three heads then waits half a millisecond
    for its slabs, so the heads go one by one."""
    if "LCBSA_ULYSSES_GROUP_HEADS" in os.environ:
        return U._stages(hn, U._heads_per_group(hn))
    if hn <= 1:
        sizes = [hn]
    elif n >= 8:
        sizes = [1] * min(hn, 4) + [2] * ((hn - 4) // 2 if hn > 4 else 0) + ([1] if hn > 4 and (hn - 4) % 2 else [])
    elif hn <= 4:
        sizes = [1, hn - 1]
    elif hn <= 8:
        sizes = [1, 3, hn - 4]
    else:
        sizes = [2, 6, hn - 8]
    out, lo = [], 0
    for sz in sizes:
        out.append((lo, lo + sz))
        lo += sz
    return out


def _generic(q, k, v, latent_shape, params, latent_shape_q=None):
    class _Layer:
        @U.ulysses_wrapper
        def attn(self, q_, k_, v_, shape):
            return B.flash_attn_bsa_3d(q_, k_, v_, latent_shape_q or shape, shape, **params)

    return _Layer().attn(q, k, v, latent_shape)


def _generic_cond(q, k, v, latent_shape, nc, n, params):
    """The reference's formulation of the conditioning split under context parallelism
    (longcat_video/modules/attention.py:124-137): two exchanges and two attention calls on copies, concatenated."""
    T, Hh, Ww = latent_shape
    sc = nc * Hh * Ww
    x_cond = _generic(q[:, :, :sc].contiguous(), k[:, :, :sc].contiguous(), v[:, :, :sc].contiguous(), (n * nc, Hh, Ww), params)
    x_noise = _generic(q[:, :, sc:].contiguous(), k, v, latent_shape, params, latent_shape_q=(T - n * nc, Hh, Ww))
    return torch.cat([x_cond, x_noise], dim=2)


@torch.compiler.disable
def flash_attn_bsa_3d_ulysses(q, k, v, latent_shape, sparsity=0.875, cdf_threshold=None, chunk_3d_shape_q=[4, 4, 8],
                              chunk_3d_shape_k=[4, 4, 8], num_cond_latents=None):
    """``q, k, v``: this rank's ``[B, H, S/N, D]`` slices (all heads, its tokens); ``latent_shape``: the rank-major
    grid ``(N*T, H', W')`` of the gathered sequence, as ``_process_attn`` receives it.  Returns ``[B, H, S/N, D]``.

    ``num_cond_latents`` (video continuation, longcat_video/modules/attention.py:124-137): the first that many frames of
    every rank's tokens are conditioning frames, which attend among themselves, while the others attend to everything.
    The reference runs two exchanges and two attention calls on copies; here it is still ONE exchange and one attention
    launch per stage: the selection kernel knows which rows belong to which part.  Same bits as the two calls."""
    n = context_parallel_util.get_cp_size()
    params = dict(sparsity=sparsity, cdf_threshold=cdf_threshold, chunk_3d_shape_q=list(chunk_3d_shape_q),
                  chunk_3d_shape_k=list(chunk_3d_shape_k))
    nc = int(num_cond_latents or 0)
    if n == 1:
        if nc > 0:
            return B.flash_attn_bsa_3d_cond(q, k, v, latent_shape, nc, **params)
        return B.flash_attn_bsa_3d(q, k, v, latent_shape, latent_shape, **params)
    group = context_parallel_util.get_cp_group()
    Bsz, H, Sl, D = q.shape
    T, Hh, Ww = latent_shape
    chunk = tuple(chunk_3d_shape_q)
    fast = (Bsz == 1 and cdf_threshold is None and sparsity is not None and tuple(chunk_3d_shape_k) == chunk and H % n == 0
            and T % n == 0 and (T // n) % chunk[0] == 0 and Hh % chunk[1] == 0 and Ww % chunk[2] == 0
            and (T // n) * Hh * Ww == Sl and q.dtype in (torch.bfloat16, torch.float16)
            and peer_exchange.available(q, group)
            and all(t[0, 0].is_contiguous() and t.shape == q.shape and t.dtype == q.dtype for t in (q, k, v)))
    if nc > 0 and not 0 < nc < T // n:
        raise ValueError(f"num_cond_latents {nc} outside (0, {T // n})")
    if nc > 0:
        nblk_all = (T // chunk[0]) * (Hh // chunk[1]) * (Ww // chunk[2]) if fast else 0
        fast = fast and nc % chunk[0] == 0 and nblk_all <= 1536
    if not fast:
        return _generic_cond(q, k, v, latent_shape, nc, n, params) if nc > 0 else _generic(q, k, v, latent_shape, params)
    hn = H // n
    local_grid = (T // n, Hh, Ww)
    nblk_l = B.num_blocks(local_grid, chunk)
    ex = peer_exchange.open_exchange(group, q, extra_elems=2 * hn * n * nblk_l * D)
    if ex is None:
        return _generic_cond(q, k, v, latent_shape, nc, n, params) if nc > 0 else _generic(q, k, v, latent_shape, params)
    main, side = ex.main, ex.side

    side.wait_stream(main)
    if not torch.cuda.is_current_stream_capturing():
        for t in (q, k, v):
            t.record_stream(side)
    scatter = _SCATTER_OUT and D == 128 and chunk[0] * chunk[1] * chunk[2] in (64, 128)  # what the tcgen05 kernels take
    stages = _stages_scattered(hn, n) if scatter else U._stages(hn, U._heads_per_group(hn))
    phases = _PhaseTimer(main) if _PHASES else None

    # 1. pooled rows of this rank's tokens, all heads, stored straight into their owners' memory; one barrier
    ex.pool_scatter(q, k, local_grid, chunk, nblk_l)
    if phases:
        phases.mark("pool_scatter+barrier")

    # 2. the q, k, v slabs of the first two stages go onto the copy engines (side stream, one barrier per stage).  The
    #    receive regions of the stages are disjoint and nothing but the inputs is needed to fill them, so every push
    #    could be queued here; but queueing a push costs the host tens of copies, and the main stream would sit idle
    #    behind them.  So the host queues stage g + 2 right after it has launched the attention of stage g: the slabs
    #    travel two stages ahead of their use, and the kernels are never waiting for the host.
    evs = [ex.push_in((q, k, v), *st) for st in stages[:2]]

    # 3. block lists of all local heads while the first slabs travel
    qc, kc = ex.pooled_received(nblk_l)  # [1, hn, N * nblk_l, D]: rank-major block order = block order of the grid
    if nc > 0:
        hw, period = (Hh // chunk[1]) * (Ww // chunk[2]), (T // n) // chunk[0]
        idx, cnt = B.get_select_indices_from_pooled_split(qc, kc, sparsity, hw, period, nc // chunk[0], hw, period, nc // chunk[0])
    else:
        idx, cnt = B.get_select_indices_from_pooled(qc, kc, sparsity, None)
    if phases:
        phases.mark("select")
    scale = 1 / D ** 0.5

    # 4. attention by head group.  The kernel stores every query block's rows straight into the result buffer of the
    #    rank that owns those tokens (the return all-to-all folded into the output stores); one barrier at the end.
    #    LCBSA_CP_SCATTER_OUT=0: the kernel writes a local [1, h, S, D] tensor and the copy engines take it back.
    ev_out = None
    for g, (lo, hi) in enumerate(stages):
        main.wait_event(evs[g])
        if phases:
            phases.mark(f"wait_slabs_{g}")
        q_, k_, v_ = ex.received(lo, hi)
        if scatter:
            ex.attn_scatter(q_, k_, v_, scale, idx[:, lo:hi], cnt[:, lo:hi], latent_shape, chunk, lo)
        else:
            o = B.attn_fwd_bsa_varlen(q_, k_, v_, scale, idx[:, lo:hi], cnt[:, lo:hi], latent_shape, latent_shape, chunk, chunk)
            ev_out = ex.push_out(o, lo)
        if phases:
            phases.mark(f"attention_{g}")
        if g + 2 < len(stages):
            evs.append(ex.push_in((q, k, v), *stages[g + 2]))
    if scatter:
        ex.finish_scatter()
    else:
        main.wait_event(ev_out)
    if phases:
        phases.mark("last_return_or_barrier")
    if os.environ.get("LCBSA_ULYSSES_ALIAS_OUT", "0") == "1":
        return ex.local_out
    return ex.local_out.clone()


_HOST_STATE = {}


def flash_attn_bsa_3d_ulysses_host(q, k, v, latent_shape, out=None, heads_per_chunk=None, device=None, **bsa_params):
    """``flash_attn_bsa_3d_ulysses`` for shards that live in (pinned) HOST memory: ``q, k, v [1, H, S/N, D]`` on the host
    in, this rank's ``[1, H, S/N, D]`` result on the host out (``out`` is filled and returned if given).

    Heads are independent, so the call is pipelined by chunks of ``heads_per_chunk`` heads (a multiple of the group
    size; default: a quarter of the heads): while the group works on chunk c, the copy engines bring chunk c+1 to the
    device and take the result of chunk c-1 back.  Every rank must call it with the same chunking.  Extension without
    counterpart in the reference, whose op takes device tensors.  Returns when the result is complete in ``out``."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise RuntimeError("flash_attn_bsa_3d_ulysses_host takes host tensors")
    n = context_parallel_util.get_cp_size()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B_, H, Sl, D = q.shape
    hc = H // 4 if heads_per_chunk is None else int(heads_per_chunk)
    hc = max(n, (hc // n) * n)
    if H % hc:
        hc = H
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    key = (dev.index, B_, hc, Sl, D, q.dtype)
    st = _HOST_STATE.get(key)
    if st is None:
        _HOST_STATE.clear()
        st = {name: [torch.empty(B_, hc, Sl, D, dtype=q.dtype, device=dev) for _ in range(2)] for name in ("q", "k", "v")}
        st["h2d"], st["d2h"] = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        _HOST_STATE[key] = st
    main = torch.cuda.current_stream(dev)
    h2d, d2h = st["h2d"], st["d2h"]
    h2d.wait_stream(main)
    d2h.wait_stream(main)
    chunks = [(lo, lo + hc) for lo in range(0, H, hc)]
    done = []

    def bring(c):
        lo, hi = chunks[c]
        with torch.cuda.stream(h2d):
            if c >= 2:
                h2d.wait_event(done[c - 2])  # the kernels and pushes of chunk c-2 are through with this staging buffer
            for name, src in (("q", q), ("k", k), ("v", v)):
                st[name][c & 1].copy_(src[:, lo:hi], non_blocking=True)
            return h2d.record_event()

    arrived = [bring(0)]
    for c, (lo, hi) in enumerate(chunks):
        if c + 1 < len(chunks):
            arrived.append(bring(c + 1))
        main.wait_event(arrived[c])
        o = flash_attn_bsa_3d_ulysses(st["q"][c & 1], st["k"][c & 1], st["v"][c & 1], latent_shape, **bsa_params)
        done.append(main.record_event())
        o.record_stream(d2h)
        with torch.cuda.stream(d2h):
            d2h.wait_event(done[c])
            out[:, lo:hi].copy_(o, non_blocking=True)
    main.wait_stream(d2h)
    main.wait_stream(h2d)
    d2h.synchronize()
    h2d.synchronize()
    return out
