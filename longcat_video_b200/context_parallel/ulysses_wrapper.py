"""Ulysses sequence <-> head all-to-all around the attention op.

Same hook names and semantics as ``longcat_video/context_parallel/ulysses_wrapper.py``
(``all_to_all`` :7-83, ``ulysses_a2a_in`` :86-95, ``ulysses_a2a_out`` :98-105,
``ulysses_wrapper`` :108-116): before attention every rank trades its ``[B, H, S/N, D]`` slice of all
heads for ``[B, H/N, S, D]`` (all tokens of its own heads, sequence rank-major); afterwards the
inverse.  Identity when the context-parallel size is 1.

What is different from the reference is how the bytes move:
  * the exchange is one grouped NCCL send/recv per peer and head, directly between ``[S/N, D]`` slabs
    of the source and destination tensors -- with B = 1 both sides are already contiguous, so the two
    permute+contiguous copies the reference makes on each side of every all-to-all disappear (other
    shapes take one staging copy instead of two);
  * ``ulysses_wrapper`` pipelines by head group: the all-to-all of group g+1 and the return
    all-to-all of group g-1 run on NCCL's stream while attention works on group g.  Heads are
    independent in BSA, so the result is the same as doing it in one piece.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import context_parallel_util, peer_exchange


class _Works:
    def __init__(self, works):
        self.works = [w for w in works if w is not None]

    def wait(self):
        for w in self.works:
            w.wait()


def _exchange_many(pairs: Sequence[Tuple[Sequence[torch.Tensor], Sequence[torch.Tensor]]], group, async_op: bool = False):
    """Every pair is ``(send, recv)`` with one contiguous tensor per peer: peer r gets send[r] and fills recv[r].
    All pairs travel in ONE grouped point-to-point launch (one NCCL kernel whatever the number of heads and
    tensors; every rank lists its pairs in the same order, which is what matches sends to receives); the
    slab a rank keeps for itself is a device copy on the current stream."""
    rank = dist.get_rank(group)
    ranks = dist.get_process_group_ranks(group)
    ops = []
    for send, recv in pairs:
        for r in range(len(send)):
            if r == rank:
                continue
            ops.append(dist.P2POp(dist.isend, send[r], ranks[r], group=group))
            ops.append(dist.P2POp(dist.irecv, recv[r], ranks[r], group=group))
    works = dist.batch_isend_irecv(ops) if ops else []
    for send, recv in pairs:
        recv[rank].copy_(send[rank])
    w = _Works(works)
    if async_op:
        return w
    w.wait()
    return None


def _exchange(send: Sequence[torch.Tensor], recv: Sequence[torch.Tensor], group, async_op: bool = False):
    """Peer r gets send[r]; recv[r] is filled by peer r.  Every entry is a contiguous tensor."""
    return _exchange_many([(send, recv)], group, async_op=async_op)


def _views_or_staging(t: torch.Tensor, views: List[torch.Tensor]) -> Tuple[List[torch.Tensor], Optional[torch.Tensor]]:
    """The per-peer views if they are contiguous, else one staging buffer ``[N, ...]`` to copy through."""
    if all(v.is_contiguous() for v in views):
        return views, None
    stage = torch.empty((len(views),) + tuple(views[0].shape), dtype=t.dtype, device=t.device)
    return [stage[i] for i in range(len(views))], stage


class _Plan:
    """What one exchange has to move: the (send, recv) slab lists, copies to make before it is launched and
    after it has arrived (only when a side is not made of contiguous slabs), and its result."""

    def __init__(self, out):
        self.out = out
        self.pairs: List[Tuple[List[torch.Tensor], List[torch.Tensor]]] = []
        self.before: List[Tuple[torch.Tensor, torch.Tensor]] = []
        self.after: List[Tuple[torch.Tensor, torch.Tensor]] = []


def _plan_heads_scatter_seq_gather(x: torch.Tensor, n: int, head_lo: int, head_hi: Optional[int]) -> _Plan:
    B, H, Sl, D = x.shape
    if H % n != 0:
        raise ValueError(f"Dimension 1 must be divisible by world size {n}")
    hn = H // n
    head_hi = hn if head_hi is None else head_hi
    h = head_hi - head_lo
    plan = _Plan(torch.empty(B, h, n * Sl, D, dtype=x.dtype, device=x.device))
    out = plan.out
    if B == 1 and x[0, 0].is_contiguous():
        for j in range(h):
            plan.pairs.append(([x[0, r * hn + head_lo + j] for r in range(n)],
                               [out[0, j, r * Sl:(r + 1) * Sl] for r in range(n)]))
    else:
        send_views = [x[:, r * hn + head_lo: r * hn + head_hi] for r in range(n)]
        recv_views = [out[:, :, r * Sl:(r + 1) * Sl] for r in range(n)]
        send, s_stage = _views_or_staging(x, send_views)
        recv, r_stage = _views_or_staging(out, recv_views)
        if s_stage is not None:
            plan.before = [(send[r], send_views[r]) for r in range(n)]
        plan.pairs.append((send, recv))
        if r_stage is not None:
            plan.after = [(recv_views[r], recv[r]) for r in range(n)]
    return plan


def _plan_seq_scatter_heads_gather(x: torch.Tensor, n: int, out: Optional[torch.Tensor], head_lo: int,
                                   heads_per_rank: Optional[int]) -> _Plan:
    B, h, S, D = x.shape
    if S % n != 0:
        raise ValueError(f"Dimension 2 must be divisible by world size {n}")
    Sl = S // n
    hn = h if heads_per_rank is None else heads_per_rank
    if out is None:
        out = torch.empty(B, n * hn, Sl, D, dtype=x.dtype, device=x.device)
    plan = _Plan(out)
    if B == 1 and x.is_contiguous() and out[0, 0].is_contiguous():
        for j in range(h):
            plan.pairs.append(([x[0, j, r * Sl:(r + 1) * Sl] for r in range(n)],
                               [out[0, r * hn + head_lo + j] for r in range(n)]))
    else:
        send_views = [x[:, :, r * Sl:(r + 1) * Sl] for r in range(n)]
        recv_views = [out[:, r * hn + head_lo: r * hn + head_lo + h] for r in range(n)]
        send, s_stage = _views_or_staging(x, send_views)
        recv, r_stage = _views_or_staging(out, recv_views)
        if s_stage is not None:
            plan.before = [(send[r], send_views[r]) for r in range(n)]
        plan.pairs.append((send, recv))
        if r_stage is not None:
            plan.after = [(recv_views[r], recv[r]) for r in range(n)]
    return plan


def _launch(plans: Sequence[_Plan], group, async_op: bool):
    """One grouped launch for all the plans; returns a function that waits for it and yields their results."""
    for p in plans:
        for dst, src in p.before:
            dst.copy_(src)
    work = _exchange_many([pr for p in plans for pr in p.pairs], group, async_op=True)

    def finish():
        work.wait()
        for p in plans:
            for dst, src in p.after:
                dst.copy_(src)
        return [p.out for p in plans]

    return finish if async_op else finish()


def heads_scatter_seq_gather(x: torch.Tensor, group, head_lo: int = 0, head_hi: Optional[int] = None,
                             async_op: bool = False):
    """``[B, H, S/N, D] -> [B, h, S, D]`` for local heads ``head_lo:head_hi`` of this rank's ``H/N``.

    With B = 1 and contiguous ``[S/N, D]`` slabs the bytes go straight between the slabs of ``x`` and of the
    result (no copy); otherwise through one staging copy per side."""
    plan = _plan_heads_scatter_seq_gather(x, dist.get_world_size(group), head_lo, head_hi)
    fin = _launch([plan], group, async_op)
    return (lambda: fin()[0]) if async_op else fin[0]


def seq_scatter_heads_gather(x: torch.Tensor, group, out: Optional[torch.Tensor] = None, head_lo: int = 0,
                             heads_per_rank: Optional[int] = None, async_op: bool = False):
    """``[B, h, S, D] -> [B, H, S/N, D]``: the inverse; ``out`` (optional) is the full ``[B, H, S/N, D]``
    result and ``x`` fills heads ``r*heads_per_rank + head_lo ...`` of it for every source rank r."""
    plan = _plan_seq_scatter_heads_gather(x, dist.get_world_size(group), out, head_lo, heads_per_rank)
    fin = _launch([plan], group, async_op)
    return (lambda: fin()[0]) if async_op else fin[0]


def all_to_all(tensor, scatter_idx, gather_idx, group=None, gather=True):
    """Generic form with the reference's signature (ulysses_wrapper.py:7).  The two cases the attention
    layer uses, (scatter heads, gather sequence) and its inverse on 4-D tensors, take the zero-copy
    route above; anything else goes through ``all_to_all_single`` on a chunked copy."""
    if not dist.is_initialized():
        return tensor
    world_size = dist.get_world_size(group)
    if world_size == 1:
        return tensor
    if scatter_idx == gather_idx:
        raise ValueError("scatter_idx and gather_idx must be different")
    if tensor.shape[scatter_idx] % world_size != 0:
        raise ValueError(f"Dimension {scatter_idx} must be divisible by world size {world_size}")
    if gather and tensor.dim() == 4 and (scatter_idx, gather_idx) == (1, 2):
        return heads_scatter_seq_gather(tensor, group)
    if gather and tensor.dim() == 4 and (scatter_idx, gather_idx) == (2, 1):
        return seq_scatter_heads_gather(tensor, group)
    # generic: chunk the scatter axis to the front, exchange, splice the source-rank axis before gather_idx
    shape = list(tensor.shape)
    chunk = shape[scatter_idx] // world_size
    x = tensor.reshape(shape[:scatter_idx] + [world_size, chunk] + shape[scatter_idx + 1:])
    x = x.movedim(scatter_idx, 0).contiguous()
    y = torch.empty_like(x)
    dist.all_to_all_single(y, x, group=group)
    if gather:
        y = y.movedim(0, gather_idx)
        new_shape = list(y.shape)
        merged = new_shape[:gather_idx] + [new_shape[gather_idx] * new_shape[gather_idx + 1]] + new_shape[gather_idx + 2:]
        return y.reshape(merged)
    return y.movedim(0, gather_idx)[:, context_parallel_util.get_cp_rank()]


@torch.compiler.disable
def ulysses_a2a_in(query, key, value):
    if context_parallel_util.get_cp_size() == 1:
        return query, key, value
    group = context_parallel_util.get_cp_group()
    # [B, H, S/N, D] -> [B, H/N, S, D], all three in one launch
    n = dist.get_world_size(group)
    return tuple(_launch([_plan_heads_scatter_seq_gather(t, n, 0, None) for t in (query, key, value)], group, False))


@torch.compiler.disable
def ulysses_a2a_out(output):
    if context_parallel_util.get_cp_size() == 1:
        return output
    # [B, H/N, S, D] -> [B, H, S/N, D]
    return seq_scatter_heads_gather(output, context_parallel_util.get_cp_group())


def _peer_pipeline(func, self, query, key, value, shape, ex, stages):
    """The pipeline of ``ulysses_wrapper`` with the exchanges done by peer DMA copies (``peer_exchange``): the
    push of stage g+1 and the return of stage g-1 run on the copy engines while attention works on stage g."""
    main, side = ex.main, ex.side
    side.wait_stream(main)
    if not torch.cuda.is_current_stream_capturing():
        for t in (query, key, value):
            t.record_stream(side)
    ev = ex.push_in((query, key, value), *stages[0])
    ev_out = None
    for g, (lo, hi) in enumerate(stages):
        main.wait_event(ev)
        q, k, v = ex.received(lo, hi)
        o = func(self, q, k, v, shape)
        # launched after this stage's kernels so that they are not held up by the host, before its return push
        ev_next = ex.push_in((query, key, value), *stages[g + 1]) if g + 1 < len(stages) else None
        if tuple(o.shape) != (1, hi - lo, ex.S, ex.D) or o.dtype != query.dtype or not o.is_contiguous():
            raise ValueError("the wrapped attention must return a contiguous [1, heads, S, D] tensor of the input dtype")
        ev_out = ex.push_out(o, lo)
        ev = ev_next
    main.wait_event(ev_out)
    if os.environ.get("LCBSA_ULYSSES_ALIAS_OUT", "0") == "1":
        return ex.local_out  # a view of the exchange buffer: valid until the call after the next one
    return ex.local_out.clone()


def _stages(hn: int, hg: int):
    """Head ranges of the pipeline stages.  Only the exchange before the first stage and the return after the last
    one cannot overlap any attention, so those two stages get half the heads of the others (unless the stage size
    was fixed by LCBSA_ULYSSES_GROUP_HEADS)."""
    if hg >= hn:
        return [(0, hn)]
    if "LCBSA_ULYSSES_GROUP_HEADS" in os.environ or hg < 2 or hn < 2 * hg:
        return [(lo, min(lo + hg, hn)) for lo in range(0, hn, hg)]
    edge = hg // 2
    sizes = [edge] + [hg] * ((hn - 2 * edge) // hg) + [edge]
    rest = hn - sum(sizes)
    if rest:
        sizes.insert(1, rest)
    out, lo = [], 0
    for sz in sizes:
        out.append((lo, lo + sz))
        lo += sz
    return out


_SIDE = {}


def _side_stream(device):
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _SIDE:
        _SIDE[key] = torch.cuda.Stream(device=device)
    return _SIDE[key]


def _heads_per_group(local_heads: int) -> int:
    """Heads per pipeline stage.  LCBSA_ULYSSES_GROUP_HEADS overrides it (0 = no pipelining); by default
    the local heads are split into four stages (two when there are four heads or fewer), which keeps every
    attention launch at several waves of work items while hiding most of the exchange."""
    default = max(1, local_heads // 4) if local_heads > 4 else max(1, local_heads // 2)
    v = int(os.environ.get("LCBSA_ULYSSES_GROUP_HEADS", str(default)))
    if v <= 0 or v >= local_heads:
        return local_heads
    while local_heads % v:
        v -= 1
    return v


def ulysses_wrapper(func):
    """Decorator with the reference's contract (ulysses_wrapper.py:108-116): ``func(self, q, k, v, shape)``
    sees ``[B, H/N, S, D]`` tensors and its result is returned as ``[B, H, S/N, D]``.  The work is
    pipelined by head group so the exchanges overlap the attention of the neighbouring groups."""

    @torch.compiler.disable
    def wrapper(self, query, key, value, shape):
        n = context_parallel_util.get_cp_size()
        if n == 1:
            return func(self, query, key, value, shape)
        group = context_parallel_util.get_cp_group()
        B, H, Sl, D = query.shape
        if H % n != 0:
            raise ValueError(f"Dimension 1 must be divisible by world size {n}")
        hn = H // n
        hg = _heads_per_group(hn)
        stages = _stages(hn, hg)
        if (B == 1 and peer_exchange.available(query, group)
                and all(t[0, 0].is_contiguous() and t.shape == query.shape and t.dtype == query.dtype for t in (query, key, value))):
            ex = peer_exchange.open_exchange(group, query)  # None if symmetric memory cannot be set up here
            if ex is not None:
                return _peer_pipeline(func, self, query, key, value, shape, ex, stages)
        if hg == hn:
            q, k, v = ulysses_a2a_in(query, key, value)
            return ulysses_a2a_out(func(self, q, k, v, shape))
        # The exchange of stage g+1 is launched from a side stream before stage g is computed, so that it
        # depends on nothing but the inputs and runs while the attention of stage g does.
        main = torch.cuda.current_stream() if query.is_cuda else None
        side = _side_stream(query.device) if query.is_cuda else None
        if side is not None:
            side.wait_stream(main)

        def start_in(lo, hi):
            plans = [_plan_heads_scatter_seq_gather(t, n, lo, hi) for t in (query, key, value)]  # results allocated on `main`
            if side is None:
                return _launch(plans, group, True), None
            with torch.cuda.stream(side):
                fin = _launch(plans, group, True)
                ev = side.record_event()  # covers the self-slab copies, which ran on the side stream
            return fin, ev

        out, pending_out, done = None, [], []
        nxt = start_in(*stages[0])
        for g, (lo, hi) in enumerate(stages):
            cur = nxt
            if g + 1 < len(stages):
                # The receive buffers of stage g+1 come from the caching allocator of `main` and may be blocks that
                # stage g-1 (its q, k, v, its block lists and workspaces) has just given back while its kernels are
                # still queued on `main`; the exchange fills them from `side`, so `side` first waits for those kernels.
                if side is not None and done:
                    side.wait_event(done[-1])
                nxt = start_in(*stages[g + 1])
            q, k, v = cur[0]()
            if cur[1] is not None:
                main.wait_event(cur[1])
            o = func(self, q, k, v, shape)
            if main is not None:
                done.append(main.record_event())
            if out is None:
                out = torch.empty(B, H, o.shape[2] // n, o.shape[3], dtype=o.dtype, device=o.device)
            pending_out.append(seq_scatter_heads_gather(o, group, out=out, head_lo=lo, heads_per_rank=hn, async_op=True))
        for f in pending_out:
            f()
        return out

    return wrapper
