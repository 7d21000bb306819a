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

from . import context_parallel_util


def _exchange(send: Sequence[torch.Tensor], recv: Sequence[torch.Tensor], group, async_op: bool = False):
    """Peer r gets send[r]; recv[r] is filled by peer r.  Every entry is a contiguous tensor."""
    rank = dist.get_rank(group)
    if dist.get_backend(group) == "nccl":
        return dist.all_to_all(list(recv), list(send), group=group, async_op=async_op)
    # backends without a list all-to-all (gloo on CPU): batched point-to-point
    ops = []
    ranks = dist.get_process_group_ranks(group)
    for r in range(len(send)):
        if r == rank:
            continue
        ops.append(dist.P2POp(dist.isend, send[r], ranks[r], group=group))
        ops.append(dist.P2POp(dist.irecv, recv[r], ranks[r], group=group))
    works = dist.batch_isend_irecv(ops) if ops else []
    recv[rank].copy_(send[rank])
    if async_op:
        return _Works(works)
    for w in works:
        w.wait()
    return None


class _Works:
    def __init__(self, works):
        self.works = works

    def wait(self):
        for w in self.works:
            w.wait()


def _views_or_staging(t: torch.Tensor, views: List[torch.Tensor]) -> Tuple[List[torch.Tensor], Optional[torch.Tensor]]:
    """The per-peer views if they are contiguous, else one staging buffer ``[N, ...]`` to copy through."""
    if all(v.is_contiguous() for v in views):
        return views, None
    stage = torch.empty((len(views),) + tuple(views[0].shape), dtype=t.dtype, device=t.device)
    return [stage[i] for i in range(len(views))], stage


def _finish(works, stage_pairs, out):
    def finish():
        for w in works:
            if w is not None:
                w.wait()
        for dst, src in stage_pairs:
            dst.copy_(src)
        return out
    return finish


def heads_scatter_seq_gather(x: torch.Tensor, group, head_lo: int = 0, head_hi: Optional[int] = None,
                             async_op: bool = False):
    """``[B, H, S/N, D] -> [B, h, S, D]`` for local heads ``head_lo:head_hi`` of this rank's ``H/N``.

    With B = 1 and contiguous ``[S/N, D]`` slabs the exchange is one grouped send/recv per head straight
    between the slabs of ``x`` and of the result (no copy); otherwise it goes through one staging copy
    per side."""
    n = dist.get_world_size(group)
    B, H, Sl, D = x.shape
    if H % n != 0:
        raise ValueError(f"Dimension 1 must be divisible by world size {n}")
    hn = H // n
    head_hi = hn if head_hi is None else head_hi
    h = head_hi - head_lo
    out = torch.empty(B, h, n * Sl, D, dtype=x.dtype, device=x.device)
    works, stage_pairs = [], []
    if B == 1 and x[0, 0].is_contiguous():
        for j in range(h):
            send = [x[0, r * hn + head_lo + j] for r in range(n)]
            recv = [out[0, j, r * Sl:(r + 1) * Sl] for r in range(n)]
            works.append(_exchange(send, recv, group, async_op=async_op))
    else:
        send_views = [x[:, r * hn + head_lo: r * hn + head_hi] for r in range(n)]
        recv_views = [out[:, :, r * Sl:(r + 1) * Sl] for r in range(n)]
        send, s_stage = _views_or_staging(x, send_views)
        recv, r_stage = _views_or_staging(out, recv_views)
        if s_stage is not None:
            for r in range(n):
                send[r].copy_(send_views[r])
        works.append(_exchange(send, recv, group, async_op=async_op))
        if r_stage is not None:
            stage_pairs = [(recv_views[r], recv[r]) for r in range(n)]
    fin = _finish(works, stage_pairs, out)
    return fin if async_op else fin()


def seq_scatter_heads_gather(x: torch.Tensor, group, out: Optional[torch.Tensor] = None, head_lo: int = 0,
                             heads_per_rank: Optional[int] = None, async_op: bool = False):
    """``[B, h, S, D] -> [B, H, S/N, D]``: the inverse; ``out`` (optional) is the full ``[B, H, S/N, D]``
    result and ``x`` fills heads ``r*heads_per_rank + head_lo ...`` of it for every source rank r."""
    n = dist.get_world_size(group)
    B, h, S, D = x.shape
    if S % n != 0:
        raise ValueError(f"Dimension 2 must be divisible by world size {n}")
    Sl = S // n
    hn = h if heads_per_rank is None else heads_per_rank
    if out is None:
        out = torch.empty(B, n * hn, Sl, D, dtype=x.dtype, device=x.device)
    works, stage_pairs = [], []
    if B == 1 and x.is_contiguous() and out[0, 0].is_contiguous():
        for j in range(h):
            send = [x[0, j, r * Sl:(r + 1) * Sl] for r in range(n)]
            recv = [out[0, r * hn + head_lo + j] for r in range(n)]
            works.append(_exchange(send, recv, group, async_op=async_op))
    else:
        send_views = [x[:, :, r * Sl:(r + 1) * Sl] for r in range(n)]
        recv_views = [out[:, r * hn + head_lo: r * hn + head_lo + h] for r in range(n)]
        send, s_stage = _views_or_staging(x, send_views)
        recv, r_stage = _views_or_staging(out, recv_views)
        if s_stage is not None:
            for r in range(n):
                send[r].copy_(send_views[r])
        works.append(_exchange(send, recv, group, async_op=async_op))
        if r_stage is not None:
            stage_pairs = [(recv_views[r], recv[r]) for r in range(n)]
    fin = _finish(works, stage_pairs, out)
    return fin if async_op else fin()


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
    # [B, H, S/N, D] -> [B, H/N, S, D]
    return (heads_scatter_seq_gather(query, group), heads_scatter_seq_gather(key, group),
            heads_scatter_seq_gather(value, group))


@torch.compiler.disable
def ulysses_a2a_out(output):
    if context_parallel_util.get_cp_size() == 1:
        return output
    # [B, H/N, S, D] -> [B, H, S/N, D]
    return seq_scatter_heads_gather(output, context_parallel_util.get_cp_group())


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
        if hg == hn:
            q, k, v = ulysses_a2a_in(query, key, value)
            return ulysses_a2a_out(func(self, q, k, v, shape))
        stages = [(lo, lo + hg) for lo in range(0, hn, hg)]
        pending_in = [tuple(heads_scatter_seq_gather(t, group, lo, hi, async_op=True) for t in (query, key, value))
                      for lo, hi in stages]
        out, pending_out = None, []
        for (lo, hi), fins in zip(stages, pending_in):
            q, k, v = (f() for f in fins)
            o = func(self, q, k, v, shape)
            if out is None:
                out = torch.empty(B, H, o.shape[2] // n, o.shape[3], dtype=o.dtype, device=o.device)
            pending_out.append(seq_scatter_heads_gather(o, group, out=out, head_lo=lo, heads_per_rank=hn, async_op=True))
        for f in pending_out:
            f()
        return out

    return wrapper
