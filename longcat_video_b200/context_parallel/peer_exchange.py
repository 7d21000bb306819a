"""Ulysses exchange by peer DMA copies over NVLink instead of NCCL send/recv kernels.

Every rank of the context-parallel group owns one symmetric buffer (``torch.distributed._symmetric_memory``:
the same allocation on every GPU, mapped into every process) that holds its receive side of the exchange:
``q, k, v`` as ``[H/N, S, D]`` each and the attention result as ``[H, S/N, D]``.  A rank *pushes*: it copies each
``[S/N, D]`` slab it owes a peer straight into that peer's buffer with a device-to-device ``cudaMemcpyAsync``
(``lcbsa_copy_slabs``), which the driver executes on the copy engines over NVLink, and then joins a barrier of the
group on the same stream.  When a
rank leaves the barrier, every slab pushed to it before the barrier has landed.

Why not NCCL here: the attention kernel is persistent and takes every SM it is given, so NCCL's send/recv
kernels cannot run beside it and the exchange does not overlap; the copy engines need no SM.  (Measured on two
B200: 203 GB/s per direction for the exchange through NCCL against 465 GB/s for pushes of the same size
including the barrier.)  The barrier is a one-CTA kernel; ``lcbsa_set_attn_sm_reserve`` keeps an SM free for it.

The three functions of the reference's hooks (``longcat_video/context_parallel/ulysses_wrapper.py:86-116``) keep
their meaning; this module only moves the bytes.  No kernel of this library reads or writes peer memory.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

_ARENAS: Dict[Tuple[int, int, torch.dtype], "PeerArena"] = {}


def available(t: torch.Tensor, group) -> bool:
    """True when the exchange of ``t`` over ``group`` can take the peer-copy path."""
    if os.environ.get("LCBSA_ULYSSES_EXCHANGE", "peer") != "peer":
        return False
    if not t.is_cuda or dist.get_backend(group) != "nccl":
        return False
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return True


class PeerArena:
    """The symmetric receive buffer of one (group, device, dtype) and the views of it in every peer."""

    def __init__(self, group, device: torch.device, dtype: torch.dtype):
        self.group, self.device, self.dtype = group, device, dtype
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.numel = 0
        self.buf: Optional[torch.Tensor] = None
        self.hdl = None

    def ensure(self, numel: int) -> None:
        """Collective: every rank asks for the same size (the exchange shapes are the same on all ranks)."""
        if numel <= self.numel:
            return
        import torch.distributed._symmetric_memory as symm_mem

        if self.buf is not None:  # growing: nobody may still be pushing into the old buffer
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        self.buf = symm_mem.empty(numel, dtype=self.dtype, device=self.device)
        self.hdl = symm_mem.rendezvous(self.buf, self.group)
        self.numel = numel
        self.__dict__.pop("_copy_plans", None)  # cached pointer tables name addresses of the old buffer

    def view(self, rank: int, offset: int, shape) -> torch.Tensor:
        """``shape`` elements at ``offset`` of rank ``rank``'s buffer, as a tensor on this device."""
        if rank == self.rank:
            n = 1
            for s in shape:
                n *= s
            return self.buf[offset:offset + n].view(shape)
        return self.hdl.get_buffer(rank, tuple(shape), self.dtype, offset)

    def barrier(self, channel: int = 0) -> None:
        """Barrier of the group on the current stream.  Barriers issued from different streams use different channels
        (each channel has its own signal pad), so that they cannot be taken for one another."""
        self.hdl.barrier(channel=channel)


def arena(group, device: torch.device, dtype: torch.dtype) -> PeerArena:
    key = (id(group), torch.device(device).index or 0, dtype)
    if key not in _ARENAS:
        _ARENAS[key] = PeerArena(group, device, dtype)
    return _ARENAS[key]


def reset() -> None:
    _ARENAS.clear()
    _SIDE.clear()
    _FAILED.clear()


_AUX_STREAMS = int(os.environ.get("LCBSA_ULYSSES_COPY_STREAMS", "4"))  # streams the slab copies of one push are spread over
_AUX: Dict[int, List[torch.cuda.Stream]] = {}


def _aux_streams(device, count: int) -> List[torch.cuda.Stream]:
    idx = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    have = _AUX.setdefault(idx, [])
    while len(have) < count:
        have.append(torch.cuda.Stream(device=device))
    return have[:count]


_SIDE: Dict[int, torch.cuda.Stream] = {}
_FAILED: Dict[int, str] = {}


def open_exchange(group, query: torch.Tensor, extra_elems: int = 0) -> Optional["PeerExchange"]:
    """The exchange object for one call, or None when the symmetric buffer cannot be set up for this group (the
    failure is remembered and reported once; the caller then takes the NCCL path).  Setting it up is a collective
    of the group, so every rank gets the same answer."""
    gid = id(group)
    if gid in _FAILED:
        return None
    idx = query.device.index if query.device.index is not None else torch.cuda.current_device()
    if idx not in _SIDE:
        _SIDE[idx] = torch.cuda.Stream(device=query.device)
    try:
        return PeerExchange(group, query, torch.cuda.current_stream(query.device), _SIDE[idx], extra_elems)
    except Exception as e:  # noqa: BLE001 - any failure of the symmetric-memory setup means "use NCCL"
        _FAILED[gid] = repr(e)
        import warnings

        warnings.warn(f"peer-copy exchange unavailable ({e!r}); using the NCCL exchange")
        return None


class PeerExchange:
    """One forward call's worth of exchange for ``[1, H, S/N, D]`` inputs: receive views and the push operations.

    All pushes and barriers are issued on ``side`` in the same order on every rank (the barrier is a collective of
    the group); ``main`` is the stream the attention kernels run on.  A push is one call of ``lcbsa_copy_slabs``
    (a loop of ``cudaMemcpyAsync`` in C: the Python cost of the hundred-odd slabs of a step would otherwise rival
    the attention itself on eight GPUs)."""

    def __init__(self, group, query: torch.Tensor, main: torch.cuda.Stream, side: torch.cuda.Stream, extra_elems: int = 0):
        from .. import _lib as L

        self._L = L
        B, H, Sl, D = query.shape
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.H, self.Sl, self.D = H, Sl, D
        self.hn = H // self.n
        self.S = self.n * Sl
        self.es = query.element_size()
        self.main, self.side = main, side
        self.ar = arena(group, query.device, query.dtype)
        self.in_elems = self.hn * self.S * D
        out_elems = H * Sl * D
        # two output regions, used alternately, so that the result of one call may still be read while the next
        # call's exchange is already writing
        self.extra_off = 3 * self.in_elems + 2 * out_elems  # `extra_elems` more for the caller (pooled rows)
        self.ar.ensure(self.extra_off + extra_elems)
        # The regions are laid out from this call's shape.  The argument that a call cannot overwrite what the
        # previous one is still using (two alternating result regions, receive regions guarded by the previous call's
        # barriers) holds between calls of ONE layout; when the layout changes, every rank first finishes what it has
        # queued and the group meets, exactly as when the buffer grows.
        layout = (H, Sl, D, int(extra_elems))
        if getattr(self.ar, "_layout", layout) != layout:
            torch.cuda.synchronize(query.device)
            dist.barrier(group=group)
        self.ar._layout = layout
        calls = getattr(self.ar, "_calls", 0)
        self.ar._calls = calls + 1
        self.out_off = 3 * self.in_elems + (calls & 1) * out_elems
        # my receive side
        self.local_in = [self.ar.view(self.rank, t * self.in_elems, (1, self.hn, self.S, D)) for t in range(3)]
        self.local_out = self.ar.view(self.rank, self.out_off, (1, H, Sl, D))
        # base address of every rank's buffer as seen from this process
        if getattr(self.ar, "_bases", None) is None or self.ar._bases_numel != self.ar.numel:
            self.ar._bases = [self.ar.view(r, 0, (1,)).data_ptr() for r in range(self.n)]
            self.ar._bases_numel = self.ar.numel
        self.bases = self.ar._bases

    def _copy(self, make_lists, key=None, nbytes: Optional[int] = None) -> None:
        """Enqueue slab copies.  Called with ``side`` current.  ``make_lists()`` returns (dst, src, lanes): device
        addresses and, per slab, its destination rank; the slabs are spread by destination over a few auxiliary
        streams, so that copies to different peers use different copy engines and links at the same time, and ``side``
        continues when all of them are done.  The pointer tables of a ``key`` (the addresses involved and the head
        range) are built once and reused by later calls: a layer repeats the same pushes step after step."""
        nbytes = self.Sl * self.D * self.es if nbytes is None else nbytes
        cache = self.ar.__dict__.setdefault("_copy_plans", {})
        plan = cache.get(key) if key is not None else None
        if plan is None:
            dst, src, lanes = make_lists()
            n_aux = min(_AUX_STREAMS, self.n) - 1 if lanes is not None else 0
            groups: List[Tuple[List[int], List[int]]] = [([], []) for _ in range(n_aux + 1)]
            for i in range(len(dst)):
                g = (lanes[i] % len(groups)) if lanes is not None else 0
                groups[g][0].append(dst[i])
                groups[g][1].append(src[i])
            plan = []
            for g, (d, s_) in enumerate(groups):
                if d:
                    m = len(d)
                    arr = (ctypes.c_void_p * (2 * m))(*d, *s_)
                    plan.append((g, m, arr, ctypes.addressof(arr)))
            if key is not None:
                if len(cache) > 256:
                    cache.clear()
                cache[key] = plan
        aux = _aux_streams(self.side.device, max((g for g, _, _, _ in plan), default=0))
        start = self.side.record_event() if any(g > 0 for g, _, _, _ in plan) else None
        for g, m, _arr, base in plan:
            stream = self.side if g == 0 else aux[g - 1]
            if g > 0:
                stream.wait_event(start)
            self._L.check(self._L.lib().lcbsa_copy_slabs(base, base + m * ctypes.sizeof(ctypes.c_void_p), nbytes, m, stream.cuda_stream))
            if g > 0:
                self.side.wait_event(stream.record_event())

    def pool_scatter(self, q: torch.Tensor, k: torch.Tensor, local_grid, chunk, rows: int) -> None:
        """Mean-pool the 3-D blocks of this rank's tokens of q and k (all heads) and store the rows of every head
        straight into the extra region of the rank that owns the head (``lcbsa_pool_scatter``: one kernel, ordinary
        stores to peer memory), then meet the group.  Runs on the CURRENT stream (barrier channel 1); when it has
        passed, ``pooled_received`` holds the pooled q and k of the gathered sequence for this rank's heads."""
        L = self._L
        part_all = self.hn * self.n * rows * self.D  # one tensor's region: [H/N][N][rows][D]
        dq = (ctypes.c_void_p * self.n)(*[self.bases[r] + self.extra_off * self.es for r in range(self.n)])
        dk = (ctypes.c_void_p * self.n)(*[self.bases[r] + (self.extra_off + part_all) * self.es for r in range(self.n)])
        qd, kd = L.tensor_desc(q), L.tensor_desc(k)
        g = L.grid_desc(local_grid, chunk)
        L.check(L.lib().lcbsa_pool_scatter(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(g), ctypes.byref(g), dq, dk, self.n, self.rank,
                                           L.current_stream(q.device)))
        self.ar.barrier(channel=1)

    def pooled_received(self, rows: int) -> List[torch.Tensor]:
        """Pooled q and k of the gathered rank-major sequence for this rank's heads, ``[1, H/N, N * rows, D]`` each:
        views of the extra region as ``pool_scatter`` of all ranks filled it (no copy)."""
        part_all = self.hn * self.n * rows * self.D
        return [self.ar.view(self.rank, self.extra_off + t * part_all, (1, self.hn, self.n * rows, self.D)) for t in range(2)]

    def attn_scatter(self, q, k, v, sm_scale, idx, cnt, latent_shape, chunk, lo: int) -> None:
        """Block-sparse attention of local heads ``lo:lo+h`` over the gathered tensors, with the return exchange folded
        into the kernel's output stores (``lcbsa_attn_fwd_scatter``): the rows of rank r's tokens go straight into rank
        r's result region.  Runs on the current stream; ``finish_scatter`` must follow the last stage."""
        L = self._L
        h = q.shape[1]
        slab = self.Sl * self.D
        dst = (ctypes.c_void_p * self.n)(*[self.bases[r] + (self.out_off + (self.rank * self.hn + lo) * slab) * self.es for r in range(self.n)])
        qd, kd, vd = L.tensor_desc(q), L.tensor_desc(k), L.tensor_desc(v)
        g = L.grid_desc(latent_shape, chunk)
        assert idx.is_contiguous() and cnt.is_contiguous() and idx.dtype == torch.int32 and idx.shape[1] == h
        L.check(L.lib().lcbsa_attn_fwd_scatter(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(vd), ctypes.byref(g), ctypes.byref(g),
                                               idx.data_ptr(), cnt.data_ptr(), idx.shape[-1], float(sm_scale), dst, self.n, slab, self.D,
                                               L.current_stream(q.device)))

    def finish_scatter(self) -> None:
        """Meet the group on the current stream: when it has passed, every rank's scattered stores have landed."""
        self.ar.barrier(channel=1)

    def push_rows(self, tensors, rows: int, after: torch.cuda.Event) -> torch.cuda.Event:
        """Heads-scatter of small per-block tensors ``[1, H, rows, D]`` (the pooled Q and K of this rank's tokens)
        into the extra region of the owners of the heads: one contiguous copy per tensor and peer, received as
        ``[tensor][source rank][H/N][rows][D]``.  ``after`` is the event that marks them computed.  The event
        returned fires when this rank's own region is complete."""
        part = self.hn * rows * self.D  # what one rank sends another per tensor
        for x in tensors:
            if not x.is_contiguous():
                raise ValueError("push_rows takes contiguous tensors")
            if not torch.cuda.is_current_stream_capturing():
                x.record_stream(self.side)

        def lists():
            dst, src, lanes = [], [], []
            for t, x in enumerate(tensors):
                xp = x.data_ptr()
                for r in range(self.n):
                    dst.append(self.bases[r] + (self.extra_off + (t * self.n + self.rank) * part) * self.es)
                    src.append(xp + r * part * self.es)  # x[0, r*hn:(r+1)*hn]
                    lanes.append(r)
            return dst, src, lanes

        with torch.cuda.stream(self.side):
            self.side.wait_event(after)
            self._copy(lists, key=("rows", self.extra_off, rows) + tuple(x.data_ptr() for x in tensors), nbytes=part * self.es)
            self.ar.barrier()
            return self.side.record_event()

    def rows_received(self, n_tensors: int, rows: int) -> List[torch.Tensor]:
        """The tensors of ``push_rows`` as ``[1, H/N, N * rows, D]`` (source-rank-major row order): a small permuting
        copy on the current stream out of the receive layout."""
        part = self.hn * rows * self.D
        out = []
        for t in range(n_tensors):
            v = self.ar.view(self.rank, self.extra_off + t * self.n * part, (self.n, self.hn, rows, self.D))
            out.append(v.permute(1, 0, 2, 3).reshape(1, self.hn, self.n * rows, self.D))
        return out

    def push_in(self, tensors, lo: int, hi: int) -> torch.cuda.Event:
        """Send heads ``lo:hi`` (of every rank's share) of q, k, v to their owners; the event fires when this
        rank's own receive views of those heads are complete."""
        slab = self.Sl * self.D

        def lists():
            dst, src, lanes = [], [], []
            for t, x in enumerate(tensors):
                xp, xs = x.data_ptr(), x.stride(1)
                for r in range(self.n):
                    b = self.bases[r] + t * self.in_elems * self.es
                    for j in range(lo, hi):
                        dst.append(b + (j * self.n + self.rank) * slab * self.es)  # [head j][source rank][S/N][D] of rank r
                        src.append(xp + (r * self.hn + j) * xs * self.es)          # x[0, r * hn + j]
                        lanes.append(r)
            return dst, src, lanes

        with torch.cuda.stream(self.side):
            self._copy(lists, key=("in", lo, hi, self.H, self.Sl, self.D) + tuple((x.data_ptr(), x.stride(1)) for x in tensors))
            self.ar.barrier()
            return self.side.record_event()

    def received(self, lo: int, hi: int) -> List[torch.Tensor]:
        return [v[:, lo:hi] for v in self.local_in]

    def push_out(self, o: torch.Tensor, lo: int) -> torch.cuda.Event:
        """Return the attention result ``o [1, h, S, D]`` of local heads ``lo:lo+h``: token chunk r goes to rank r."""
        done = self.main.record_event()
        if not torch.cuda.is_current_stream_capturing():
            o.record_stream(self.side)
        slab = self.Sl * self.D
        op, nh = o.data_ptr(), o.shape[1]

        def lists():
            dst, src, lanes = [], [], []
            for r in range(self.n):
                b = self.bases[r] + self.out_off * self.es
                for j in range(nh):
                    dst.append(b + (self.rank * self.hn + lo + j) * slab * self.es)  # out[head rank*hn+lo+j] of rank r
                    src.append(op + (j * self.S + r * self.Sl) * self.D * self.es)   # o[0, j, r*Sl:(r+1)*Sl]
                    lanes.append(r)
            return dst, src, lanes

        with torch.cuda.stream(self.side):
            self.side.wait_event(done)
            self._copy(lists, key=("out", lo, nh, self.out_off, self.H, self.Sl, self.D, op))
            self.ar.barrier()
            return self.side.record_event()
