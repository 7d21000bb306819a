"""The entry point that allocates nothing (lcbsa_block_select_static), called through the C ABI.

It exists for hosts that may not allocate device memory when they call the library (a frozen memory
pool, a plugin that only gets its input and output buffers); its scratch is a 32 MiB array inside the
library.  The block lists it returns must be identical to those of lcbsa_block_select (integer work:
bit-exact), on two calls in a row -- the second call finds the first call's data in the scratch.
This file sorts last on purpose, so that a run that stops at the first failure has run everything else.
"""
import ctypes

import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import Workload, make_qkv

pytestmark = pytest.mark.gpu


def _select_static(q, k, grid_q, grid_k, sparsity, chunk, check_driver_memory=False):
    Bsz, H, _, _ = q.shape
    nq, nk = B.num_blocks(grid_q, chunk), B.num_blocks(grid_k, chunk)
    nsel = B.num_selected(sparsity, nk)
    cap = max(nsel, 1)
    idx = torch.full((Bsz, H, nq, cap), -7, dtype=torch.int32, device=q.device)
    cnt = torch.full((Bsz, H, nq), -7, dtype=torch.int32, device=q.device)
    qd, kd = L.tensor_desc(q), L.tensor_desc(k)
    gq, gk = L.grid_desc(grid_q, chunk), L.grid_desc(grid_k, chunk)
    # torch's own counter cannot see a cudaMalloc made inside the library, the driver's free-memory figure can.
    # (The first call on a device may make the CUDA runtime load the module that holds the array; from the second
    # call on, the figure must not move.)
    torch.cuda.synchronize()
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    rc = L.lib().lcbsa_block_select_static(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(gq), ctypes.byref(gk), nsel, cap,
                                           idx.data_ptr(), cnt.data_ptr(), L.current_stream(q.device))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    if check_driver_memory:
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
    return rc, idx, cnt


def test_static_scratch_matches_workspace_version_twice():
    wl_a = Workload("a", 5001, 1, 3, 128, (8, 12, 20), (8, 16, 20), (4, 4, 4), 0.75, torch.bfloat16, "scaled_lowrank")
    wl_b = Workload("b", 5002, 2, 2, 128, (4, 8, 8), (5, 7, 9), (4, 4, 4), 0.5, torch.bfloat16, "normal")  # ragged K grid
    for n, wl in enumerate((wl_a, wl_b)):  # two calls in a row on one device: the second finds the first one's rows in the scratch
        q, k, _ = (t.cuda() for t in make_qkv(wl))
        want_idx, want_cnt = B.get_select_indices(q, k, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
        rc, idx, cnt = _select_static(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, check_driver_memory=n > 0)
        L.check(rc)
        torch.cuda.synchronize()
        assert torch.equal(cnt, want_cnt)
        assert torch.equal(idx, want_idx)


def test_static_scratch_rejects_oversized_problems():
    # pooled Q + K of this shape is 2 * 64 * 9216 * 128 * 2 B = 302 MB > 32 MiB: refused on the host, nothing launched
    q = torch.empty(1, 64, 9216 * 1, 128, dtype=torch.bfloat16, device="cuda")
    rc, _, _ = _select_static(q, q, (9216, 1, 1), (9216, 1, 1), 0.999, (1, 1, 1))
    assert rc == -3
    assert b"built-in array" in L.lib().lcbsa_last_error()
