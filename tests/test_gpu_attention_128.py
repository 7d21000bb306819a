"""Parity of the tcgen05 attention kernel for 128-token blocks (the chunk shape flash_attn_bsa_3d takes by default,
[4, 4, 8]) against the CPU oracle.

Covered: block shapes whose split into two 64-key units falls on the t, the h and the w axis; bf16 and fp16; batch 2;
query grids shorter than the key grid; ragged grids, where the second unit of an edge block can lie wholly outside the
grid; explicit block lists of 0 .. 33 entries; list entries outside the key grid; agreement with the generic
(mma.sync) kernel that served these shapes before.

Tolerance (bf16/fp16 result against the fp32 oracle): rel-L2 <= 1e-2, max-abs <= 3e-2, LSE abs <= 2e-2.
"""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import Workload, make_qkv
from oracle import bsa_oracle as O
from tests.helpers import max_abs, rel_l2

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2
MAX_ABS_TOL = 3e-2
LSE_TOL = 2e-2


def _check(wl, idx, cnt, q, k, v, impl=L.ATTN_TC):
    ref, ref_lse = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx.clamp_min(0).contiguous(), cnt)
    L.lib().lcbsa_check_device_status()  # clear
    out, lse = B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), wl.head_dim ** -0.5, idx.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k,
                                     wl.chunk, wl.chunk, return_lse=True, impl=impl)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    r, m = rel_l2(got, ref), max_abs(got, ref)
    assert r <= REL_L2_TOL, f"rel-L2 {r}"
    assert m <= MAX_ABS_TOL, f"max-abs {m}"
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    le = float((lse.cpu()[fin] - ref_lse[fin]).abs().max()) if fin.any() else 0.0
    assert le <= LSE_TOL, f"lse {le}"
    return out, r, m, le


@pytest.mark.parametrize("chunk,grid", [((4, 4, 8), (8, 16, 32)), ((2, 8, 8), (6, 16, 24)), ((8, 4, 4), (16, 8, 12)),
                                        ((1, 8, 16), (5, 16, 32)), ((1, 1, 128), (3, 4, 256)), ((1, 2, 64), (2, 6, 128))])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_block_shapes_against_oracle(chunk, grid, dtype):
    """The key block is cut along its outermost even axis: t for (4,4,8), (2,8,8), (8,4,4); h for (1,8,16), (1,2,64);
    w for (1,1,128).  Lists come from the CUDA block-select and are compared with the oracle's bit for bit."""
    wl = Workload("b128", 5000 + sum(chunk), 2, 2, 128, grid, grid, chunk, 0.75, dtype, "normal")
    q, k, v = make_qkv(wl)
    idx, cnt = B.get_select_indices(q.cuda(), k.cuda(), wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    ref_idx, ref_cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    nsel = int(ref_cnt.flatten()[0])
    assert torch.equal(cnt.cpu(), ref_cnt) and torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel])
    out, r, m, le = _check(wl, idx.cpu(), cnt.cpu(), q, k, v)
    whole = B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), wl.grid_q, wl.grid_k, sparsity=wl.sparsity,
                                chunk_3d_shape_q=list(chunk), chunk_3d_shape_k=list(chunk))
    assert torch.equal(whole, out), "the drop-in entry point runs another kernel than ATTN_TC"
    print(f"PARITY b128 chunk {chunk} {dtype}: {nsel} of {O.num_blocks(grid, chunk)} blocks, rel-L2 {r:.3e} max-abs {m:.3e} lse {le:.3e}")


def test_default_parameters_of_the_entry_point():
    """flash_attn_bsa_3d with no chunk arguments: [4, 4, 8] blocks, sparsity 0.875 on a 16x32x64 grid (256 blocks, 32 kept)."""
    wl = Workload("b128_default", 5100, 1, 2, 128, (16, 32, 64), (16, 32, 64), (4, 4, 8), 0.875, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    got = B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), wl.grid_q, wl.grid_k)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    ref, _ = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx, cnt)
    r, m = rel_l2(got.float().cpu(), ref), max_abs(got.float().cpu(), ref)
    assert r <= REL_L2_TOL and m <= MAX_ABS_TOL, (r, m)


def test_continuation_shape_query_grid_shorter_than_key_grid():
    wl = Workload("b128_vc", 5200, 1, 2, 128, (4, 16, 32), (12, 16, 32), (4, 4, 8), 0.75, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    _check(wl, idx, cnt, q, k, v)


@pytest.mark.parametrize("grid", [(10, 18, 29), (5, 7, 40), (9, 16, 32)])
def test_ragged_grids(grid):
    """(10, 18, 29): the last frame block holds 2 of 4 frames, so its second unit (frames 2-3 of the block) lies wholly
    outside the grid; h and w edges hold 2 of 4 and 5 of 8.  (9, 16, 32): 1 of 4 frames, nothing else ragged."""
    wl = Workload("b128_ragged", 5300 + grid[0], 1, 2, 128, grid, grid, (4, 4, 8), 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    out, r, m, le = _check(wl, idx, cnt, q, k, v)
    mma, _ = B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), wl.head_dim ** -0.5, idx.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k,
                                   wl.chunk, wl.chunk, return_lse=True, impl=L.ATTN_MMA)
    assert max_abs(out.float().cpu(), mma.float().cpu()) <= MAX_ABS_TOL
    print(f"PARITY b128 ragged {grid}: rel-L2 {r:.3e} max-abs {m:.3e} lse {le:.3e}")


def test_lists_whose_only_entries_are_edge_blocks():
    """Every list holds only blocks of the last frame row of a (10, 16, 32) grid, so the second unit of every listed
    block is empty, and the first block a warpgroup sees can be one of which it sees nothing."""
    grid, chunk = (10, 16, 32), (4, 4, 8)
    wl = Workload("b128_edge", 5400, 1, 2, 128, grid, grid, chunk, 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    nq = O.num_blocks(grid, chunk)
    per_t = 4 * 4
    cnt = torch.full((1, 2, nq), 3, dtype=torch.int32)
    idx = torch.full((1, 2, nq, 8), -1, dtype=torch.int32)
    g = torch.Generator().manual_seed(3)
    for h in range(2):
        for i in range(nq):
            idx[0, h, i, :3] = torch.sort(2 * per_t + torch.randperm(per_t, generator=g)[:3]).values.to(torch.int32)
    cnt[0, 1, ::3] = 1
    _check(wl, idx, cnt, q, k, v)


@pytest.mark.parametrize("length", [0, 1, 2, 3, 15, 16, 17, 31, 32, 33])
def test_list_lengths(length):
    """Random ascending lists of `length` entries in head 0; lengths length, 0, 1, length + 2 in rotation in head 1
    (an empty list yields zeros and LSE = -inf)."""
    wl = Workload("b128_lists", 5500 + length, 1, 2, 128, (12, 16, 32), (12, 16, 32), (4, 4, 8), 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    nq = nk = O.num_blocks(wl.grid_q, wl.chunk)
    assert nk == 48
    g = torch.Generator().manual_seed(length)
    cnt = torch.full((1, 2, nq), length, dtype=torch.int32)
    rot = [length, 0, 1, min(length + 2, 48)]
    for i in range(nq):
        cnt[0, 1, i] = rot[i % 4]
    idx = torch.full((1, 2, nq, 48), -1, dtype=torch.int32)
    for h in range(2):
        for i in range(nq):
            n = int(cnt[0, h, i])
            idx[0, h, i, :n] = torch.sort(torch.randperm(nk, generator=g)[:n]).values.to(torch.int32)
    out, *_ = _check(wl, idx, cnt, q, k, v)
    empty = (cnt == 0)
    if empty.any():
        tm = O.token_map(wl.grid_q, wl.chunk)
        for h in range(2):
            for i in range(nq):
                if empty[0, h, i]:
                    assert float(out[0, h, tm[i]].float().abs().max()) == 0.0


def test_list_entry_outside_the_key_grid_is_flagged_not_dereferenced():
    wl = Workload("b128_badidx", 5600, 1, 2, 128, (8, 8, 16), (8, 8, 16), (4, 4, 8), 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    nk = O.num_blocks(wl.grid_k, wl.chunk)
    ref, _ = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx, cnt)
    bad = idx.clone()
    bad[0, 0, 3, 1] = nk + 5
    bad[0, 1, 6, 0] = -3
    L.lib().lcbsa_check_device_status()
    out = B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), wl.head_dim ** -0.5, bad.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k,
                                wl.chunk, wl.chunk, impl=L.ATTN_TC)
    rc = L.lib().lcbsa_check_device_status()
    assert rc == -5, rc
    assert b"outside [0, Nk)" in L.lib().lcbsa_last_error()
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    tm = O.token_map(wl.grid_q, wl.chunk)
    keep = torch.ones(got.shape[1], got.shape[2], dtype=torch.bool)
    keep[0, tm[3]] = False
    keep[1, tm[6]] = False
    assert max_abs(got[0][keep], ref[0][keep]) <= MAX_ABS_TOL


def test_head_dim_64_still_takes_the_generic_kernel():
    """The tcgen05 kernels handle head_dim 128; with LCBSA_ATTN_TC forced, head_dim 64 is refused, and AUTO falls back."""
    wl = Workload("b128_d64", 5700, 1, 2, 64, (8, 8, 16), (8, 8, 16), (4, 4, 8), 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    with pytest.raises(Exception):
        B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), wl.head_dim ** -0.5, idx.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k,
                              wl.chunk, wl.chunk, impl=L.ATTN_TC)
    _check(wl, idx, cnt, q, k, v, impl=L.ATTN_AUTO)


@pytest.mark.parametrize("chunk_k,grid,dtype", [((4, 8, 8), (8, 16, 32), torch.bfloat16), ((8, 8, 8), (8, 16, 32), torch.bfloat16),
                                                ((4, 4, 16), (8, 8, 64), torch.float16), ((4, 8, 8), (10, 20, 29), torch.bfloat16)])
def test_key_blocks_larger_than_query_blocks(chunk_k, grid, dtype):
    """Query blocks of 128 tokens against key blocks of 256 and 512 tokens (the shapes for which the reference switches
    to its multi-tile kernel): 4 and 8 units of 64 keys per selected block.  The last case is ragged on every axis."""
    chunk_q = (4, 4, 8)
    wl = Workload("b128_bigk", 5800 + sum(chunk_k), 1, 2, 128, grid, grid, chunk_q, 0.5, dtype, "normal")
    q, k, v = make_qkv(wl)
    ragged = any(g % c for g, c in zip(grid, chunk_k))
    idx, cnt, _, _ = O.block_select(q, k, grid, grid, 0.5, chunk_q, chunk_k)
    ref, ref_lse = O.attention(q, k, v, grid, grid, chunk_q, chunk_k, idx, cnt)
    L.lib().lcbsa_check_device_status()
    out, lse = B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), wl.head_dim ** -0.5, idx.cuda(), cnt.cuda(), grid, grid,
                                     chunk_q, chunk_k, return_lse=True, impl=L.ATTN_TC)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    got = out.float().cpu()
    r, m = rel_l2(got, ref), max_abs(got, ref)
    assert r <= REL_L2_TOL and m <= MAX_ABS_TOL, (r, m)
    assert float((lse.cpu() - ref_lse).abs().max()) <= LSE_TOL
    whole = B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), grid, grid, sparsity=0.5, chunk_3d_shape_q=list(chunk_q),
                                chunk_3d_shape_k=list(chunk_k), allow_ragged=ragged)
    assert torch.equal(whole, out)
    gi, gc = B.get_select_indices(q.cuda(), k.cuda(), grid, grid, 0.5, None, chunk_q, chunk_k)
    nsel = int(cnt.flatten()[0])
    assert torch.equal(gc.cpu(), cnt) and torch.equal(gi.cpu()[..., :nsel], idx[..., :nsel])
    print(f"PARITY b128 key blocks {chunk_k} {dtype}: {nsel} of {O.num_blocks(grid, chunk_k)} blocks, rel-L2 {r:.3e} max-abs {m:.3e}")
