"""Parity of the CUDA block-sparse attention forward (through the C ABI) against the CPU oracle.

Tolerance (bf16 / fp16 result against the fp32 oracle): rel-L2 <= 1e-2 and max-abs <= 3e-2.
"""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import Workload, make_qkv
from oracle import bsa_oracle as O
from tests.golden.cases import CASES
from tests.helpers import load_golden, max_abs, rel_l2

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2
MAX_ABS_TOL = 3e-2

TC, MMA = L.ATTN_TC, L.ATTN_MMA

SEEDED = {
    "ragged_bf16": Workload("ragged_bf16", 4001, 1, 2, 128, (5, 7, 9), (6, 7, 10), (4, 4, 4), 0.5, torch.bfloat16, "normal"),
    "multiwork_bf16": Workload("multiwork_bf16", 4002, 1, 3, 128, (8, 12, 20), (8, 12, 20), (4, 4, 4), 0.75, torch.bfloat16, "scaled_lowrank"),
    "cross_fp16": Workload("cross_fp16", 4003, 1, 2, 128, (4, 8, 12), (12, 8, 12), (4, 4, 4), 0.875, torch.float16, "normal"),
    "batch2_bf16": Workload("batch2_bf16", 4004, 2, 2, 128, (4, 8, 8), (4, 8, 8), (4, 4, 4), 0.5, torch.bfloat16, "normal"),
    "chunk248_bf16": Workload("chunk248_bf16", 4005, 1, 2, 128, (4, 8, 16), (4, 8, 16), (2, 4, 8), 0.5, torch.bfloat16, "normal"),
    "large_logits_bf16": Workload("large_logits_bf16", 4006, 1, 1, 128, (4, 8, 8), (8, 8, 8), (4, 4, 4), 0.25, torch.bfloat16, "normal"),
}


def _impls(wl):
    tc_ok = wl.head_dim == 128 and wl.chunk[0] * wl.chunk[1] * wl.chunk[2] in (64, 128)  # one tcgen05 kernel for each
    return [TC, MMA] if tc_ok else [MMA]


def _check(out, ref):
    assert torch.isfinite(out.float()).all()
    r, m = rel_l2(out.float().cpu(), ref), max_abs(out.float().cpu(), ref)
    assert r <= REL_L2_TOL, f"rel-L2 {r}"
    assert m <= MAX_ABS_TOL, f"max-abs {m}"
    return r, m


def _attn(q, k, v, wl, idx, cnt, impl, **kw):
    return B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), 1 / wl.head_dim ** 0.5, idx.cuda(), cnt.cuda(),
                                 wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, impl=impl, **kw)


@pytest.mark.parametrize("name", [n for n, (_, a) in CASES.items() if a and CASES[n][0].dtype != torch.float32])
def test_golden_cases(name):
    """Reference lists -> our attention -> the reference's masked-SDPA result."""
    wl, _ = CASES[name]
    gold = load_golden(name)
    q, k, v = make_qkv(wl)
    idx = torch.sort(torch.from_numpy(gold["idx"].astype("int32")), dim=-1).values.contiguous()
    cnt = torch.from_numpy(gold["lens"].astype("int32"))
    ref = torch.from_numpy(gold["attn"])
    for impl in _impls(wl):
        out = _attn(q, k, v, wl, idx, cnt, impl)
        print(name, impl, _check(out, ref))
        L.check(L.lib().lcbsa_check_device_status())


def test_config1_tensors_through_the_whole_forward():
    """The reference's CPU-runnable configuration (B=1, 4 heads x 128, grid 4x8x8, 4x4x4 blocks, sparsity 0.5, N(0,1)
    fp32).  fp32: the CUDA block-select reproduces the lists the reference's own functions produced (fixture
    cfg1_fp32) and the attention kernels refuse the dtype.  The same tensors in bf16 go through the drop-in entry point
    and are held against the oracle."""
    wl, _ = CASES["cfg1_fp32"]
    gold = load_golden("cfg1_fp32")
    q, k, v = make_qkv(wl)
    idx, cnt = B.get_select_indices(q.cuda(), k.cuda(), wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    want = torch.sort(torch.from_numpy(gold["idx"].astype("int32")), dim=-1).values
    assert torch.equal(idx.cpu()[..., :want.shape[-1]], want)
    with pytest.raises(Exception):
        B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), wl.grid_q, wl.grid_k, sparsity=wl.sparsity,
                            chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    qb, kb, vb = (t.to(torch.bfloat16) for t in (q, k, v))
    out = B.flash_attn_bsa_3d(qb.cuda(), kb.cuda(), vb.cuda(), wl.grid_q, wl.grid_k, sparsity=wl.sparsity,
                              chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    L.check(L.lib().lcbsa_check_device_status())
    oi, oc, _, _ = O.block_select(qb, kb, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    ref, _ = O.attention(qb, kb, vb, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, oi, oc)
    print("cfg1 in bf16", _check(out, ref))


@pytest.mark.parametrize("name", list(SEEDED))
def test_seeded_cases(name):
    wl = SEEDED[name]
    q, k, v = make_qkv(wl)
    if name == "large_logits_bf16":
        q, k = q * 6, k * 6  # logits of a few hundred: the running maximum moves a lot
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    ref, ref_lse = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx, cnt)
    for impl in _impls(wl):
        out, lse = _attn(q, k, v, wl, idx, cnt, impl, return_lse=True)
        print(name, impl, _check(out, ref))
        assert torch.allclose(lse.cpu(), ref_lse, rtol=0, atol=2e-2)
        L.check(L.lib().lcbsa_check_device_status())


def test_ragged_lengths_and_empty_lists():
    """Per-row list lengths that differ, including empty lists (output 0, lse -inf)."""
    wl = SEEDED["multiwork_bf16"]
    q, k, v = make_qkv(wl, heads=2)
    nq, nk = O.num_blocks(wl.grid_q, wl.chunk), O.num_blocks(wl.grid_k, wl.chunk)
    g = torch.Generator().manual_seed(11)
    cap = 9
    cnt = torch.randint(0, cap + 1, (1, 2, nq), generator=g, dtype=torch.int32)
    cnt[0, 0, 0] = 0
    cnt[0, 1, nq - 1] = 0
    idx = torch.full((1, 2, nq, cap), -1, dtype=torch.int32)
    for h in range(2):
        for i in range(nq):
            n = int(cnt[0, h, i])
            idx[0, h, i, :n] = torch.sort(torch.randperm(nk, generator=g)[:n]).values.to(torch.int32)
    ref, ref_lse = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx.clamp_min(0), cnt)
    for impl in (TC, MMA):
        out, lse = _attn(q, k, v, wl, idx.clamp_min(0), cnt, impl, return_lse=True)
        _check(out, ref)
        finite = torch.isfinite(ref_lse)
        assert torch.equal(torch.isfinite(lse.cpu()), finite)
        assert torch.allclose(lse.cpu()[finite], ref_lse[finite], rtol=0, atol=2e-2)
        L.check(L.lib().lcbsa_check_device_status())


def test_strided_inputs_match_contiguous():
    """q,k in [B,S,H,D] memory order and v as a slice of a fused qkv buffer (attention.py:113-115)."""
    wl = SEEDED["batch2_bf16"]
    q, k, v = make_qkv(wl)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    ref, _ = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx, cnt)
    Bsz, H, S, D = k.shape
    qkv = torch.zeros(Bsz, S, 3, H, D, dtype=k.dtype, device="cuda")
    qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2] = (t.cuda().permute(0, 2, 1, 3) for t in (q, k, v))
    qs, ks, vs = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    assert not vs.is_contiguous()
    for impl in (TC, MMA):
        out = B.attn_fwd_bsa_varlen(qs, ks, vs, 1 / D ** 0.5, idx.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k, wl.chunk, wl.chunk,
                                    impl=impl)
        _check(out, ref)
        L.check(L.lib().lcbsa_check_device_status())


def test_flash_attn_bsa_3d_signature_and_result():
    """The drop-in entry point, called the way attention.py:67 calls it."""
    wl = SEEDED["multiwork_bf16"]
    q, k, v = make_qkv(wl)
    bsa_params = dict(sparsity=wl.sparsity, cdf_threshold=None, chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    out = B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), wl.grid_q, wl.grid_k, **bsa_params)
    assert out.shape == q.shape and out.dtype == q.dtype and out.is_contiguous()
    ref = O.flash_attn_bsa_3d(q, k, v, wl.grid_q, wl.grid_k, **bsa_params)
    _check(out, ref)
    with pytest.raises(AssertionError):
        B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), (8, 12, 21), wl.grid_k, **bsa_params)
    with pytest.raises(ValueError):
        B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), wl.grid_q, wl.grid_k, sparsity=None, cdf_threshold=None,
                            chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])


def test_tc_matches_generic_kernel_at_size():
    """Size-independent property at a benchmark-sized head: both kernels agree, and both runs of one kernel are bit-identical."""
    wl = Workload("480p_one_head", 1002, 1, 1, 128, (24, 32, 52), (24, 32, 52), (4, 4, 4), 0.9375, torch.bfloat16, "scaled_lowrank")
    q, k, v = (t.cuda() for t in make_qkv(wl))
    idx, cnt = B.get_select_indices(q, k, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    assert int(cnt.min()) == int(cnt.max()) == 39
    srt = torch.sort(idx, dim=-1).values
    assert torch.equal(srt, idx) and int((srt[..., 1:] == srt[..., :-1]).sum()) == 0
    a = B.attn_fwd_bsa_varlen(q, k, v, 128 ** -0.5, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, impl=TC)
    a2 = B.attn_fwd_bsa_varlen(q, k, v, 128 ** -0.5, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, impl=TC)
    b = B.attn_fwd_bsa_varlen(q, k, v, 128 ** -0.5, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, impl=MMA)
    L.check(L.lib().lcbsa_check_device_status())
    assert torch.equal(a, a2)
    assert rel_l2(a.float().cpu(), b.float().cpu()) <= REL_L2_TOL
    assert max_abs(a.float().cpu(), b.float().cpu()) <= MAX_ABS_TOL


@pytest.mark.gpu
@pytest.mark.parametrize("heads,chunk_heads", [(6, 4), (5, 2), (3, 8)])
def test_host_entry_point_matches_device_call(heads, chunk_heads):
    """flash_attn_bsa_3d_host (pinned host tensors in and out, pipelined by head chunks) returns exactly what
    flash_attn_bsa_3d returns for the same tensors on the device; repeated calls reuse its staging buffers."""
    grid, chunk = (8, 8, 16), (4, 4, 4)
    S = grid[0] * grid[1] * grid[2]
    g = torch.Generator().manual_seed(11)
    q, k, v = ((torch.randn(1, heads, S, 128, generator=g) * 0.5).to(torch.bfloat16).pin_memory() for _ in range(3))
    kw = dict(sparsity=0.75, chunk_3d_shape_q=list(chunk), chunk_3d_shape_k=list(chunk))
    want = B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), grid, grid, **kw).cpu()
    out = torch.empty_like(want).pin_memory()
    for _ in range(3):
        out.zero_()
        got = B.flash_attn_bsa_3d_host(q, k, v, grid, grid, out=out, heads_per_chunk=chunk_heads, **kw)
        torch.cuda.synchronize()
        assert got is out
        assert torch.equal(out, want)
    L.check(L.lib().lcbsa_check_device_status())
    with pytest.raises(RuntimeError):
        B.flash_attn_bsa_3d_host(q.cuda(), k, v, grid, grid, **kw)


@pytest.mark.gpu
def test_copy_slabs_and_sm_reserve():
    """lcbsa_copy_slabs moves every slab; lcbsa_set_attn_sm_reserve validates its range and returns the old value."""
    import ctypes

    src = torch.arange(8 * 1024, dtype=torch.int32, device="cuda").view(8, 1024)
    dst = torch.zeros_like(src)
    order = [3, 0, 7, 1, 6, 2, 5, 4]
    n = len(order)
    arr = (ctypes.c_void_p * (2 * n))(*[dst[i].data_ptr() for i in range(n)], *[src[j].data_ptr() for j in order])
    base = ctypes.addressof(arr)
    L.check(L.lib().lcbsa_copy_slabs(base, base + n * ctypes.sizeof(ctypes.c_void_p), 1024 * 4, n,
                                     torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(dst, src[order])
    assert L.lib().lcbsa_copy_slabs(None, None, 16, 1, None) == -1
    lib = L.lib()
    old = lib.lcbsa_set_attn_sm_reserve(4)
    assert old >= 0
    assert lib.lcbsa_set_attn_sm_reserve(old) == 4
    assert lib.lcbsa_set_attn_sm_reserve(-1) == -1 and lib.lcbsa_set_attn_sm_reserve(1000) == -1
    assert lib.lcbsa_set_attn_sm_reserve(old) == old
