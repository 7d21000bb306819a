"""Parity of the CUDA block-select stage (through the C ABI) against the CPU oracle.  Bit-exact."""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import WORKLOADS, Workload, make_qkv
from oracle import bsa_oracle as O
from tests.golden.cases import CASES
from tests.helpers import from_bits, load_golden

pytestmark = pytest.mark.gpu

SEEDED = {
    # name: workload   (beyond the golden cases: ragged grids, larger block counts, odd chunks)
    "ragged_bf16": Workload("ragged_bf16", 3001, 1, 2, 128, (5, 7, 9), (6, 7, 10), (4, 4, 4), 0.5, torch.bfloat16, "normal"),
    "ragged_fp16_d64": Workload("ragged_fp16_d64", 3002, 1, 2, 64, (3, 9, 10), (3, 9, 10), (2, 4, 8), 0.75, torch.float16, "normal"),
    "mid_bf16": Workload("mid_bf16", 3003, 1, 2, 128, (8, 20, 28), (8, 20, 28), (4, 4, 4), 0.9375, torch.bfloat16, "scaled_lowrank"),
    "batch2_fp32": Workload("batch2_fp32", 3004, 2, 3, 128, (4, 8, 8), (8, 8, 8), (4, 4, 4), 0.5, torch.float32, "normal"),
    "chunk448_bf16": Workload("chunk448_bf16", 3005, 1, 2, 128, (8, 12, 24), (8, 12, 24), (4, 4, 8), 0.875, torch.bfloat16, "normal"),
}


def _bits(t):
    return t.view(torch.int16) if t.dtype != torch.float32 else t.view(torch.int32)


def _all_workloads():
    out = {n: wl for n, (wl, _) in CASES.items() if n != "bf16_ties_720p"}
    out.update(SEEDED)
    return out


@pytest.fixture(scope="module", params=list(_all_workloads()))
def wl_data(request):
    wl = _all_workloads()[request.param]
    q, k, v = make_qkv(wl)
    return wl, q, k, v


def test_pool_bit_exact(wl_data):
    wl, q, k, _ = wl_data
    for x, grid in ((q, wl.grid_q), (k, wl.grid_k)):
        ref = O.pool(x, grid, wl.chunk)
        got = B.mean_pooling_compression_3d(x.cuda(), grid, wl.chunk).cpu()
        assert torch.equal(_bits(got), _bits(ref))


def test_pool_strided_inputs(wl_data):
    """[B,S,H,D] memory order and a slice of a fused buffer, as attention.py:113-115 produces them."""
    wl, q, k, _ = wl_data
    ref = O.pool(k, wl.grid_k, wl.chunk)
    k_bshd = k.cuda().permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)  # shape [B,H,S,D], memory [B,S,H,D]
    assert k.shape[1] == 1 or not k_bshd.is_contiguous()
    got = B.mean_pooling_compression_3d(k_bshd, wl.grid_k, wl.chunk).cpu()
    assert torch.equal(_bits(got), _bits(ref))
    Bsz, H, S, D = k.shape
    qkv = torch.zeros(Bsz, S, 3, H, D, dtype=k.dtype, device="cuda")
    qkv[:, :, 2] = k.cuda().permute(0, 2, 1, 3)
    k_slice = qkv[:, :, 2].permute(0, 2, 1, 3)
    got = B.mean_pooling_compression_3d(k_slice, wl.grid_k, wl.chunk).cpu()
    assert torch.equal(_bits(got), _bits(ref))


def test_score_topk_bit_exact(wl_data):
    wl, q, k, _ = wl_data
    qc, kc = O.pool(q, wl.grid_q, wl.chunk), O.pool(k, wl.grid_k, wl.chunk)
    sc = O.score(qc, kc)
    nsel = O.num_selected(wl.sparsity, kc.shape[2])
    ref_idx, ref_cnt, _ = O.topk(sc, nsel)
    idx, cnt = B.get_select_indices_from_pooled(qc.cuda(), kc.cuda(), wl.sparsity)
    assert torch.equal(cnt.cpu(), ref_cnt)
    assert torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel])


def test_block_select_end_to_end(wl_data):
    wl, q, k, _ = wl_data
    ref_idx, ref_cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    idx, cnt = B.get_select_indices(q.cuda(), k.cuda(), wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    nsel = int(ref_cnt.flatten()[0])
    assert torch.equal(cnt.cpu(), ref_cnt)
    assert torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel])


@pytest.mark.parametrize("sparsity", [0.0, 0.5, 0.97, 1.0])
def test_topk_extremes(sparsity):
    """nsel = Nk (everything), a middle value, a single block and nsel = 0."""
    wl = SEEDED["mid_bf16"]
    q, k, _ = make_qkv(wl, heads=1)
    qc, kc = O.pool(q, wl.grid_q, wl.chunk), O.pool(k, wl.grid_k, wl.chunk)
    nsel = O.num_selected(sparsity, kc.shape[2])
    ref_idx, ref_cnt, _ = O.topk(O.score(qc, kc), nsel)
    idx, cnt = B.get_select_indices_from_pooled(qc.cuda(), kc.cuda(), sparsity)
    assert torch.equal(cnt.cpu(), ref_cnt)
    if nsel:
        assert torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel])


def test_topk_heavy_ties():
    """Scores drawn from four distinct values: almost every row has a tie across the cut."""
    g = torch.Generator().manual_seed(7)
    Nq, Nk, D = 70, 333, 128
    qc = torch.zeros(1, 2, Nq, D, dtype=torch.bfloat16)
    qc[..., 0] = 1.0
    kc = torch.zeros(1, 2, Nk, D, dtype=torch.bfloat16)
    kc[..., 0] = torch.randint(0, 4, (1, 2, Nk), generator=g).to(torch.bfloat16)
    nsel = O.num_selected(0.7, Nk)
    ref_idx, _, ties = O.topk(O.score(qc, kc), nsel)
    assert int((ties > 0).sum()) > 0
    idx, _ = B.get_select_indices_from_pooled(qc.cuda(), kc.cuda(), 0.7)
    assert torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel])


def test_reference_sets_tie_aware():
    """Against the reference's own CPU top-k at 720p scale: equal sets once boundary ties are set aside."""
    wl, _ = CASES["bf16_ties_720p"]
    gold = load_golden("bf16_ties_720p")
    qc, kc = from_bits(gold["q_cmp"], wl.dtype), from_bits(gold["k_cmp"], wl.dtype)
    nk = kc.shape[2]
    nsel = O.num_selected(wl.sparsity, nk)
    idx, _ = B.get_select_indices_from_pooled(qc.cuda(), kc.cuda(), wl.sparsity)
    idx = idx.cpu()
    sc = O.score(qc, kc).float()
    ref = torch.from_numpy(gold["idx"].astype("int64"))
    strict = 0
    for i in range(idx.shape[2]):
        mine, theirs = set(idx[0, 0, i, :nsel].tolist()), set(ref[0, 0, i].tolist())
        if mine == theirs:
            strict += 1
            continue
        kth = sorted(sc[0, 0, i].tolist(), reverse=True)[nsel - 1]
        assert {j for j in mine if sc[0, 0, i, j] != kth} == {j for j in theirs if sc[0, 0, i, j] != kth}
    print(f"720p bucket grid, 1 head: {strict}/{idx.shape[2]} rows strictly equal to the reference's CPU top-k")


def test_rejects_bad_arguments():
    from longcat_video_b200._lib import LcbsaError
    x = torch.zeros(1, 1, 64, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(LcbsaError):
        B.mean_pooling_compression_3d(x, (4, 4, 5), (4, 4, 4))  # grid does not match S
    with pytest.raises(LcbsaError):
        B.mean_pooling_compression_3d(x[..., :100].contiguous(), (4, 4, 4), (4, 4, 4))  # 200-byte rows
    with pytest.raises(ValueError):
        B.get_select_indices(x, x, (4, 4, 4), (4, 4, 4), None, None, (4, 4, 4), (4, 4, 4))


def _block_select(q, k, grid, chunk, nsel, ws_bytes):
    import ctypes

    qd, kd = L.tensor_desc(q), L.tensor_desc(k)
    g = L.grid_desc(grid, chunk)
    Nq = B.num_blocks(grid, chunk)
    idx = torch.empty(q.shape[0], q.shape[1], Nq, max(nsel, 1), dtype=torch.int32, device=q.device)
    cnt = torch.empty(q.shape[0], q.shape[1], Nq, dtype=torch.int32, device=q.device)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    L.check(L.lib().lcbsa_block_select(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(g), ctypes.byref(g), nsel, max(nsel, 1),
                                       idx.data_ptr(), cnt.data_ptr(), ws.data_ptr(), ws_bytes, L.current_stream(q.device)))
    return idx, cnt


def test_two_kernel_form_equals_fused_form_at_full_size():
    """At the size of the 720p configuration (1440 blocks a side; two heads) the register-tiled GEMM + row-selection
    kernels and the fused kernel return the same lists bit for bit, and both are deterministic.  The form is chosen by
    the size of the workspace handed to lcbsa_block_select."""
    import ctypes

    wl = WORKLOADS["720p_legal"]
    q, k, _ = (t.cuda() for t in make_qkv(wl, heads=2))
    nsel = B.num_selected(wl.sparsity, B.num_blocks(wl.grid_k, wl.chunk))
    qd, kd = L.tensor_desc(q), L.tensor_desc(k)
    g = L.grid_desc(wl.grid_k, wl.chunk)
    small = L.lib().lcbsa_select_workspace_bytes(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(g), ctypes.byref(g))
    big = L.lib().lcbsa_select_workspace_bytes_fast(ctypes.byref(qd), ctypes.byref(kd), ctypes.byref(g), ctypes.byref(g))
    assert big > small > 0
    fused = _block_select(q, k, wl.grid_k, wl.chunk, nsel, small)
    gemm = _block_select(q, k, wl.grid_k, wl.chunk, nsel, big)
    again = _block_select(q, k, wl.grid_k, wl.chunk, nsel, big)
    torch.cuda.synchronize()
    assert torch.equal(fused[0], gemm[0]) and torch.equal(fused[1], gemm[1])
    assert torch.equal(gemm[0], again[0])
    lists = gemm[0]
    assert int(gemm[1].min()) == nsel == int(gemm[1].max())
    assert bool((lists[..., 1:] > lists[..., :-1]).all()) and int(lists.min()) >= 0 and int(lists.max()) < 1440
