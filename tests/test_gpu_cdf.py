"""The cdf_threshold selectors on the GPU (lcbsa_score_cdf) against the CPU oracle, bit for bit, against the fixtures
produced by the reference's functions (longcat_video/block_sparse_attention/bsa_interface.py:226-266), and through the
whole forward ``flash_attn_bsa_3d(..., cdf_threshold=...)``."""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import Workload, make_qkv
from oracle import bsa_oracle as O
from tests.test_oracle_cdf import NAMES, check_against_reference, load, nsel_min

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", NAMES)
def test_kernel_equals_oracle_and_reference_fixture(name):
    c = load(name)
    idx, cnt = B.get_select_indices_from_pooled(c["q"].cuda(), c["k"].cuda(), c["sparsity"], c["thr"])
    torch.cuda.synchronize()
    assert idx.dtype == torch.int32 and idx.shape[-1] == c["Nk"]
    want_idx, want_cnt = O.cdf_select(O.score(c["q"], c["k"]), c["thr"], c["scale"], nsel_min(c))
    assert torch.equal(cnt.cpu(), want_cnt)
    assert torch.equal(idx.cpu(), want_idx)
    check_against_reference(c, idx, cnt)


@pytest.mark.parametrize("nk,thr,nmin", [(1, 0.5, 0), (2, 0.5, 0), (33, 2.0, 0), (64, 0.0, 0), (65, 0.0, 7), (257, 0.8, 0), (1000, 0.99, 100), (2048, 0.9, 0), (2500, 0.7, 0)])
def test_edge_sizes_and_thresholds(nk, thr, nmin):
    """Rows shorter than a warp, rows that are not a power of two, rows above 2048 entries (the shared-memory form of the
    kernel), thresholds nothing or everything exceeds."""
    g = torch.Generator().manual_seed(nk)
    q = torch.randn(1, 2, 9, 64, generator=g).bfloat16()
    k = torch.randn(1, 2, nk, 64, generator=g).bfloat16()
    sparsity = None if nmin == 0 else 1 - (nmin + 0.5) / nk
    assert nmin == (0 if sparsity is None else B.num_selected(sparsity, nk))
    idx, cnt = B.get_select_indices_from_pooled(q.cuda(), k.cuda(), sparsity, thr)
    want_idx, want_cnt = O.cdf_select(O.score(q, k), thr, 1 / 64 ** 0.5, nmin)
    assert torch.equal(cnt.cpu(), want_cnt) and torch.equal(idx.cpu(), want_idx)
    if thr >= 1.5:
        assert bool((cnt == nk).all())
    if thr == 0.0:
        assert bool((cnt == nmin).all())


@pytest.mark.parametrize("sparsity,thr", [(None, 0.6), (None, 0.95), (0.75, 0.3), (None, 0.0)])
def test_forward_with_cdf_threshold_matches_oracle(sparsity, thr):
    wl = Workload("cdf_small", 21, 1, 3, 128, (8, 8, 16), (8, 8, 16), (4, 4, 4), 0.75, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    # a common offset per 3-D block, so that pooled rows differ and the lists have different lengths
    g = torch.Generator().manual_seed(22)
    tm = O.token_map(wl.grid_q, wl.chunk)
    for x in (q, k):
        off = (torch.randn(1, wl.heads, tm.shape[0], 1, wl.head_dim, generator=g) * 1.5).expand(-1, -1, -1, tm.shape[1], -1)
        x[:, :, tm.reshape(-1)] = (x[:, :, tm.reshape(-1)].float() + off.reshape(1, wl.heads, -1, wl.head_dim)).to(x.dtype)
    got = B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), wl.grid_q, wl.grid_k, sparsity=sparsity, cdf_threshold=thr,
                              chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    want = O.flash_attn_bsa_3d(q, k, v, wl.grid_q, wl.grid_k, sparsity, thr, wl.chunk, wl.chunk)
    got = got.float().cpu()
    if thr == 0.0 and sparsity is None:
        assert float(got.abs().max()) == 0.0 and float(want.abs().max()) == 0.0  # empty lists: zeros, as in the reference kernel
        return
    rel = float((got - want).norm() / want.norm())
    assert rel <= 1e-2 and float((got - want).abs().max()) <= 3e-2, rel  # the tolerances of the top-k forward tests


def test_full_size_properties():
    """720p block counts (1440 x 1440 per head, 8 heads): every row is a permutation, the order does not depend on the
    threshold, the count grows with the threshold and respects the top-k floor."""
    g = torch.Generator(device="cuda").manual_seed(5)
    H, N, D = 8, 1440, 128
    q = (torch.randn(1, H, N, D, generator=g, device="cuda") * 0.8).bfloat16()
    k = (torch.randn(1, H, N, D, generator=g, device="cuda") * 0.8).bfloat16()
    idx_a, cnt_a = B.get_select_indices_from_pooled(q, k, None, 0.5)
    idx_b, cnt_b = B.get_select_indices_from_pooled(q, k, None, 0.9)
    idx_c, cnt_c = B.get_select_indices_from_pooled(q, k, 0.9375, 0.5)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    assert torch.equal(idx_a, idx_b) and torch.equal(idx_a, idx_c)
    assert torch.equal(idx_a.sort(-1).values, torch.arange(N, device="cuda", dtype=torch.int32).expand_as(idx_a))
    assert bool((cnt_b >= cnt_a).all()) and bool((cnt_a >= 1).all()) and bool((cnt_b < N).all())
    assert torch.equal(cnt_c, cnt_a.clamp(min=90))
    # the weights the rows point at do not increase: recompute them for one head with torch
    w = torch.softmax((q[0, 0].float() @ k[0, 0].float().T).bfloat16() * (1 / D ** 0.5), dim=-1)
    ws = torch.gather(w, -1, idx_a[0, 0].long()).float()
    assert float((ws[:, 1:] - ws[:, :-1]).max()) <= 2 ** -7 * float(ws.max())  # up to a rounding step of the largest weight
