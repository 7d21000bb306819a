"""This library against the reference's own Triton kernels on the same GPU (comparator, informational parity).

The reference's block-sparse attention (``longcat_video/block_sparse_attention``) is loaded from ``baseline/_ref``
(``baseline/install_reference.py`` puts it there; the directory is not part of this repository).  Where it is absent,
or where this machine's Triton cannot compile the reference's kernels, the tests skip and say why.

  * attention kernel against attention kernel on the SAME block lists: rel-L2 <= 1e-2, max-abs <= 3e-2 (both results
    are bf16 roundings of the same fp32 arithmetic; the reference's launcher is ``attn_fwd_bsa_varlen_triton``,
    bsa_interface.py:290-341, its kernel flash_attn_bsa_varlen_mask.py:172-285);
  * block lists against ``torch.topk`` on CUDA as the reference runs it (bsa_interface.py:212-224): strict set
    equality is reported, equality outside the elements tied with the k-th score is asserted.
"""
import contextlib
import os
import sys

import pytest
import torch

from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import WORKLOADS, Workload, make_qkv
from tests.helpers import max_abs, rel_l2

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def _reference():
    import reference_gpu as R
    with contextlib.redirect_stdout(sys.stderr):
        m = R.load()
    if m is None:
        pytest.skip(f"reference unavailable: {R.why()}")
    return m


def _one_head(name):
    wl = WORKLOADS[name]
    return Workload(wl.name + "_1head", wl.seed, 1, 2, wl.head_dim, wl.grid_q, wl.grid_k, wl.chunk, wl.sparsity, wl.dtype, wl.recipe)


def _block_major(m, x, grid, chunk):
    T, H, W = grid
    t, h, w = chunk
    return m.rearrange_THW_to_3d_block(x, T // t, H // h, W // w, t, h, w, x.shape[-1])


@pytest.mark.parametrize("name", ["480p_legal"])
def test_attention_kernel_against_the_reference_triton_kernel(name):
    m = _reference()
    wl = _one_head(name)
    q, k, v = (t.cuda() for t in make_qkv(wl))
    idx, cnt = B.get_select_indices(q, k, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    ours = B.attn_fwd_bsa_varlen(q, k, v, wl.head_dim ** -0.5, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
    bs = wl.chunk[0] * wl.chunk[1] * wl.chunk[2]
    qb, kb, vb = (_block_major(m, x, g, wl.chunk) for x, g in ((q, wl.grid_q), (k, wl.grid_k), (v, wl.grid_k)))
    try:
        with contextlib.redirect_stdout(sys.stderr):
            o_ref, lse_ref = m.attn_fwd_bsa_varlen_triton(qb, kb, vb, wl.head_dim ** -0.5, idx.long(), cnt, bs, bs, wl.sparsity)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"the reference's Triton kernel does not run here: {e!r}"[:300])
    T, H, W = wl.grid_q
    t, h, w = wl.chunk
    o_ref = m.rearrange_3d_block_to_THW(o_ref, T // t, H // h, W // w, t, h, w, o_ref.shape[-1])
    r, mx = rel_l2(ours.float().cpu(), o_ref.float().cpu()), max_abs(ours.float().cpu(), o_ref.float().cpu())
    print(f"PARITY triton {name}: same lists, rel-L2 {r:.3e} max-abs {mx:.3e}")
    assert r <= 1e-2 and mx <= 3e-2


@pytest.mark.parametrize("name", ["480p_legal", "720p_bucket"])
def test_block_lists_against_cuda_topk(name):
    m = _reference()
    wl = _one_head(name)
    q, k, _ = (t.cuda() for t in make_qkv(wl))
    idx, cnt = B.get_select_indices(q, k, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    qc = B.mean_pooling_compression_3d(q, wl.grid_q, wl.chunk)
    kc = B.mean_pooling_compression_3d(k, wl.grid_k, wl.chunk)
    try:
        with contextlib.redirect_stdout(sys.stderr):
            score = m.cal_score(qc, kc)
            ref_idx, ref_len = m.get_select_indices_topk_from_score(score, wl.sparsity)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"the reference's gating does not run here: {e!r}"[:300])
    nsel = int(cnt.flatten()[0])
    assert int(ref_len.flatten()[0]) == nsel
    ours = torch.zeros_like(score, dtype=torch.bool).scatter_(-1, idx[..., :nsel].long(), True)
    theirs = torch.zeros_like(score, dtype=torch.bool).scatter_(-1, ref_idx.long(), True)
    strict = (ours == theirs).all(-1)
    kth = torch.gather(score, -1, ref_idx).min(-1, keepdim=True).values  # the lowest selected score of the row
    tied = score == kth
    aware = ((ours == theirs) | tied).all(-1)
    print(f"PARITY topk {name}: {int(strict.sum())} of {strict.numel()} rows strictly equal, "
          f"{int(aware.sum())} equal outside the elements tied with the k-th score")
    assert bool(aware.all())


def test_backward_against_the_reference_triton_backward():
    """dq, dk, dv of this library against ``attn_bwd_bsa_varlen_triton`` (bsa_interface.py:343-461) on the SAME block
    lists, forward outputs and dout; tensors go to the reference in its block-major order and come back."""
    m = _reference()
    wl = Workload("bwd_cmp", 7001, 1, 2, 128, (8, 16, 16), (8, 16, 16), (4, 4, 4), 0.75, torch.bfloat16, "normal")
    q, k, v = (t.cuda() for t in make_qkv(wl))
    g = torch.Generator().manual_seed(3)
    do = (torch.randn(q.shape, generator=g) * 0.5).to(q.dtype).cuda()
    idx, cnt = B.get_select_indices(q, k, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    o, lse = B.attn_fwd_bsa_varlen(q, k, v, wl.head_dim ** -0.5, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, return_lse=True)
    dq, dk, dv = B.attn_bwd_bsa_varlen(do, q, k, v, o, lse, wl.head_dim ** -0.5, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
    bs = wl.chunk[0] * wl.chunk[1] * wl.chunk[2]
    T, H, W = wl.grid_q
    t, h, w = wl.chunk
    to_blocks = lambda x: _block_major(m, x, wl.grid_q, wl.chunk).contiguous()  # noqa: E731
    qb, kb, vb, ob, dob = (to_blocks(x) for x in (q, k, v, o, do))
    lse_b = to_blocks(lse.unsqueeze(-1)).squeeze(-1).contiguous()
    rq, rk, rv = torch.empty_like(qb), torch.empty_like(kb), torch.empty_like(vb)
    try:
        with contextlib.redirect_stdout(sys.stderr):
            m.attn_bwd_bsa_varlen_triton(dob, qb, kb, vb, ob, rq, rk, rv, wl.head_dim ** -0.5, lse_b, idx.long(), cnt, bs, bs, wl.sparsity)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"the reference's Triton backward does not run here: {e!r}"[:300])
    back = lambda x: m.rearrange_3d_block_to_THW(x, T // t, H // h, W // w, t, h, w, x.shape[-1])  # noqa: E731
    for name, ours, ref in (("dq", dq, back(rq)), ("dk", dk, back(rk)), ("dv", dv, back(rv))):
        r = rel_l2(ours.float().cpu(), ref.float().cpu())
        print(f"PARITY triton backward {name}: rel-L2 {r:.3e}")
        assert r <= 2e-2, (name, r)
