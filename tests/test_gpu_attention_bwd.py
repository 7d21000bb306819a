"""Parity of the CUDA backward of the block-sparse attention (through the C ABI) against the CPU oracle
(oracle/bsa_backward.py: float64 autograd through the masked-softmax attention with the block lists held fixed).

Tolerance (bf16 / fp16 gradients against the float64 oracle on the same 16-bit inputs): rel-L2 <= 1e-2 per gradient.
"""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import Workload, make_qkv
from oracle import bsa_backward as OB
from oracle import bsa_oracle as O
from tests.helpers import rel_l2

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2

CASES = {
    "blocks64_bf16": Workload("blocks64_bf16", 6001, 1, 2, 128, (8, 8, 16), (8, 8, 16), (4, 4, 4), 0.5, torch.bfloat16, "normal"),
    "blocks128_bf16": Workload("blocks128_bf16", 6002, 1, 2, 128, (8, 8, 16), (8, 8, 16), (4, 4, 8), 0.5, torch.bfloat16, "normal"),
    "d64_fp16": Workload("d64_fp16", 6003, 2, 2, 64, (4, 8, 16), (4, 8, 16), (4, 4, 4), 0.5, torch.float16, "normal"),
    "cross_ragged_bf16": Workload("cross_ragged_bf16", 6004, 1, 2, 128, (5, 7, 9), (6, 7, 10), (4, 4, 4), 0.5, torch.bfloat16, "normal"),
    "sparse_bf16": Workload("sparse_bf16", 6005, 1, 1, 128, (8, 16, 16), (8, 16, 16), (4, 4, 4), 0.875, torch.bfloat16, "scaled_lowrank"),
}


def _dout(wl, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(wl.batch, wl.heads, wl.sq, wl.head_dim, generator=g) * 0.5).to(wl.dtype)


def _forward_and_backward(wl, q, k, v, do, idx, cnt, chunk_k=None):
    chunk_k = chunk_k or wl.chunk
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o, lse = B.attn_fwd_bsa_varlen(qd, kd, vd, wl.head_dim ** -0.5, idx.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k, wl.chunk, chunk_k,
                                   return_lse=True)
    L.lib().lcbsa_check_device_status()
    dq, dk, dv = B.attn_bwd_bsa_varlen(do.cuda(), qd, kd, vd, o, lse, wl.head_dim ** -0.5, idx.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k,
                                       wl.chunk, chunk_k)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    return o, dq, dk, dv


def _compare(name, got, want):
    out = []
    for n, g, w in zip(("dq", "dk", "dv"), got, want):
        g = g.float().cpu()
        assert torch.isfinite(g).all(), f"{name} {n} not finite"
        r = rel_l2(g, w)
        assert r <= REL_L2_TOL, f"{name} {n} rel-L2 {r}"
        out.append(f"{n} {r:.2e}")
    return ", ".join(out)


@pytest.mark.parametrize("name", list(CASES))
def test_gradients_against_oracle(name):
    wl = CASES[name]
    q, k, v = make_qkv(wl)
    do = _dout(wl, 17)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    _, rq, rk, rv = OB.attention_backward(q, k, v, do, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
    _, dq, dk, dv = _forward_and_backward(wl, q, k, v, do, idx, cnt)
    print(f"BWD PARITY {name}:", _compare(name, (dq, dk, dv), (rq, rk, rv)))


def test_key_blocks_of_another_size_than_query_blocks():
    wl = Workload("mixed", 6006, 1, 2, 128, (8, 8, 16), (8, 8, 16), (4, 4, 4), 0.5, torch.bfloat16, "normal")
    chunk_k = (4, 4, 8)
    q, k, v = make_qkv(wl)
    do = _dout(wl, 18)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, chunk_k)
    _, rq, rk, rv = OB.attention_backward(q, k, v, do, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, chunk_k)
    _, dq, dk, dv = _forward_and_backward(wl, q, k, v, do, idx, cnt, chunk_k=chunk_k)
    print("BWD PARITY mixed:", _compare("mixed", (dq, dk, dv), (rq, rk, rv)))


def test_lists_of_different_lengths_empty_lists_and_unselected_key_blocks():
    """Rows of a query block with an empty list get dq = 0; key blocks that nothing selected get dk = dv = 0."""
    wl = CASES["blocks64_bf16"]
    q, k, v = make_qkv(wl)
    do = _dout(wl, 19)
    nq = nk = O.num_blocks(wl.grid_q, wl.chunk)
    g = torch.Generator().manual_seed(5)
    cap = 6
    cnt = torch.randint(0, cap + 1, (1, 2, nq), generator=g, dtype=torch.int32)
    cnt[0, 0, 0] = 0
    idx = torch.full((1, 2, nq, cap), -1, dtype=torch.int32)
    for h in range(2):
        for i in range(nq):
            n = int(cnt[0, h, i])
            idx[0, h, i, :n] = torch.sort(torch.randperm(nk - 2, generator=g)[:n]).values.to(torch.int32)  # the last two key blocks stay unselected
    _, rq, rk, rv = OB.attention_backward(q, k, v, do, idx.clamp_min(0), cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
    _, dq, dk, dv = _forward_and_backward(wl, q, k, v, do, idx.clamp_min(0), cnt)
    print("BWD PARITY ragged lists:", _compare("lists", (dq, dk, dv), (rq, rk, rv)))
    tm = O.token_map(wl.grid_k, wl.chunk)
    for blk in (nk - 2, nk - 1):
        assert float(dk[0, :, tm[blk]].float().abs().max()) == 0.0 and float(dv[0, :, tm[blk]].float().abs().max()) == 0.0
    assert float(dq[0, 0, O.token_map(wl.grid_q, wl.chunk)[0]].float().abs().max()) == 0.0


def test_autograd_through_the_entry_point_and_determinism():
    """flash_attn_bsa_3d with tensors that require grad goes through the autograd function; two runs give the same bits."""
    wl = CASES["blocks128_bf16"]
    q, k, v = make_qkv(wl)
    do = _dout(wl, 20).cuda()
    grads = []
    for _ in range(2):
        qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
        out = B.flash_attn_bsa_3d(qd, kd, vd, wl.grid_q, wl.grid_k, sparsity=wl.sparsity, chunk_3d_shape_q=list(wl.chunk),
                                  chunk_3d_shape_k=list(wl.chunk))
        out.backward(do)
        grads.append((qd.grad.clone(), kd.grad.clone(), vd.grad.clone()))
    for a, b in zip(*grads):
        assert torch.equal(a, b)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    _, rq, rk, rv = OB.attention_backward(q, k, v, do.cpu(), idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
    print("BWD PARITY autograd:", _compare("autograd", grads[0], (rq, rk, rv)))
    with torch.no_grad():
        plain = B.flash_attn_bsa_3d(q.cuda(), k.cuda(), v.cuda(), wl.grid_q, wl.grid_k, sparsity=wl.sparsity,
                                    chunk_3d_shape_q=list(wl.chunk), chunk_3d_shape_k=list(wl.chunk))
    assert torch.equal(plain, out.detach())
