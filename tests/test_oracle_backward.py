"""The backward oracle (oracle/bsa_backward.py) against the forward oracle and against finite differences (CPU)."""
import torch

from longcat_video_b200.synthetic import Workload, make_qkv
from oracle import bsa_backward as OB
from oracle import bsa_oracle as O


def test_forward_of_the_backward_oracle_equals_the_forward_oracle():
    wl = Workload("bwd_oracle", 6100, 1, 2, 128, (5, 7, 9), (6, 7, 10), (4, 4, 4), 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    do = torch.ones(1, 2, wl.sq, 128)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    o, dq, dk, dv = OB.attention_backward(q, k, v, do, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
    ref, _ = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx, cnt)
    assert float((o - ref.double()).norm() / ref.double().norm()) < 1e-6
    assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape


def test_gradients_against_finite_differences():
    wl = Workload("bwd_fd", 6101, 1, 1, 16, (4, 4, 8), (4, 4, 8), (4, 4, 4), 0.5, torch.float32, "normal")
    q, k, v = (t.double() for t in make_qkv(wl))
    g = torch.Generator().manual_seed(1)
    do = torch.randn(q.shape, generator=g, dtype=torch.float64)
    idx, cnt, _, _ = O.block_select(q.float(), k.float(), wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    _, dq, dk, dv = OB.attention_backward(q, k, v, do, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)

    def loss(q_, k_, v_):
        o, *_ = OB.attention_backward(q_, k_, v_, do, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
        return float((o * do).sum())

    eps = 1e-5
    for name, x, gx in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        for pos in [(0, 0, 3, 5), (0, 0, 77, 0), (0, 0, 127, 15)]:
            xp, xm = x.clone(), x.clone()
            xp[pos] += eps
            xm[pos] -= eps
            args_p = [xp if n == name else t for n, t in (("q", q), ("k", k), ("v", v))]
            args_m = [xm if n == name else t for n, t in (("q", q), ("k", k), ("v", v))]
            fd = (loss(*args_p) - loss(*args_m)) / (2 * eps)
            assert abs(fd - float(gx[pos])) <= 1e-6 * max(1.0, abs(fd)), (name, pos, fd, float(gx[pos]))


# ---- pinned on the reference: gradients of the reference's CPU path under torch autograd (tests/golden/make_golden_backward.py)

import os  # noqa: E402

import numpy as np  # noqa: E402
import pytest  # noqa: E402

from tests.golden.cases import BWD_CASES, make_dout  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_backward_fixture(name):
    wl = BWD_CASES[name]
    f = np.load(os.path.join(GOLDEN, name + ".npz"))
    q, k, v = make_qkv(wl)
    do = make_dout(wl)
    got = [q.double().sum().item(), k.double().sum().item(), v.double().sum().item(), do.double().sum().item()]
    assert np.allclose(f["checksum"], got, rtol=0, atol=0), "the seeded inputs are not the ones the fixture was made from"
    idx = torch.sort(torch.from_numpy(f["idx"].astype("int32")), dim=-1).values.contiguous()
    cnt = torch.from_numpy(f["lens"].astype("int32"))
    grads = tuple(torch.from_numpy(f[n]) for n in ("dq", "dk", "dv"))
    return wl, q, k, v, do, idx, cnt, grads


@pytest.mark.parametrize("name", list(BWD_CASES))
def test_backward_oracle_against_the_reference_fixtures(name):
    """The float64 oracle on the reference's lists against the fp32 gradients that torch autograd took through the
    reference's own block mask and scaled_dot_product_attention: rel-L2 <= 1e-5 (fp32 against float64 arithmetic)."""
    wl, q, k, v, do, idx, cnt, want = load_backward_fixture(name)
    _, dq, dk, dv = OB.attention_backward(q, k, v, do, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk)
    for n, g, w in zip(("dq", "dk", "dv"), (dq, dk, dv), want):
        r = float((g.double() - w.double()).norm() / w.double().norm())
        assert r <= 1e-5, f"{name} {n}: rel-L2 {r}"
