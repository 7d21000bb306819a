"""The CPU oracle of the cdf_threshold selectors against fixtures produced by the reference's own functions
(tests/golden/make_golden_cdf.py: get_select_indices_cdf_from_score and get_select_indices_cdf_topk_from_score of
longcat_video/block_sparse_attention/bsa_interface.py:234-266).  Counts must agree exactly; the sorted index rows must
point at the same sequence of weights (torch.sort leaves the order of equal weights open, the oracle orders them by
ascending index; its exp and summation order are its own, so a weight can land on the neighbouring value and swap two
entries)."""
import os

import numpy as np
import pytest
import torch

from oracle import bsa_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
NAMES = ["cdf_nk360", "cdf_nk360_peaked", "cdf_topk_nk1440", "cdf_nk100_d64_fp16", "cdf_topk_nk24"]


def load(name):
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    H, Nq, Nk, D, is_fp16 = (int(v) for v in z["meta"])
    dtype = torch.float16 if is_fp16 else torch.bfloat16
    t = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(dtype)  # noqa: E731
    thr, sparsity, scale = (float(v) for v in z["params"])
    return dict(q=t(z["q"]), k=t(z["k"]), score=t(z["score"]), weights=t(z["weights"]), idx=torch.from_numpy(z["idx"].astype(np.int64)),
                lens=torch.from_numpy(z["lens"]), thr=thr, sparsity=None if sparsity < 0 else sparsity, scale=scale, Nk=Nk)


def check_against_reference(c, idx, cnt):
    """idx int32 [1,H,Nq,Nk], cnt int32 [1,H,Nq] from the oracle or the kernel."""
    assert torch.equal(cnt.cpu(), c["lens"].int())
    idx = idx.cpu().long()
    assert torch.equal(idx.sort(-1).values, torch.arange(c["Nk"]).expand_as(idx))  # every row is a permutation
    w = c["weights"].view(torch.int16)
    # the same sequence of weights; where the oracle's exp or its summation order moves a weight to the neighbouring
    # value of the dtype, two entries may change places
    mine, ref = torch.gather(w, -1, idx).int(), torch.gather(w, -1, c["idx"]).int()
    assert float((mine == ref).float().mean()) > 0.999
    assert int((mine - ref).abs().max()) <= 1


def nsel_min(c):
    return 0 if c["sparsity"] is None else int((1 - c["sparsity"]) * c["Nk"])


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference_selector(name):
    c = load(name)
    # the selector is pinned on the reference's own score bits; the oracle's scores (one fmaf chain per entry) differ from
    # the reference's matmul only where the summation order changes the rounding
    same = (O.score(c["q"], c["k"]).view(torch.int16) == c["score"].view(torch.int16)).float().mean().item()
    assert same > 0.99, same
    idx, cnt = O.cdf_select(c["score"], c["thr"], c["scale"], nsel_min(c))
    check_against_reference(c, idx, cnt)


def test_threshold_extremes():
    g = torch.Generator().manual_seed(0)
    score = (torch.randn(1, 1, 8, 40, generator=g) * 4).bfloat16()
    _, cnt = O.cdf_select(score, 2.0, 0.1)  # nothing exceeds it: the whole row
    assert bool((cnt == 40).all())
    _, cnt = O.cdf_select(score, 0.0, 0.1)  # the first weight already exceeds it: empty lists
    assert bool((cnt == 0).all())
    _, cnt = O.cdf_select(score, 0.0, 0.1, 5)
    assert bool((cnt == 5).all())
