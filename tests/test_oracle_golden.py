"""Pin the CPU oracle against fixtures produced by the reference's own PyTorch code
(tests/golden/make_golden.py).  CPU only."""
import pytest
import torch

from longcat_video_b200.synthetic import make_qkv
from oracle import bsa_oracle as O
from tests.golden.cases import CASES
from tests.helpers import from_bits, load_golden, max_abs, rel_l2


@pytest.fixture(scope="module", params=list(CASES))
def case(request):
    wl, has_attn = CASES[request.param]
    gold = load_golden(request.param)
    q, k, v = make_qkv(wl)
    chk = [q.double().sum().item(), k.double().sum().item(), v.double().sum().item()]
    assert chk == pytest.approx(list(gold["checksum"]), rel=1e-12, abs=1e-9), "seeded inputs drifted"
    return wl, has_attn, gold, (q, k, v)


def test_pool_matches_reference(case):
    wl, _, gold, (q, k, _) = case
    for x, grid, key in ((q, wl.grid_q, "q_cmp"), (k, wl.grid_k, "k_cmp")):
        mine = O.pool(x, grid, wl.chunk)
        ref = from_bits(gold[key], wl.dtype)
        if wl.dtype == torch.float32:
            # fp32 sums of fp32 values depend on the order; the reference's order is the library's
            assert max_abs(mine, ref) < 2e-6
        else:
            # 64..128 half-precision values: the fp32 running sum is exact or within one fp32 ulp, so
            # the rounded result agrees bit for bit (any mismatch would be reported here)
            assert torch.equal(mine.view(torch.int16), ref.view(torch.int16))


def test_score_matches_reference(case):
    wl, _, gold, _ = case
    if "score" not in gold:
        pytest.skip("scores not stored for this case")
    qc, kc = from_bits(gold["q_cmp"], wl.dtype), from_bits(gold["k_cmp"], wl.dtype)
    mine = O.score(qc, kc)
    ref = from_bits(gold["score"], wl.dtype)
    if wl.dtype == torch.float32:
        assert max_abs(mine, ref) < 1e-5
    else:
        # the fp32 accumulation order of the library GEMM differs from the oracle's FMA chain: allow the
        # last place of the 16-bit result to differ in a small fraction of entries
        diff = (mine.view(torch.int16).int() - ref.view(torch.int16).int()).abs()
        assert int(diff.max()) <= 1
        assert float((diff != 0).float().mean()) < 5e-3


def _tie_aware_equal(mine_row, ref_row, score_row, nsel):
    """Sets agree after removing the entries whose score equals the nsel-th largest score."""
    if sorted(mine_row) == sorted(ref_row):
        return True, True
    kth = sorted(score_row.tolist(), reverse=True)[nsel - 1]
    a = {i for i in mine_row if score_row[i] != kth}
    b = {i for i in ref_row if score_row[i] != kth}
    return False, a == b


def test_topk_sets_match_reference(case):
    wl, _, gold, _ = case
    qc, kc = from_bits(gold["q_cmp"], wl.dtype), from_bits(gold["k_cmp"], wl.dtype)
    # score with the reference's own GEMM so that only the tie rule is under test here
    sc = torch.matmul(qc, kc.transpose(-1, -2))
    nk = kc.shape[2]
    nsel = O.num_selected(wl.sparsity, nk)
    ref_idx = torch.from_numpy(gold["idx"].astype("int64"))
    assert ref_idx.shape[-1] == nsel
    assert int(gold["lens"].min()) == nsel and int(gold["lens"].max()) == nsel
    idx, cnt, ties = O.topk(sc, nsel)
    assert int(cnt.min()) == nsel and int(cnt.max()) == nsel
    B, H, Nq, _ = idx.shape
    strict = tie_ok = rows = tied_rows = 0
    scf = sc.float()
    for b in range(B):
        for h in range(H):
            for i in range(Nq):
                mine = idx[b, h, i, :nsel].tolist()
                assert mine == sorted(mine) and len(set(mine)) == nsel
                s, t = _tie_aware_equal(mine, ref_idx[b, h, i].tolist(), scf[b, h, i], nsel)
                strict += s
                tie_ok += t
                rows += 1
                tied_rows += int(ties[b, h, i] > 0)
                if not s:
                    assert ties[b, h, i] > 0, "sets differ on a row without a boundary tie"
    assert tie_ok == rows
    print(f"{wl.name}: rows={rows} strict_equal={strict} boundary_tie_rows={tied_rows}")
    if wl.dtype == torch.float32:
        assert strict == rows


def test_attention_matches_reference(case):
    wl, has_attn, gold, (q, k, v) = case
    if not has_attn:
        pytest.skip("selection-only case")
    # use the reference's own lists so that only the attention arithmetic is compared
    ref_idx = torch.from_numpy(gold["idx"].astype("int32"))
    idx = torch.sort(ref_idx, dim=-1).values.contiguous()
    cnt = torch.from_numpy(gold["lens"].astype("int32"))
    out, lse = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx, cnt)
    ref = torch.from_numpy(gold["attn"])
    assert rel_l2(out, ref) < 2e-6
    assert max_abs(out, ref) < 2e-5
    assert torch.isfinite(lse).all()


def test_end_to_end_signature(case):
    wl, has_attn, gold, (q, k, v) = case
    if not has_attn:
        pytest.skip("selection-only case")
    out = O.flash_attn_bsa_3d(q, k, v, wl.grid_q, wl.grid_k, sparsity=wl.sparsity,
                              chunk_3d_shape_q=wl.chunk, chunk_3d_shape_k=wl.chunk)
    ref = torch.from_numpy(gold["attn"])
    # the oracle's own selection may differ from the reference's on tied rows only
    assert rel_l2(out, ref) < 5e-2
