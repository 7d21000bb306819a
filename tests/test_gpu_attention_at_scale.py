"""Parity of the tcgen05 attention kernel against the CPU oracle at the sizes that are benchmarked.

One head of each benchmark configuration goes through the whole CUDA path (block-select, then attention with the
kernel that LCBSA_ATTN_AUTO picks); the block lists are compared with the oracle's over the whole head, bit for bit,
and the attention output with the oracle's exact-softmax fp32 result on a spread-out sample of query blocks (the
oracle is a scalar double-precision loop: a whole 720p head would take it half a minute, a sample takes seconds).
The kernel itself always computes the whole head.  Also here: block lists of 15 .. 48 entries on a small grid (the
lengths at which the kernel's producer warp refills its window of decoded block coordinates), lists whose two tiles of
a query-block pair differ in length, and a cdf_threshold forward whose lists are longer than 32 entries.

Tolerance (bf16 result against the fp32 oracle): rel-L2 <= 1e-2, max-abs <= 3e-2, LSE abs <= 2e-2.
"""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import bsa_interface as B
from longcat_video_b200.synthetic import WORKLOADS, Workload, make_qkv
from oracle import bsa_oracle as O
from tests.helpers import max_abs, rel_l2

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-2
MAX_ABS_TOL = 3e-2
LSE_TOL = 2e-2


def _one_head(wl: Workload, **kw) -> Workload:
    d = dict(name=wl.name + "_1head", seed=wl.seed, batch=1, heads=1, head_dim=wl.head_dim, grid_q=wl.grid_q, grid_k=wl.grid_k,
             chunk=wl.chunk, sparsity=wl.sparsity, dtype=wl.dtype, recipe=wl.recipe)
    d.update(kw)
    return Workload(**d)


def _sample_blocks(nq: int, n_sample: int):
    """First, last and evenly spread query blocks, with neighbours so that both tiles of some pairs are covered."""
    n_sample = max(2, min(n_sample, nq))
    step = max(1, nq // n_sample)
    picks = set(range(0, nq, step)) | {nq - 1, nq - 2 if nq > 1 else 0, 1 if nq > 1 else 0}
    return sorted(picks)


def _compare_on_sample(wl, q, k, v, idx_dev, cnt_dev, out_dev, lse_dev, n_sample):
    """Oracle attention on the sampled query blocks only (cnt = 0 elsewhere is skipped by the oracle at once)."""
    nq = O.num_blocks(wl.grid_q, wl.chunk)
    picks = _sample_blocks(nq, n_sample)
    idx, cnt = idx_dev.cpu(), cnt_dev.cpu()
    masked = torch.zeros_like(cnt)
    masked[..., picks] = cnt[..., picks]
    ref, ref_lse = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx.clamp_min(0).contiguous(), masked)
    tm = O.token_map(wl.grid_q, wl.chunk)[picks].reshape(-1)
    tok = tm[tm >= 0]
    got, want = out_dev.float().cpu()[:, :, tok], ref[:, :, tok]
    assert torch.isfinite(got).all()
    r, m = rel_l2(got, want), max_abs(got, want)
    le = float((lse_dev.cpu()[:, :, tok] - ref_lse[:, :, tok]).abs().max())
    assert r <= REL_L2_TOL, f"rel-L2 {r}"
    assert m <= MAX_ABS_TOL, f"max-abs {m}"
    assert le <= LSE_TOL, f"lse {le}"
    return r, m, le, len(picks)


def _run_config(wl, n_sample, allow_ragged=False):
    q, k, v = make_qkv(wl)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    idx, cnt = B.get_select_indices(qd, kd, wl.grid_q, wl.grid_k, wl.sparsity, None, wl.chunk, wl.chunk)
    ref_idx, ref_cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    nsel = int(ref_cnt.flatten()[0])
    assert torch.equal(cnt.cpu(), ref_cnt)
    assert torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel]), "block lists differ from the oracle's"
    out, lse = B.attn_fwd_bsa_varlen(qd, kd, vd, wl.head_dim ** -0.5, idx, cnt, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk,
                                     return_lse=True, impl=L.ATTN_TC)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    r, m, le, n = _compare_on_sample(wl, q, k, v, idx, cnt, out, lse, n_sample)
    # the drop-in entry point returns the same bits
    whole = B.flash_attn_bsa_3d(qd, kd, vd, wl.grid_q, wl.grid_k, sparsity=wl.sparsity, chunk_3d_shape_q=list(wl.chunk),
                                chunk_3d_shape_k=list(wl.chunk), allow_ragged=allow_ragged)
    assert torch.equal(whole, out)
    print(f"PARITY {wl.name}: selected {nsel} of {O.num_blocks(wl.grid_k, wl.chunk)}, lists bit-exact, "
          f"{n} query blocks sampled: rel-L2 {r:.3e} max-abs {m:.3e} lse {le:.3e}")


@pytest.mark.parametrize("name,n_sample", [("480p_legal", 80), ("720p_legal", 60), ("720p_bucket", 60), ("720p_ragged", 60),
                                           ("480p_ragged", 80), ("vc_legal", 60), ("vc_ragged", 60),
                                           ("480p_blocks128", 40), ("720p_blocks128", 30), ("720p_defaults", 30)])
def test_one_head_of_benchmark_configs(name, n_sample):
    """k = 39 (480p), 90 (720p legal and ragged), 82 (720p bucket); the vc shapes have Tq = 12 / 11 against Tk = 24.  The
    last three run the 128-token kernel: [4, 4, 8] blocks at the headline's sparsity (21 of 336, 45 of 720 blocks) and with
    every parameter of the entry point at its default (90 of 720)."""
    wl = _one_head(WORKLOADS[name])
    ragged = any(g % c for grid in (wl.grid_q, wl.grid_k) for g, c in zip(grid, wl.chunk))
    _run_config(wl, n_sample, allow_ragged=ragged)


@pytest.mark.parametrize("sparsity,n_sample", [(0.5, 6), (0.75, 12), (0.875, 24), (0.9375, 48), (0.96875, 64)])
def test_sparsity_sweep_on_continuation_shape(sparsity, n_sample):
    """Video continuation: 12 generated frames attend to 24 (12 conditioning + 12 generated); k = 720 ... 45 of 1440."""
    wl = _one_head(WORKLOADS["vc_legal"], sparsity=sparsity, name=f"vc_legal_s{sparsity}")
    _run_config(wl, n_sample)


def test_ragged_grid_21x45x79():
    """Every axis ragged: 21 % 4 = 1, 45 % 4 = 1, 79 % 4 = 3 -- edge blocks hold 1/4, 1/4 and 3/4 of their rows."""
    wl = Workload("ragged_21x45x79", 1005, 1, 1, 128, (21, 45, 79), (21, 45, 79), (4, 4, 4), 0.9375, torch.bfloat16, "normal")
    _run_config(wl, 60, allow_ragged=True)


@pytest.mark.parametrize("length", [1, 2, 3, 15, 16, 17, 31, 32, 33, 47, 48])
@pytest.mark.parametrize("pattern", ["equal", "pair_differs"])
def test_list_lengths_around_the_window_refill(length, pattern):
    """Random ascending lists of exactly `length` entries ("equal"), or `length` for the first and a shorter list for
    the second query block of every pair ("pair_differs": one tile of the pair runs out of blocks before the other)."""
    wl = Workload("lists", 4100 + length, 1, 2, 128, (12, 16, 16), (12, 16, 16), (4, 4, 4), 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    nq, nk = O.num_blocks(wl.grid_q, wl.chunk), O.num_blocks(wl.grid_k, wl.chunk)
    assert nk == 48
    g = torch.Generator().manual_seed(length)
    cnt = torch.full((1, 2, nq), length, dtype=torch.int32)
    if pattern == "pair_differs":
        cnt[..., 1::2] = max(length - 5, 0)
        cnt[0, 1, 0::2] = max(length - 18, 1)  # and the other way round in the second head
        cnt[0, 1, 1::2] = length
    idx = torch.full((1, 2, nq, 48), -1, dtype=torch.int32)
    for h in range(2):
        for i in range(nq):
            n = int(cnt[0, h, i])
            idx[0, h, i, :n] = torch.sort(torch.randperm(nk, generator=g)[:n]).values.to(torch.int32)
    ref, ref_lse = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx.clamp_min(0).contiguous(), cnt)
    out, lse = B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), wl.head_dim ** -0.5, idx.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k,
                                     wl.chunk, wl.chunk, return_lse=True, impl=L.ATTN_TC)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    assert rel_l2(got, ref) <= REL_L2_TOL and max_abs(got, ref) <= MAX_ABS_TOL
    fin = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse.cpu()), fin)
    assert float((lse.cpu()[fin] - ref_lse[fin]).abs().max()) <= LSE_TOL


def test_cdf_forward_with_long_lists():
    """cdf_threshold forward on 180 key blocks: descending-weight lists of very different lengths, most above 32."""
    wl = Workload("cdf_long", 4200, 1, 2, 128, (12, 24, 40), (12, 24, 40), (4, 4, 4), 0.9, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    g = torch.Generator().manual_seed(7)
    tm = O.token_map(wl.grid_q, wl.chunk)
    for x in (q, k):  # a common offset per block so that pooled rows, and with them the list lengths, differ
        off = (torch.randn(1, wl.heads, tm.shape[0], 1, wl.head_dim, generator=g) * 0.6).expand(-1, -1, -1, tm.shape[1], -1)
        x[:, :, tm.reshape(-1)] = (x[:, :, tm.reshape(-1)].float() + off.reshape(1, wl.heads, -1, wl.head_dim)).to(x.dtype)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    idx, cnt = B.get_select_indices(qd, kd, wl.grid_q, wl.grid_k, None, 0.9, wl.chunk, wl.chunk)
    qc, kc = O.pool(q, wl.grid_q, wl.chunk), O.pool(k, wl.grid_k, wl.chunk)
    want_idx, want_cnt = O.cdf_select(O.score(qc, kc), 0.9, wl.head_dim ** -0.5, 0)
    assert torch.equal(cnt.cpu(), want_cnt) and torch.equal(idx.cpu(), want_idx)
    assert int(cnt.max()) > 32 and float((cnt > 32).float().mean()) > 0.5, "the case is meant to have long lists"
    got = B.flash_attn_bsa_3d(qd, kd, vd, wl.grid_q, wl.grid_k, sparsity=None, cdf_threshold=0.9, chunk_3d_shape_q=list(wl.chunk),
                              chunk_3d_shape_k=list(wl.chunk))
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    want, _ = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, want_idx, want_cnt)
    r, m = rel_l2(got.float().cpu(), want), max_abs(got.float().cpu(), want)
    assert r <= REL_L2_TOL and m <= MAX_ABS_TOL, (r, m)
    print(f"PARITY cdf_long: lists {int(cnt.min())}..{int(cnt.max())} entries (mean {float(cnt.float().mean()):.1f}): rel-L2 {r:.3e} max-abs {m:.3e}")


@pytest.mark.parametrize("impl", [L.ATTN_TC, L.ATTN_MMA])
def test_list_entry_outside_the_key_grid_is_flagged_not_dereferenced(impl):
    """A caller's list may hold anything.  Both kernels range-check every entry before it becomes an address: the
    generic kernel skips the block, the tcgen05 kernel reads zeros for it (its TMA box is placed outside the tensor
    map); the call is flagged through the device status word and every output value stays finite.  Rows of other
    query blocks are untouched."""
    wl = Workload("badidx", 4300, 1, 2, 128, (8, 8, 16), (8, 8, 16), (4, 4, 4), 0.5, torch.bfloat16, "normal")
    q, k, v = make_qkv(wl)
    idx, cnt, _, _ = O.block_select(q, k, wl.grid_q, wl.grid_k, wl.sparsity, wl.chunk, wl.chunk)
    nk = O.num_blocks(wl.grid_k, wl.chunk)
    ref, _ = O.attention(q, k, v, wl.grid_q, wl.grid_k, wl.chunk, wl.chunk, idx, cnt)
    bad = idx.clone()
    bad[0, 0, 3, 1] = nk + 5       # beyond the grid
    bad[0, 1, 6, 0] = -3           # negative
    L.lib().lcbsa_check_device_status()  # clear
    out = B.attn_fwd_bsa_varlen(q.cuda(), k.cuda(), v.cuda(), wl.head_dim ** -0.5, bad.cuda(), cnt.cuda(), wl.grid_q, wl.grid_k,
                                wl.chunk, wl.chunk, impl=impl)
    rc = L.lib().lcbsa_check_device_status()
    assert rc == -5, rc
    assert b"outside [0, Nk)" in L.lib().lcbsa_last_error()
    assert L.lib().lcbsa_check_device_status() == 0  # reported once, then cleared
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    tm = O.token_map(wl.grid_q, wl.chunk)
    keep = torch.ones(got.shape[1], got.shape[2], dtype=torch.bool)
    keep[0, tm[3]] = False
    keep[1, tm[6]] = False
    assert max_abs(got[0][keep], ref[0][keep]) <= MAX_ABS_TOL
