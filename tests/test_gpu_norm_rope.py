"""The fused q/k RMSNorm + 3-D rotary kernel (lcbsa_norm_rope) against the CPU oracle, bit for bit, on the strided q/k
views of a fused qkv projection as Attention.forward has them (longcat_video/modules/attention.py:107-121), and
against the fixtures produced by the reference's own modules (tests/golden/make_golden_norm_rope.py)."""
import ctypes

import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.modules import rope_3d as R
from oracle import bsa_oracle as O
from tests.test_oracle_norm_rope import NAMES, close_to_reference, load

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _qkv(seed, B, S, H, D, dtype):
    g = torch.Generator().manual_seed(seed)
    qkv = (torch.randn(B, S, 3, H, D, generator=g) * 1.7).to(dtype)
    w = (1.0 + 0.2 * torch.randn(2, D, generator=g)).to(dtype)
    return qkv, w[0].contiguous(), w[1].contiguous()


def _bits(t):
    return t.contiguous().view(torch.int16)


def _tables(grid, D):
    """The [S, D] cos / sin tables the oracle takes, expanded from the very table the kernel reads: the angles are an
    input of both sides (two evaluations of cosf on differently shaped arrays need not agree in the last bit)."""
    T, H, W = grid
    dh = 2 * (D // 6)
    dt = D - 2 * dh
    tab = R.rope_table(grid, D, DEV).cpu()
    sizes = [T * dt, T * dt, H * dh, H * dh, W * dh, W * dh]
    ct, st, ch, sh, cw, sw = torch.split(tab, sizes)
    full = lambda a, b, c: torch.cat([a.view(T, 1, 1, dt).expand(T, H, W, dt), b.view(1, H, 1, dh).expand(T, H, W, dh),  # noqa: E731
                                      c.view(1, 1, W, dh).expand(T, H, W, dh)], dim=-1).reshape(T * H * W, D).contiguous()
    cos, sin = full(ct, ch, cw), full(st, sh, sw)
    ref_cos, ref_sin = O.rope_tables(grid, D)
    assert float((cos - ref_cos).abs().max()) <= 2 ** -22 and float((sin - ref_sin).abs().max()) <= 2 ** -22
    return cos, sin


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,D,grid", [(1, 3, 128, (3, 8, 10)), (2, 2, 64, (2, 6, 8)), (1, 5, 128, (5, 7, 9))])
def test_kernel_equals_oracle_bit_for_bit(dtype, B, H, D, grid):
    S = grid[0] * grid[1] * grid[2]
    qkv, wq, wk = _qkv(11 + D + S, B, S, H, D, dtype)
    cos, sin = _tables(grid, D)
    q_in, k_in, _ = qkv.permute(2, 0, 3, 1, 4).unbind(0)  # [B, H, S, D] views with strides of the fused projection
    want_q, want_k = O.norm_rope(q_in, wq, cos, sin, 1e-6), O.norm_rope(k_in, wk, cos, sin, 1e-6)
    dq, dk, _ = qkv.to(DEV).permute(2, 0, 3, 1, 4).unbind(0)
    assert not dq.is_contiguous()
    got_q, got_k = R.qk_norm_rope(dq, dk, wq, wk, grid)
    torch.cuda.synchronize()
    assert torch.equal(_bits(got_q.cpu()), _bits(want_q))
    assert torch.equal(_bits(got_k.cpu()), _bits(want_k))


def test_strided_output_and_in_place():
    """The output may be any [B, H, S, D] view, e.g. a [B, S, H, D] buffer seen through a permute, or the input itself."""
    B, H, D, grid = 1, 4, 128, (2, 4, 6)
    S = 48
    qkv, wq, _ = _qkv(5, B, S, H, D, torch.bfloat16)
    cos, sin = _tables(grid, D)
    q_in = qkv.permute(2, 0, 3, 1, 4)[0]
    want = O.norm_rope(q_in, wq, cos, sin, 1e-6)
    dq = qkv.to(DEV).permute(2, 0, 3, 1, 4)[0]
    buf = torch.zeros(B, S, H, D, dtype=torch.bfloat16, device=DEV)
    out = R.norm_rope(dq, wq, grid, out=buf.permute(0, 2, 1, 3))
    assert out.data_ptr() == buf.data_ptr()
    assert torch.equal(_bits(buf.permute(0, 2, 1, 3).cpu()), _bits(want))
    R.norm_rope(dq, wq, grid, out=dq)  # every row is read in full by its warp before it is written
    torch.cuda.synchronize()
    assert torch.equal(_bits(dq.cpu()), _bits(want))


@pytest.mark.parametrize("name", NAMES)
def test_kernel_against_reference_fixtures(name):
    c = load(name)
    for x, w, want in ((c["q_in"], c["wq"], c["q"]), (c["k_in"], c["wk"], c["k"])):
        got = R.norm_rope(x.to(DEV), w, c["grid"]).cpu()
        # same bound as the oracle's pin: the reference's reduction order is unspecified, so rare neighbouring-bf16 results
        same = (_bits(got) == _bits(want)).float().mean().item()
        assert same > 0.999, same
        diff = (got.float() - want.float()).abs()
        assert float((diff / (want.float().abs() + 1e-3)).max()) < 2 ** -6


@pytest.mark.parametrize("name", NAMES)
def test_halves_and_kv_cache_flow(name):
    """Normalisation alone, embedding alone, and the frame offset, as the KV-cache path of the attention layer uses them
    (longcat_video/modules/attention.py:118-119, 156-171): bit for bit against the oracle, and against the reference's
    fixtures within the bound of the oracle's own pin."""
    c = load(name)
    T, H, W = c["grid"]
    nc, sc = c["nc"], c["nc"] * H * W
    got = R.rms_norm(c["q_in"].to(DEV), c["wq"]).cpu()
    assert torch.equal(_bits(got), _bits(O.norm_rope(c["q_in"], c["wq"], None, None)))
    close_to_reference(got, c["q_normed"])
    q_out, k_full = R.qk_norm_rope_with_kv_cache(c["q_in"].to(DEV), c["k_in"].to(DEV), c["wq"], c["wk"], c["k_cache"].to(DEV),
                                                 c["grid"], nc)
    torch.cuda.synchronize()
    q_out, k_full = q_out.cpu(), k_full.cpu()
    cos, sin = _tables((T + nc, H, W), c["D"])
    assert torch.equal(_bits(k_full[:, :, :sc]), _bits(O.norm_rope(c["k_cache"], None, cos[:sc], sin[:sc])))
    assert torch.equal(_bits(k_full[:, :, sc:]), _bits(O.norm_rope(c["k_in"], c["wk"], cos[sc:], sin[sc:])))
    assert torch.equal(_bits(q_out), _bits(O.norm_rope(c["q_in"], c["wq"], cos[sc:], sin[sc:])))
    close_to_reference(k_full, c["k_full"])
    close_to_reference(q_out, c["q_kv"])


def test_full_size_rows_keep_their_norm():
    """720p-sized property check: a rotation keeps the length of every pair, so with weight 1 every output row has
    mean square 1 (up to the two bf16 roundings), whatever its position."""
    grid, H, D = (24, 48, 80), 4, 128
    S = grid[0] * grid[1] * grid[2]
    g = torch.Generator(device=DEV).manual_seed(3)
    x = (torch.randn(1, H, S, D, generator=g, device=DEV) * 3).to(torch.bfloat16)
    y = R.norm_rope(x, torch.ones(D), grid)
    ms = y.float().pow(2).mean(-1)
    assert float((ms - 1).abs().max()) < 2e-2
    # position (0, 0, 0) is not rotated: it is the plain normalised row
    x0 = x[0, :, 0].float()
    n0 = (x0 * torch.rsqrt(x0.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)
    assert float((y[0, :, 0].float() - n0.float()).abs().max()) <= 2 ** -5


def test_bad_arguments_are_refused():
    grid = (2, 4, 4)
    x = torch.zeros(1, 2, 32, 128, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(L.LcbsaError, match="does not match the latent grid"):
        R.norm_rope(x, torch.ones(128), (2, 4, 5))
    with pytest.raises(L.LcbsaError, match="head_dim 64 or 128"):
        R.norm_rope(torch.zeros(1, 2, 32, 96, dtype=torch.bfloat16, device=DEV), torch.ones(96), grid)
    with pytest.raises(L.LcbsaError, match="dtypes differ"):
        R.norm_rope(x, torch.ones(128), grid, out=torch.zeros(1, 2, 32, 128, dtype=torch.float16, device=DEV))
    xd, g = L.tensor_desc(x), L.grid_desc(grid, (1, 1, 1))
    rc = L.lib().lcbsa_norm_rope(ctypes.byref(xd), None, ctypes.byref(g), None, ctypes.c_float(1e-6), ctypes.byref(xd), None)
    assert rc == -1
    with pytest.raises(L.LcbsaError, match="outside the table"):  # frames 3..4 of a table that holds 4
        R.norm_rope(x, torch.ones(128), grid, t_offset=3, table_frames=4)
    with pytest.raises(ValueError):
        R.norm_rope(x, None, grid, rope=False)
