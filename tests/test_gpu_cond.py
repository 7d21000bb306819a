"""The cond / noise split of Attention.forward (longcat_video/modules/attention.py:124-137) as one op on views,
against the reference's formulation: contiguous copies, two calls, torch.cat."""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.block_sparse_attention import flash_attn_bsa_3d, flash_attn_bsa_3d_cond
from oracle import bsa_oracle as O

pytestmark = pytest.mark.gpu


def _reference_form(q, k, v, shape, nc, fn, **params):
    T, H, W = shape
    sc = nc * H * W
    q_cond, k_cond, v_cond = (x[:, :, :sc].contiguous() for x in (q, k, v))
    x_cond = fn(q_cond, k_cond, v_cond, (nc, H, W), (nc, H, W), **params)
    x_noise = fn(q[:, :, sc:].contiguous(), k.contiguous(), v.contiguous(), (T - nc, H, W), (T, H, W), **params)
    return torch.cat([x_cond, x_noise], dim=2).contiguous()


@pytest.mark.parametrize("params", [dict(sparsity=0.5), dict(sparsity=None, cdf_threshold=0.7)])
@pytest.mark.parametrize("strided", [False, True])
@pytest.mark.parametrize("shape,nc", [((12, 8, 8), 4), ((16, 8, 12), 12), ((10, 8, 8), 3)])  # whole blocks: one selection, one attention launch; ragged: two launches on views
def test_cond_split_equals_two_calls(params, strided, shape, nc):
    heads, D = 3, 128
    ragged = nc % 4 != 0
    if ragged and params.get("cdf_threshold") is not None:
        pytest.skip("one selector is enough for the ragged split")
    S = shape[0] * shape[1] * shape[2]
    params = dict(params, chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])
    if ragged:
        params["allow_ragged"] = True
    g = torch.Generator().manual_seed(31)
    qkv = torch.randn(1, S, 3, heads, D, generator=g).bfloat16()
    q, k, v = qkv.cuda().permute(2, 0, 3, 1, 4).unbind(0)  # the strided views of the fused projection
    if not strided:
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    got = flash_attn_bsa_3d_cond(q, k, v, shape, nc, **params)
    want = _reference_form(q, k, v, shape, nc, flash_attn_bsa_3d, **params)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    assert got.shape == (1, heads, S, D) and torch.equal(got, want)
    if ragged:
        return  # partial blocks are an extension without a reference formulation
    # and against the fp32 oracle in the same formulation
    qc, kc, vc = (x.cpu().contiguous() for x in (q, k, v))
    ofn = lambda a, b, c, gq, gk, **p: O.flash_attn_bsa_3d(a, b, c, gq, gk, p.get("sparsity"), p.get("cdf_threshold"),  # noqa: E731
                                                           p["chunk_3d_shape_q"], p["chunk_3d_shape_k"])
    ref = _reference_form(qc, kc, vc, shape, nc, ofn, **params)
    diff = got.float().cpu() - ref
    assert float(diff.norm() / ref.norm()) <= 1e-2 and float(diff.abs().max()) <= 3e-2


def test_no_cond_latents_is_the_plain_call():
    shape, heads, D = (4, 8, 8), 2, 128
    g = torch.Generator().manual_seed(32)
    q, k, v = (torch.randn(1, heads, 256, D, generator=g).bfloat16().cuda() for _ in range(3))
    params = dict(sparsity=0.5, chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])
    assert torch.equal(flash_attn_bsa_3d_cond(q, k, v, shape, None, **params), flash_attn_bsa_3d(q, k, v, shape, shape, **params))
    with pytest.raises(ValueError):
        flash_attn_bsa_3d_cond(q, k, v, shape, 4, **params)
