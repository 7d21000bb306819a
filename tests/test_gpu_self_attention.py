"""The self-attention layer between its projections as single calls (longcat_video_b200/modules/attention.py) against
the CPU oracle in the reference's formulation of Attention.forward and Attention.forward_with_kv_cache
(longcat_video/modules/attention.py:107-181): RMSNorm + rotary embedding bit for bit, the attention result within
rel-L2 <= 1e-2 and max-abs <= 3e-2 of the fp32 oracle."""
import pytest
import torch

from longcat_video_b200 import _lib as L
from longcat_video_b200.modules import attention as A
from oracle import bsa_oracle as O
from tests.test_gpu_norm_rope import _bits, _tables

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PARAMS = dict(sparsity=0.5, cdf_threshold=None, chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])


def _layer_inputs(seed, B, heads, D, S, cache_tokens=0):
    g = torch.Generator().manual_seed(seed)
    qkv = (torch.randn(B, S, 3, heads, D, generator=g) * 1.3).bfloat16()
    w = (1.0 + 0.2 * torch.randn(2, D, generator=g)).bfloat16()
    cache = None
    if cache_tokens:
        k_cache = torch.randn(1, heads, cache_tokens, D, generator=g).bfloat16()  # normalised keys have unit RMS
        v_cache = torch.randn(1, heads, cache_tokens, D, generator=g).bfloat16()
        cache = (k_cache, v_cache)
    return qkv, w[0].contiguous(), w[1].contiguous(), cache


def _oracle_attention(q, k, v, gq, gk):
    return O.flash_attn_bsa_3d(q, k, v, gq, gk, PARAMS["sparsity"], None, PARAMS["chunk_3d_shape_q"], PARAMS["chunk_3d_shape_k"])


def _close(got, ref):
    diff = got.float().cpu() - ref
    assert torch.isfinite(got.float()).all()
    assert float(diff.norm() / ref.norm()) <= 1e-2 and float(diff.abs().max()) <= 3e-2


@pytest.mark.parametrize("nc", [None, 4])
def test_forward_between_the_projections(nc):
    """Attention.forward, attention.py:116-137, with and without cond frames, and what return_kv hands back."""
    shape, heads, D = (12, 8, 8), 2, 128
    T, H, W = shape
    S = T * H * W
    qkv, wq, wk, _ = _layer_inputs(71, 1, heads, D, S)
    q, k, v = qkv.to(DEV).permute(2, 0, 3, 1, 4).unbind(0)  # attention.py:113-115: strided views
    x, (k_cache, v_cache) = A.self_attention(q, k, v, wq, wk, shape, PARAMS, num_cond_latents=nc, return_kv=True)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    qc, kc, vc = (t.cpu().contiguous() for t in (q, k, v))
    assert torch.equal(_bits(k_cache.cpu()), _bits(O.norm_rope(kc, wk, None, None)))  # attention.py:118-119
    assert torch.equal(v_cache.cpu(), vc)
    cos, sin = _tables(shape, D)
    q_e, k_e = O.norm_rope(qc, wq, cos, sin), O.norm_rope(kc, wk, cos, sin)
    if nc:
        sc = nc * H * W
        ref = torch.cat([_oracle_attention(q_e[:, :, :sc].contiguous(), k_e[:, :, :sc].contiguous(), vc[:, :, :sc].contiguous(),
                                           (nc, H, W), (nc, H, W)),
                         _oracle_attention(q_e[:, :, sc:].contiguous(), k_e, vc, (T - nc, H, W), shape)], dim=2)
    else:
        ref = _oracle_attention(q_e, k_e, vc, shape, shape)
    assert x.shape == (1, heads, S, D)
    _close(x, ref)
    assert torch.equal(x, A.self_attention(q, k, v, wq, wk, shape, PARAMS, num_cond_latents=nc))


@pytest.mark.parametrize("B", [1, 2])
def test_forward_with_kv_cache(B):
    """Attention.forward_with_kv_cache, attention.py:156-173: T new frames against NC cached ones and themselves; a
    cache of batch 1 serves both batch entries."""
    shape, nc, heads, D = (8, 8, 8), 4, 2, 128
    T, H, W = shape
    S, sc = T * H * W, nc * H * W
    qkv, wq, wk, (k_cache, v_cache) = _layer_inputs(72, B, heads, D, S, cache_tokens=sc)
    q, k, v = qkv.to(DEV).permute(2, 0, 3, 1, 4).unbind(0)
    x = A.self_attention_with_kv_cache(q, k, v, wq, wk, shape, (k_cache.to(DEV), v_cache.to(DEV)), PARAMS, nc)
    torch.cuda.synchronize()
    L.check(L.lib().lcbsa_check_device_status())
    qc, kc, vc = (t.cpu().contiguous() for t in (q, k, v))
    cos, sin = _tables((T + nc, H, W), D)
    kcb, vcb = k_cache.expand(B, -1, -1, -1).contiguous(), v_cache.expand(B, -1, -1, -1).contiguous()  # attention.py:160-162
    k_full = torch.cat([O.norm_rope(kcb, None, cos[:sc], sin[:sc]), O.norm_rope(kc, wk, cos[sc:], sin[sc:])], dim=2).contiguous()
    v_full = torch.cat([vcb, vc], dim=2).contiguous()
    q_e = O.norm_rope(qc, wq, cos[sc:], sin[sc:])
    ref = _oracle_attention(q_e, k_full, v_full, shape, (T + nc, H, W))
    assert x.shape == (B, heads, S, D)
    _close(x, ref)


def test_kv_cache_arguments_are_checked():
    shape, heads, D = (4, 8, 8), 1, 128
    qkv, wq, wk, (k_cache, v_cache) = _layer_inputs(73, 1, heads, D, 256, cache_tokens=256)
    q, k, v = qkv.to(DEV).permute(2, 0, 3, 1, 4).unbind(0)
    cache = (k_cache.to(DEV), v_cache.to(DEV))
    with pytest.raises(ValueError):
        A.self_attention_with_kv_cache(q, k, v, wq, wk, shape, cache, PARAMS, 0)  # the reference has no k_full then
    with pytest.raises(ValueError):
        A.self_attention_with_kv_cache(q, k, v, wq, wk, shape, cache, PARAMS, 8)  # 512 cached tokens expected, 256 given
    with pytest.raises(ValueError):
        A.self_attention_with_kv_cache(q, k, v, wq, wk, shape, (cache[0].expand(3, -1, -1, -1), cache[1]), PARAMS, 4)
