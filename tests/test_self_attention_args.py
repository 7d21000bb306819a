"""Argument checks of the layer-body entry points (longcat_video_b200/modules/attention.py) that happen on the host, before
any CUDA call: they run without a GPU."""
import pytest
import torch

from longcat_video_b200.modules import attention as A

PARAMS = dict(sparsity=0.5, cdf_threshold=None, chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])


def _qkv(B=1, H=1, S=256, D=128):
    return tuple(torch.zeros(B, H, S, D) for _ in range(3))


def test_kv_cache_needs_cond_frames():
    """The reference builds k_full and v_full only when num_cond_latents > 0 (longcat_video/modules/attention.py:164-171)."""
    q, k, v = _qkv()
    for nc in (None, 0, -1):
        with pytest.raises(ValueError):
            A.self_attention_with_kv_cache(q, k, v, None, None, (4, 8, 8), (k, v), PARAMS, nc)


def test_kv_cache_sizes_and_batches_are_checked():
    q, k, v = _qkv(B=2)
    cache_ok = (torch.zeros(1, 1, 256, 128), torch.zeros(1, 1, 256, 128))
    with pytest.raises(ValueError):  # 8 cached frames would be 512 tokens
        A.self_attention_with_kv_cache(q, k, v, None, None, (4, 8, 8), cache_ok, PARAMS, 8)
    with pytest.raises(ValueError):  # cache batch must be 1 or B, and equal for k and v (attention.py:158-162)
        A.self_attention_with_kv_cache(q, k, v, None, None, (4, 8, 8), (torch.zeros(3, 1, 256, 128), cache_ok[1]), PARAMS, 4)
    with pytest.raises(ValueError):  # the new tokens do not fill the grid
        A.self_attention_with_kv_cache(q, k, v, None, None, (5, 8, 8), cache_ok, PARAMS, 4)


def test_no_cpu_path():
    """The ops refuse CPU tensors instead of falling back."""
    q, k, v = _qkv()
    w = torch.ones(128)
    with pytest.raises(Exception):
        A.self_attention(q, k, v, w, w, (4, 8, 8), PARAMS)
