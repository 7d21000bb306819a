"""CPU-only checks of the C ABI: the library loads without a GPU, exports every function that
include/lcbsa.h declares, and its host-side helpers and argument validation behave."""
import ctypes
import os
import re

import pytest
import torch

from longcat_video_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "lcbsa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lcbsa_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = _declared()
    assert len(names) >= 12
    lib = L.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/lcbsa.h but not exported by liblcbsa.so"
        assert n in L.SIGNATURES, f"{n} has no ctypes signature in _lib.py"


def test_host_helpers():
    lib = L.lib()
    assert lib.lcbsa_version() == 100
    g = L.grid_desc((24, 45, 80), (4, 4, 4))
    assert lib.lcbsa_num_blocks(ctypes.byref(g)) == 6 * 12 * 20
    g = L.grid_desc((24, 48, 80), (4, 4, 8))
    assert lib.lcbsa_num_blocks(ctypes.byref(g)) == 6 * 12 * 10
    for sp, nk in ((0.9375, 1440), (0.9, 10), (0.875, 1320), (0.5, 4), (0.96875, 1440), (0.0, 7), (1.0, 7)):
        assert lib.lcbsa_num_selected(sp, nk) == int((1 - sp) * nk)
    assert lib.lcbsa_static_scratch_bytes() == 32 << 20


def test_validation_happens_before_any_launch():
    """Bad descriptions are refused on the host (no GPU is needed to get the error)."""
    lib = L.lib()
    t = L.LcbsaTensor()
    t.data, t.dtype = 4096, L.LCBSA_BF16
    for i, (n, s) in enumerate(zip((1, 2, 64, 128), (2 * 64 * 128, 64 * 128, 128, 1))):
        t.size[i], t.stride[i] = n, s
    good = L.grid_desc((4, 4, 4), (4, 4, 4))
    bad = L.grid_desc((4, 4, 5), (4, 4, 4))
    assert lib.lcbsa_pool(ctypes.byref(t), ctypes.byref(bad), 4096, None) == -1
    assert b"does not match the latent grid" in lib.lcbsa_last_error()
    t.data = 4100
    assert lib.lcbsa_pool(ctypes.byref(t), ctypes.byref(good), 4096, None) == -1
    assert b"16-byte aligned" in lib.lcbsa_last_error()
    t.data = 4096
    assert lib.lcbsa_block_select(ctypes.byref(t), ctypes.byref(t), ctypes.byref(good), ctypes.byref(good), 1, 1, 4096, 4096,
                                  None, 0, None) == -3
    assert lib.lcbsa_score_topk(4096, 4096, L.LCBSA_BF16, 1, 4, 4, 128, 5, 5, 4096, 4096, None) == -1


def test_norm_rope_host_side():
    """Table size and argument checks of the q/k RMSNorm + rotary entry point run on the host."""
    lib = L.lib()
    g = L.grid_desc((24, 48, 80), (1, 1, 1))
    assert lib.lcbsa_rope_table_floats(ctypes.byref(g), 128) == 2 * (24 * 44 + 48 * 42 + 80 * 42)
    assert lib.lcbsa_rope_table_floats(ctypes.byref(g), 64) == 2 * (24 * 24 + 48 * 20 + 80 * 20)
    assert lib.lcbsa_rope_table_floats(ctypes.byref(g), 127) == 0
    t = L.LcbsaTensor()
    t.data, t.dtype = 4096, L.LCBSA_BF16
    for i, (n, s) in enumerate(zip((1, 2, 64, 128), (2 * 64 * 128, 64 * 128, 128, 1))):
        t.size[i], t.stride[i] = n, s
    g = L.grid_desc((4, 4, 4), (1, 1, 1))
    assert lib.lcbsa_norm_rope(ctypes.byref(t), None, ctypes.byref(g), 4096, 1e-6, ctypes.byref(t), None) == -1
    assert b"null weight" in lib.lcbsa_last_error()
    bad = L.grid_desc((4, 4, 5), (1, 1, 1))
    assert lib.lcbsa_norm_rope(ctypes.byref(t), 4096, ctypes.byref(bad), 4096, 1e-6, ctypes.byref(t), None) == -1
    assert b"does not match the latent grid" in lib.lcbsa_last_error()
    assert lib.lcbsa_norm_rope_ex(ctypes.byref(t), None, ctypes.byref(g), None, 4, 0, 1e-6, ctypes.byref(t), None) == -1
    assert b"nothing to do" in lib.lcbsa_last_error()
    assert lib.lcbsa_norm_rope_ex(ctypes.byref(t), 4096, ctypes.byref(g), 4096, 4, 1, 1e-6, ctypes.byref(t), None) == -1
    assert b"outside the table" in lib.lcbsa_last_error()
    from longcat_video_b200.modules import norm_rope
    with pytest.raises(RuntimeError):
        norm_rope(torch.zeros(1, 1, 64, 128, dtype=torch.bfloat16), torch.ones(128), (4, 4, 4))


def test_python_wrapper_refuses_cpu_tensors():
    from longcat_video_b200.block_sparse_attention import flash_attn_bsa_3d
    q = torch.zeros(1, 1, 64, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        flash_attn_bsa_3d(q, q, q, (4, 4, 4), (4, 4, 4), sparsity=0.5, chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])
    with pytest.raises(AssertionError):
        flash_attn_bsa_3d(q, q, q, (4, 4, 5), (4, 4, 4), sparsity=0.5, chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])
    with pytest.raises(ValueError):
        flash_attn_bsa_3d(q, q, q, (4, 4, 4), (4, 4, 4), sparsity=None, cdf_threshold=None, chunk_3d_shape_q=[4, 4, 4],
                          chunk_3d_shape_k=[4, 4, 4])
