"""ctypes binding of ``liblcbsa.so`` (declared in ``include/lcbsa.h``).

There is no fallback: if the library is missing or a CUDA device is absent the calls raise.
"""
from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# LCBSA_LIBRARY points at another build of the same ABI (e.g. one compiled with extra checks)
LIB_PATH = os.environ.get("LCBSA_LIBRARY") or os.path.join(_HERE, "csrc", "liblcbsa.so")

LCBSA_BF16, LCBSA_FP16, LCBSA_FP32 = 0, 1, 2
ATTN_AUTO, ATTN_TC, ATTN_MMA = 0, 1, 2

_DTYPES = {torch.bfloat16: LCBSA_BF16, torch.float16: LCBSA_FP16, torch.float32: LCBSA_FP32}


class LcbsaError(RuntimeError):
    """A call into liblcbsa.so failed; ``code`` is the negative LCBSA_E* value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"lcbsa error {code}: {message}")
        self.code = code


class LcbsaTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int32), ("reserved", ctypes.c_int32),
                ("size", ctypes.c_int64 * 4), ("stride", ctypes.c_int64 * 4)]


class LcbsaGrid(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("T", "H", "W", "ct", "ch", "cw")]


class LcbsaSplit(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("hw_q", "period_q", "split_q", "hw_k", "period_k", "split_k", "nsel_first")]


# every symbol include/lcbsa.h declares, with its C signature
_P = ctypes.POINTER
SIGNATURES = {
    "lcbsa_version": (ctypes.c_int, []),
    "lcbsa_last_error": (ctypes.c_char_p, []),
    "lcbsa_num_blocks": (ctypes.c_int, [_P(LcbsaGrid)]),
    "lcbsa_num_selected": (ctypes.c_int, [ctypes.c_double, ctypes.c_int]),
    "lcbsa_pool": (ctypes.c_int, [_P(LcbsaTensor), _P(LcbsaGrid), ctypes.c_void_p, ctypes.c_void_p]),
    "lcbsa_pool_scatter": (ctypes.c_int, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid), ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "lcbsa_score_topk": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p]),
    "lcbsa_select_workspace_bytes": (ctypes.c_size_t, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid)]),
    "lcbsa_score_keys_bytes": (ctypes.c_size_t, [ctypes.c_int] * 5),
    "lcbsa_score_topk_ws": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 7
                            + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "lcbsa_score_topk_split": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 5 + [_P(LcbsaSplit), ctypes.c_int, ctypes.c_int,
                                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "lcbsa_block_select_split": (ctypes.c_int, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid)] + [ctypes.c_int] * 7
                                 + [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "lcbsa_select_workspace_bytes_fast": (ctypes.c_size_t, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid)]),
    "lcbsa_block_select": (ctypes.c_int, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid), ctypes.c_int,
                                          ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_size_t, ctypes.c_void_p]),
    "lcbsa_attn_fwd": (ctypes.c_int, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid),
                                      ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, _P(LcbsaTensor),
                                      ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]),
    "lcbsa_attn_fwd_scatter": (ctypes.c_int, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid),
                                              ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_int,
                                              ctypes.c_int64, ctypes.c_int64, ctypes.c_void_p]),
    "lcbsa_attn_bwd_workspace_bytes": (ctypes.c_size_t, [_P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid), ctypes.c_int]),
    "lcbsa_attn_bwd": (ctypes.c_int, [_P(LcbsaTensor)] * 5 + [_P(LcbsaGrid), _P(LcbsaGrid), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                      ctypes.c_float, ctypes.c_void_p, _P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaTensor), ctypes.c_void_p,
                                      ctypes.c_size_t, ctypes.c_void_p]),
    "lcbsa_static_scratch_bytes": (ctypes.c_size_t, []),
    "lcbsa_block_select_static": (ctypes.c_int, [_P(LcbsaTensor), _P(LcbsaTensor), _P(LcbsaGrid), _P(LcbsaGrid), ctypes.c_int,
                                                 ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]),
    "lcbsa_set_attn_sm_reserve": (ctypes.c_int, [ctypes.c_int]),
    "lcbsa_norm_rope_ex": (ctypes.c_int, [_P(LcbsaTensor), ctypes.c_void_p, _P(LcbsaGrid), ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_float, _P(LcbsaTensor), ctypes.c_void_p]),
    "lcbsa_score_cdf": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_float, ctypes.c_int,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "lcbsa_rope_table_floats": (ctypes.c_size_t, [_P(LcbsaGrid), ctypes.c_int]),
    "lcbsa_norm_rope": (ctypes.c_int, [_P(LcbsaTensor), ctypes.c_void_p, _P(LcbsaGrid), ctypes.c_void_p, ctypes.c_float,
                                       _P(LcbsaTensor), ctypes.c_void_p]),
    "lcbsa_copy_slabs": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]),
    "lcbsa_check_device_status": (ctypes.c_int, []),
}

_lib = None


def lib() -> ctypes.CDLL:
    """Load liblcbsa.so once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m longcat_video_b200.build`")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise LcbsaError(code, lib().lcbsa_last_error().decode())


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}") from None


def tensor_desc(t: torch.Tensor) -> LcbsaTensor:
    """Describe a CUDA ``[B,H,S,D]`` tensor (any strides) for the C ABI."""
    if t.dim() != 4:
        raise ValueError("expected a [B, H, S, D] tensor")
    if not t.is_cuda:
        raise RuntimeError("lcbsa runs on CUDA tensors only (there is no CPU path)")
    d = LcbsaTensor()
    d.data = t.data_ptr()
    d.dtype = dtype_code(t.dtype)
    for i in range(4):
        d.size[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    return d


def grid_desc(latent_shape: Sequence[int], chunk: Sequence[int]) -> LcbsaGrid:
    return LcbsaGrid(int(latent_shape[0]), int(latent_shape[1]), int(latent_shape[2]),
                     int(chunk[0]), int(chunk[1]), int(chunk[2]))


def current_stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def abi_ok(t: torch.Tensor) -> bool:
    """True when a tensor can be handed over as it is (head_dim contiguous, 16-byte rules)."""
    es = t.element_size()
    return (t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all((t.stride(i) * es) % 16 == 0 and t.stride(i) >= 0
                                                                  for i in range(3)))
