"""The reference's own Triton block-sparse attention, loaded from ``baseline/_ref/`` (see ``install_reference.py``).

Comparator only: the benchmark times it next to this library's kernels on the same GPU and the same inputs, and a test
reports how far the two outputs are apart.  Nothing under ``longcat_video_b200/`` imports this module.
"""
from __future__ import annotations

import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")

_mod = None
_why = None


def load():
    """The reference's ``bsa_interface`` module, or None (``why()`` then says what went wrong)."""
    global _mod, _why
    if _mod is not None or _why is not None:
        return _mod
    if not os.path.isdir(os.path.join(REF_ROOT, "longcat_video", "block_sparse_attention")):
        _why = "baseline/_ref is absent (run baseline/install_reference.py where the reference checkout is)"
        return None
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    try:
        _mod = importlib.import_module("longcat_video.block_sparse_attention.bsa_interface")
    except Exception as e:  # noqa: BLE001 - Triton or torch version mismatches surface here
        _why = f"import failed: {e!r}"[:300]
    return _mod


def why() -> str:
    return _why or ""


def versions() -> dict:
    import torch
    out = {"torch": torch.__version__}
    try:
        import triton
        out["triton"] = triton.__version__
    except Exception:  # noqa: BLE001
        out["triton"] = None
    return out


def flash_attn_bsa_3d(q, k, v, latent_shape_q, latent_shape_k, **bsa_params):
    """The reference's entry point (bsa_interface.py:612-660), called exactly as the DiT calls it."""
    m = load()
    if m is None:
        raise RuntimeError(why())
    return m.flash_attn_bsa_3d(q, k, v, latent_shape_q, latent_shape_k, **bsa_params)
