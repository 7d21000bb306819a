"""The CPU oracle of the pre-attention producer (q/k RMSNorm + 3-D rotary embedding) against fixtures produced by the
reference's own modules (tests/golden/make_golden_norm_rope.py: RMSNorm_FP32 of longcat_video/modules/blocks.py:42-53
and RotaryPositionalEmbedding of longcat_video/modules/rope_3d.py, chained as in attention.py:113-121)."""
import os

import numpy as np
import pytest
import torch

from oracle import bsa_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
NAMES = ["norm_rope_d128", "norm_rope_d64_b2"]


def load(name):
    z = np.load(os.path.join(HERE, "golden", name + ".npz"))
    seed, B, H, D = (int(v) for v in z["meta"])
    grid = tuple(int(v) for v in z["grid"])
    bf = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)  # noqa: E731
    qkv = bf(z["qkv"])
    q_in, k_in, _ = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    return dict(q_in=q_in, k_in=k_in, wq=bf(z["wq"]), wk=bf(z["wk"]), q=bf(z["q"]), k=bf(z["k"]), grid=grid, D=D)


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference_modules(name):
    c = load(name)
    cos, sin = O.rope_tables(c["grid"], c["D"])
    for x, w, want in ((c["q_in"], c["wq"], c["q"]), (c["k_in"], c["wk"], c["k"])):
        got = O.norm_rope(x, w, cos, sin, eps=1e-6)
        assert got.shape == want.shape
        # The reference's mean over the head dimension is a library reduction whose order is not specified; the oracle
        # fixes an order.  The normalised value can therefore land on the neighbouring bf16 in rare rows; everything
        # else is elementwise arithmetic that is restated exactly.
        same = (got.view(torch.int16) == want.view(torch.int16)).float().mean().item()
        assert same > 0.999, same
        diff = (got.float() - want.float()).abs()
        assert float((diff / (want.float().abs() + 1e-3)).max()) < 2 ** -6


def test_rope_tables_shape_and_first_position():
    cos, sin = O.rope_tables((2, 3, 4), 128)
    assert cos.shape == (24, 128) and sin.shape == (24, 128)
    assert torch.all(cos[0] == 1) and torch.all(sin[0] == 0)  # position (0, 0, 0): no rotation
    # W is the fastest axis and only turns the last 2*(D//6) elements
    assert torch.equal(cos[1, :86], cos[0, :86]) and not torch.equal(cos[1, 86:], cos[0, 86:])
