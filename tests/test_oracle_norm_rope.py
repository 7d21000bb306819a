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
    return dict(q_in=q_in, k_in=k_in, wq=bf(z["wq"]), wk=bf(z["wk"]), q=bf(z["q"]), k=bf(z["k"]), grid=grid, D=D,
                q_normed=bf(z["q_normed"]), k_normed=bf(z["k_normed"]), k_cache=bf(z["k_cache"]), q_kv=bf(z["q_kv"]),
                k_full=bf(z["k_full"]), nc=2)


def close_to_reference(got, want):
    """The reference's mean over the head dimension is a library reduction whose order is not specified; the oracle fixes
    an order, so the normalised value can land on the neighbouring value of the dtype in rare rows.  Everything else is
    elementwise arithmetic restated exactly."""
    assert got.shape == want.shape
    same = (got.contiguous().view(torch.int16) == want.contiguous().view(torch.int16)).float().mean().item()
    assert same > 0.999, same
    diff = (got.float() - want.float()).abs()
    assert float((diff / (want.float().abs() + 1e-3)).max()) < 2 ** -6


@pytest.mark.parametrize("name", NAMES)
def test_oracle_matches_reference_modules(name):
    c = load(name)
    cos, sin = O.rope_tables(c["grid"], c["D"])
    for x, w, want in ((c["q_in"], c["wq"], c["q"]), (c["k_in"], c["wk"], c["k"])):
        close_to_reference(O.norm_rope(x, w, cos, sin, eps=1e-6), want)


def test_rope_tables_shape_and_first_position():
    cos, sin = O.rope_tables((2, 3, 4), 128)
    assert cos.shape == (24, 128) and sin.shape == (24, 128)
    assert torch.all(cos[0] == 1) and torch.all(sin[0] == 0)  # position (0, 0, 0): no rotation
    # W is the fastest axis and only turns the last 2*(D//6) elements
    assert torch.equal(cos[1, :86], cos[0, :86]) and not torch.equal(cos[1, 86:], cos[0, 86:])


@pytest.mark.parametrize("name", NAMES)
def test_oracle_halves_and_kv_cache_flow(name):
    """Normalisation alone (what return_kv caches, attention.py:118-119) and the KV-cache flow of
    forward_with_kv_cache (attention.py:156-171): cached keys embedded at frames 0..NC-1, new q and k at NC.."""
    c = load(name)
    T, H, W = c["grid"]
    nc, sc = c["nc"], c["nc"] * H * W
    close_to_reference(O.norm_rope(c["q_in"], c["wq"], None, None), c["q_normed"])
    close_to_reference(O.norm_rope(c["k_in"], c["wk"], None, None), c["k_normed"])
    cos, sin = O.rope_tables((T + nc, H, W), c["D"])
    head = O.norm_rope(c["k_cache"], None, cos[:sc], sin[:sc])
    assert torch.equal(head.view(torch.int16), c["k_full"][:, :, :sc].contiguous().view(torch.int16))  # no reduction: exact
    close_to_reference(O.norm_rope(c["k_in"], c["wk"], cos[sc:], sin[sc:]), c["k_full"][:, :, sc:])
    close_to_reference(O.norm_rope(c["q_in"], c["wq"], cos[sc:], sin[sc:]), c["q_kv"])


def test_rope_table_of_a_context_parallel_shard():
    """A rank that holds rows h0.. and columns w0.. of the frame takes the angles of its own positions
    (longcat_video/modules/rope_3d.py:91-95): the table built with pos_offset equals the slice of the full one."""
    from longcat_video_b200.modules import rope_3d as R
    T, H, W, D = 3, 8, 12, 128
    dh = 2 * (D // 6)
    dt = D - 2 * dh
    full = R.rope_table((T, H, W), D, "cpu")
    part = R.rope_table((T, H // 2, W // 3), D, "cpu", pos_offset=(0, H // 2, 2 * (W // 3)))
    f = torch.split(full, [T * dt, T * dt, H * dh, H * dh, W * dh, W * dh])
    p = torch.split(part, [T * dt, T * dt, (H // 2) * dh, (H // 2) * dh, (W // 3) * dh, (W // 3) * dh])
    assert torch.equal(p[0], f[0]) and torch.equal(p[1], f[1])
    assert float((p[2].view(-1, dh) - f[2].view(H, dh)[H // 2:]).abs().max()) <= 2 ** -22
    assert float((p[5].view(-1, dh) - f[5].view(W, dh)[2 * (W // 3):]).abs().max()) <= 2 ** -22
