"""World-size-2 and -4 checks of the Ulysses hooks on CPU (gloo): index math, inverse property,
head-group pipelining, error behaviour.  Expected values are built from an all_gather of every rank's
input, following the layout rules of longcat_video/context_parallel/ulysses_wrapper.py:54-79
(after the exchange the sequence axis is rank-major)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, H, Sl, D, group_heads):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), LCBSA_ULYSSES_GROUP_HEADS=str(group_heads))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from longcat_video_b200.context_parallel import context_parallel_util as cpu_, ulysses_wrapper as U
        cpu_.init_context_parallel(world, rank, world)
        assert cpu_.get_cp_size() == world and cpu_.get_cp_rank() == rank
        g = torch.Generator().manual_seed(100 + rank)
        q, k, v = (torch.randn(B, H, Sl, D, generator=g) for _ in range(3))
        everyone = [torch.empty(3, B, H, Sl, D) for _ in range(world)]
        dist.all_gather(everyone, torch.stack([q, k, v]))
        hn = H // world

        def expect_in(t_index):
            return torch.cat([everyone[src][t_index][:, rank * hn:(rank + 1) * hn] for src in range(world)], dim=2)

        qi, ki, vi = U.ulysses_a2a_in(q, k, v)
        for got, ti in ((qi, 0), (ki, 1), (vi, 2)):
            assert got.shape == (B, hn, world * Sl, D)
            assert torch.equal(got, expect_in(ti))
        # inverse
        assert torch.equal(U.ulysses_a2a_out(qi), q)
        # generic entry point: same result through the reference's signature
        assert torch.equal(U.all_to_all(q, 1, 2, group=cpu_.get_cp_group()), qi)
        assert torch.equal(U.all_to_all(qi, 2, 1, group=cpu_.get_cp_group()), q)
        # strided input ([B,S,H,D] memory order, as the attention layer produces it)
        q_bshd = q.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
        assert torch.equal(U.heads_scatter_seq_gather(q_bshd, cpu_.get_cp_group()), qi)

        # the decorator, pipelined by head group, against the unpipelined composition
        class Layer:
            @U.ulysses_wrapper
            def attn(self, q_, k_, v_, shape):
                assert q_.shape[1] <= hn and q_.shape[2] == world * Sl and shape == "shape"
                return torch.softmax(q_ @ k_.transpose(-1, -2) / D ** 0.5, -1) @ v_

        got = Layer().attn(q, k, v, "shape")
        full = torch.softmax(qi @ ki.transpose(-1, -2) / D ** 0.5, -1) @ vi
        want = U.ulysses_a2a_out(full)
        assert got.shape == (B, H, Sl, D)
        assert torch.allclose(got, want, atol=1e-6)

        with pytest.raises(ValueError):
            U.heads_scatter_seq_gather(torch.zeros(B, world + 1, Sl, D), cpu_.get_cp_group())
        with pytest.raises(ValueError):
            U.all_to_all(q, 1, 1, group=cpu_.get_cp_group())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B,H,group_heads", [(2, 1, 4, 1), (2, 2, 4, 2), (4, 1, 8, 1), (2, 1, 6, 0)])
def test_ulysses_hooks(world, B, H, group_heads):
    mp.spawn(_worker, args=(world, _free_port(), B, H, 6, 8, group_heads), nprocs=world, join=True)


def test_identity_without_context_parallel():
    from longcat_video_b200.context_parallel import context_parallel_util as cpu_, ulysses_wrapper as U
    cpu_.reset_context_parallel()
    q = torch.randn(1, 2, 3, 4)
    a, b, c = U.ulysses_a2a_in(q, q, q)
    assert a is q and b is q and c is q and U.ulysses_a2a_out(q) is q
    assert U.all_to_all(q, 1, 2) is q  # process group not initialised
    assert cpu_.get_optimal_split(2) == [1, 2] and cpu_.get_optimal_split(4) == [2, 2] and cpu_.get_optimal_split(8) == [2, 4]


def test_stage_plan_of_the_context_parallel_op():
    """Host logic of flash_attn_bsa_3d_ulysses: the head ranges of the stages partition the rank's heads for every group
    size; the first stage is never larger than two heads; on eight ranks the first four heads go one by one."""
    from longcat_video_b200.context_parallel.bsa_context_parallel import _stages_scattered

    for n in (2, 4, 8):
        for hn in (1, 2, 3, 4, 5, 6, 8, 12, 16, 32):
            st = _stages_scattered(hn, n)
            assert st[0][0] == 0 and st[-1][1] == hn
            assert all(a[1] == b[0] for a, b in zip(st, st[1:])) and all(lo < hi for lo, hi in st)
            assert st[0][1] - st[0][0] <= 2
    assert _stages_scattered(4, 8) == [(0, 1), (1, 2), (2, 3), (3, 4)]
    assert _stages_scattered(8, 4) == [(0, 1), (1, 4), (4, 8)]
    assert _stages_scattered(16, 2) == [(0, 2), (2, 8), (8, 16)]
