"""Two-GPU check of the Ulysses pipeline with the peer-DMA exchange (symmetric buffers, copy engines) against the
NCCL exchange without pipelining, around the real block-sparse attention op, and of the context-parallel op
`flash_attn_bsa_3d_ulysses`: the results must be identical bit for bit (same arithmetic, different transport and order).  Skipped on a box with fewer than two GPUs.  Layout rules as in
longcat_video/context_parallel/ulysses_wrapper.py:54-79 and longcat_video/modules/attention.py:60-66."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, heads):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from longcat_video_b200 import _lib as L
        from longcat_video_b200.block_sparse_attention import bsa_interface as B
        from longcat_video_b200.context_parallel import context_parallel_util as cpu_, ulysses_wrapper as U

        assert L.lib().lcbsa_set_attn_sm_reserve(2) >= 0
        cpu_.init_context_parallel(world, rank, world)
        sh, sw = cpu_.get_optimal_split(world)
        T, Hh, W = 8, 16, 16
        chunk = (4, 4, 4)
        local_grid = (T, Hh // sh, W // sw)
        grid = (world * T, Hh // sh, W // sw)
        Sl = local_grid[0] * local_grid[1] * local_grid[2]
        g = torch.Generator().manual_seed(7 + rank)
        q, k, v = ((torch.randn(1, heads, Sl, 128, generator=g) * 0.3).to(torch.bfloat16).to(dev) for _ in range(3))

        class Layer:
            @U.ulysses_wrapper
            def attn(self, q_, k_, v_, shape):
                return B.flash_attn_bsa_3d(q_, k_, v_, shape, shape, sparsity=0.75, chunk_3d_shape_q=list(chunk),
                                           chunk_3d_shape_k=list(chunk))

        layer = Layer()
        os.environ["LCBSA_ULYSSES_EXCHANGE"] = "peer"
        got = [layer.attn(q, k, v, grid).clone() for _ in range(3)]  # repeated calls reuse the exchange buffers
        os.environ["LCBSA_ULYSSES_EXCHANGE"] = "nccl"
        os.environ["LCBSA_ULYSSES_GROUP_HEADS"] = "0"
        want = layer.attn(q, k, v, grid)
        torch.cuda.synchronize()
        L.check(L.lib().lcbsa_check_device_status())
        assert want.shape == q.shape
        assert float(want.float().abs().max()) > 0
        for o in got:
            assert torch.equal(o, want)
        # the context-parallel op (local pooling, pooled rows exchanged first, one block-select for all local heads)
        from longcat_video_b200.context_parallel.bsa_context_parallel import flash_attn_bsa_3d_ulysses

        os.environ["LCBSA_ULYSSES_EXCHANGE"] = "peer"
        del os.environ["LCBSA_ULYSSES_GROUP_HEADS"]
        for _ in range(2):
            fused = flash_attn_bsa_3d_ulysses(q, k, v, grid, sparsity=0.75, chunk_3d_shape_q=list(chunk), chunk_3d_shape_k=list(chunk))
            torch.cuda.synchronize()
            assert torch.equal(fused, want)
        L.check(L.lib().lcbsa_check_device_status())
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [4, 16])
def test_peer_exchange_matches_nccl(heads):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), heads), nprocs=2, join=True)
