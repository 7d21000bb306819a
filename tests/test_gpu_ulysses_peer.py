"""Two-GPU check of the Ulysses paths around the real block-sparse attention op.

  * against the CPU ORACLE: every rank holds its context-parallel slice of ONE seeded tensor; the N-GPU result,
    gathered rank-major, must match the oracle's block lists (bit for bit) and exact-softmax attention (rel-L2 <= 1e-2,
    max-abs <= 3e-2) on the gathered rank-major grid;
  * transports against each other, bit for bit (same arithmetic, different transport and order): the peer-DMA pipeline,
    the NCCL exchange without pipelining, the NCCL exchange pipelined over four stages (its receive buffers are
    recycled by the caching allocator while earlier stages still run), the context-parallel op
    ``flash_attn_bsa_3d_ulysses`` and its host-resident form.
Skipped on a box with fewer than two GPUs.  NVLS is off and every rank stays until the final barrier.  Layout rules as in
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


def _worker(rank, world, port, heads, chunk=(4, 4, 4)):
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
        local_grid = (T, Hh // sh, W // sw)
        grid = (world * T, Hh // sh, W // sw)
        Sl = local_grid[0] * local_grid[1] * local_grid[2]
        # one seeded full tensor (the same on every rank); this rank holds its slice of the H x W plane
        g = torch.Generator().manual_seed(7)
        full = [(torch.randn(1, heads, T * Hh * W, 128, generator=g) * 0.3).to(torch.bfloat16) for _ in range(3)]

        def shard(x, r):
            Hl, Wl = Hh // sh, W // sw
            rh, rw = r // sw, r % sw
            return x.view(1, heads, T, Hh, W, 128)[:, :, :, rh * Hl:(rh + 1) * Hl, rw * Wl:(rw + 1) * Wl].reshape(1, heads, Sl, 128)

        q, k, v = (shard(x, rank).contiguous().to(dev) for x in full)

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
        # against the oracle: gather the result rank-major and compare with the oracle on the gathered rank-major grid
        from oracle import bsa_oracle as O

        everyone = [torch.empty_like(want) for _ in range(world)]
        dist.all_gather(everyone, want)
        if rank == 0:
            gathered = torch.cat(everyone, dim=2).float().cpu()  # [1, H, N * S/N, D], sequence rank-major
            qg, kg, vg = (torch.cat([shard(x, r) for r in range(world)], dim=2).contiguous() for x in full)
            ref_idx, ref_cnt, _, _ = O.block_select(qg, kg, grid, grid, 0.75, chunk, chunk)
            idx, cnt = B.get_select_indices(qg.to(dev), kg.to(dev), grid, grid, 0.75, None, chunk, chunk)
            nsel = int(ref_cnt.flatten()[0])
            assert torch.equal(cnt.cpu(), ref_cnt) and torch.equal(idx.cpu()[..., :nsel], ref_idx[..., :nsel])
            ref, _ = O.attention(qg, kg, vg, grid, grid, chunk, chunk, ref_idx, ref_cnt)
            rel = float((gathered.double() - ref.double()).norm() / ref.double().norm())
            mx = float((gathered.double() - ref.double()).abs().max())
            print(f"PARITY ulysses{world} heads {heads}: lists bit-exact, rel-L2 {rel:.3e} max-abs {mx:.3e}")
            assert rel <= 1e-2 and mx <= 3e-2, (rel, mx)
        # the NCCL exchange pipelined over four stages must give the same bits as the unpipelined one
        if heads // world >= 4:
            os.environ["LCBSA_ULYSSES_GROUP_HEADS"] = str(heads // world // 4)
            for _ in range(3):
                piped = layer.attn(q, k, v, grid)
                torch.cuda.synchronize()
                assert torch.equal(piped, want)
        # the context-parallel op (local pooling, pooled rows exchanged first, one block-select for all local heads)
        from longcat_video_b200.context_parallel.bsa_context_parallel import flash_attn_bsa_3d_ulysses

        from longcat_video_b200.context_parallel import bsa_context_parallel as CP

        os.environ["LCBSA_ULYSSES_EXCHANGE"] = "peer"
        del os.environ["LCBSA_ULYSSES_GROUP_HEADS"]
        for scatter_out in (True, False, True):  # result rows stored straight into their owners' memory / sent back by copies
            CP._SCATTER_OUT = scatter_out
            for _ in range(2):
                fused = flash_attn_bsa_3d_ulysses(q, k, v, grid, sparsity=0.75, chunk_3d_shape_q=list(chunk), chunk_3d_shape_k=list(chunk))
                torch.cuda.synchronize()
                assert torch.equal(fused, want)
        # the stage plan of an eight-rank group (heads one by one, pushes queued two stages ahead), run on this group
        plan = CP._stages_scattered
        CP._stages_scattered = lambda hn, n=2: plan(hn, 8)
        try:
            for _ in range(2):
                fused = flash_attn_bsa_3d_ulysses(q, k, v, grid, sparsity=0.75, chunk_3d_shape_q=list(chunk), chunk_3d_shape_k=list(chunk))
                torch.cuda.synchronize()
                assert torch.equal(fused, want)
        finally:
            CP._stages_scattered = plan
        L.check(L.lib().lcbsa_check_device_status())
        # video continuation: the first 4 of every rank's 8 frames are conditioning frames; one exchange and one attention
        # launch per stage against the reference's formulation (two exchanges, two calls on copies, concatenated)
        kw = dict(sparsity=0.75, chunk_3d_shape_q=list(chunk), chunk_3d_shape_k=list(chunk))
        want_cond = CP._generic_cond(q, k, v, grid, 4, world, dict(kw, cdf_threshold=None))
        for _ in range(2):
            got_cond = flash_attn_bsa_3d_ulysses(q, k, v, grid, num_cond_latents=4, **kw)
            torch.cuda.synchronize()
            assert torch.equal(got_cond, want_cond)
        assert not torch.equal(got_cond, want)
        L.check(L.lib().lcbsa_check_device_status())
        # host-resident form: pinned shards in, pinned result out, pipelined by head chunk
        from longcat_video_b200.context_parallel.bsa_context_parallel import flash_attn_bsa_3d_ulysses_host

        qh, kh, vh = (t.cpu().pin_memory() for t in (q, k, v))
        oh = torch.empty_like(qh).pin_memory()
        for _ in range(2):
            oh.zero_()
            flash_attn_bsa_3d_ulysses_host(qh, kh, vh, grid, out=oh, heads_per_chunk=max(world, heads // 2), sparsity=0.75,
                                           chunk_3d_shape_q=list(chunk), chunk_3d_shape_k=list(chunk))
            assert torch.equal(oh, want.cpu())
        L.check(L.lib().lcbsa_check_device_status())
    finally:
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.parametrize("heads,chunk", [(4, (4, 4, 4)), (8, (4, 4, 4)), (16, (4, 4, 4)), (4, (4, 4, 8))])
def test_peer_exchange_matches_nccl(heads, chunk):
    """(4, 4, 8): the 128-token blocks that flash_attn_bsa_3d takes by default, served by the other tcgen05 kernel."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), heads, chunk), nprocs=2, join=True)
