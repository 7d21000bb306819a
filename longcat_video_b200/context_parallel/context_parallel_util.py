"""Context-parallel process state: the getters the attention layer reads.

Mirrors the part of ``longcat_video/context_parallel/context_parallel_util.py`` that the BSA path
uses (``init_context_parallel`` :13-37 and the getters :40-81): module-level ``cp_size`` /
``cp_rank`` / ``cp_group`` with the same names and meaning.  Ranks are laid out as a
``dp x cp`` mesh with the cp index fastest, the same grouping ``init_device_mesh`` produces there.
The sequence split / gather helpers of the DiT are callers of this path and are not rebuilt here.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

dp_size = dp_group = cp_group = cp_stream = dp_ranks = cp_ranks = dp_rank = None
cp_size: int = 1
cp_rank: int = 0


def init_context_parallel(context_parallel_size: int = 1, global_rank: int = 0, world_size: int = 1):
    global dp_size, cp_size, dp_group, cp_group, dp_ranks, cp_ranks, dp_rank, cp_rank
    if world_size % context_parallel_size != 0:
        raise RuntimeError(f"world_size {world_size} must be multiple of context_parallel_size {context_parallel_size}")
    cp_size = context_parallel_size
    dp_size = world_size // context_parallel_size
    # every rank creates every group, in the same order (a torch.distributed requirement)
    for d in range(dp_size):
        ranks = list(range(d * cp_size, (d + 1) * cp_size))
        grp = dist.new_group(ranks)
        if global_rank in ranks:
            cp_group, cp_ranks = grp, ranks
    for c in range(cp_size):
        ranks = list(range(c, world_size, cp_size))
        grp = dist.new_group(ranks)
        if global_rank in ranks:
            dp_group, dp_ranks = grp, ranks
    dp_rank = dist.get_rank(group=dp_group)
    cp_rank = dist.get_rank(group=cp_group)
    if cp_size > 1:
        # The attention kernel owns every SM it is given; the barrier kernel of the overlapped exchange
        # (peer_exchange) needs one to start on.  LCBSA_ATTN_SM_RESERVE overrides the two SMs kept free.
        import os

        from .. import _lib

        if _lib.lib().lcbsa_set_attn_sm_reserve(int(os.environ.get("LCBSA_ATTN_SM_RESERVE", "2"))) < 0:
            _lib.check(-1)


def reset_context_parallel():
    """Back to the single-process state (used between tests)."""
    global dp_size, cp_size, dp_group, cp_group, dp_ranks, cp_ranks, dp_rank, cp_rank, cp_stream
    dp_size = dp_group = cp_group = cp_stream = dp_ranks = cp_ranks = dp_rank = None
    cp_size, cp_rank = 1, 0


def get_cp_size():
    return cp_size


def get_dp_size():
    return dp_size


def get_cp_stream():
    """Side stream the all-to-all of the next head group is issued from."""
    global cp_stream
    if cp_stream is None:
        cp_stream = torch.cuda.Stream()
    return cp_stream


def get_dp_group():
    return dp_group


def get_cp_group():
    return cp_group


def get_dp_rank():
    return dp_rank


def get_cp_rank():
    return cp_rank


def get_cp_rank_list():
    global cp_ranks
    if cp_ranks is None:
        cp_ranks = dist.get_process_group_ranks(cp_group)
    return cp_ranks


def get_optimal_split(size):
    """(rows, cols) split of the latent H x W plane over `size` ranks, rows <= cols, closest to square
    (``context_parallel_util.py:238-243``: 2 -> (1,2), 4 -> (2,2), 8 -> (2,4))."""
    best = [1, size]
    for a in range(1, int(size ** 0.5) + 1):
        if size % a == 0:
            best = [a, size // a]
    return best
