"""The golden cases: seeded workloads small enough to commit the reference's outputs for."""
import torch

from longcat_video_b200.synthetic import Workload

CASES = {
    # name: (workload, store_attention)
    "cfg1_fp32": (Workload("cfg1_fp32", 1001, 1, 4, 128, (4, 8, 8), (4, 8, 8), (4, 4, 4), 0.5,
                           torch.float32, "normal"), True),
    "bf16_lowrank": (Workload("bf16_lowrank", 2002, 1, 1, 128, (8, 16, 16), (8, 16, 16), (4, 4, 4), 0.75,
                              torch.bfloat16, "scaled_lowrank"), True),
    "bf16_chunk448": (Workload("bf16_chunk448", 2003, 1, 2, 128, (8, 8, 16), (8, 8, 16), (4, 4, 8), 0.5,
                               torch.bfloat16, "normal"), True),
    "bf16_cross": (Workload("bf16_cross", 2004, 1, 2, 128, (4, 8, 16), (12, 8, 16), (4, 4, 4), 0.875,
                            torch.bfloat16, "normal"), True),
    "fp16_d64": (Workload("fp16_d64", 2005, 1, 3, 64, (4, 8, 8), (4, 8, 8), (2, 4, 8), 0.5,
                          torch.float16, "normal"), True),
    # selection only, at the scale where bf16 score ties decide many rows (720p bucket grid, 1 head)
    "bf16_ties_720p": (Workload("bf16_ties_720p", 1003, 1, 1, 128, (24, 44, 80), (24, 44, 80), (4, 4, 4), 0.9375,
                                torch.bfloat16, "scaled_lowrank"), False),
}

# Backward: gradients of the reference's "block-select + masked SDPA" path under torch autograd (make_golden_backward.py)
BWD_CASES = {
    "bwd_blocks64": Workload("bwd_blocks64", 8001, 1, 1, 128, (4, 8, 8), (4, 8, 8), (4, 4, 4), 0.5, torch.bfloat16, "normal"),
    "bwd_blocks128_cross": Workload("bwd_blocks128_cross", 8002, 1, 1, 128, (4, 8, 8), (8, 8, 8), (4, 4, 8), 0.5, torch.bfloat16, "normal"),
    "bwd_fp16_d64": Workload("bwd_fp16_d64", 8003, 1, 2, 64, (4, 8, 8), (4, 8, 8), (2, 4, 8), 0.5, torch.float16, "normal"),
}


def make_dout(wl: Workload) -> torch.Tensor:
    """The seeded upstream gradient of a backward case, ``[B, H, Sq, D]`` in the case's dtype."""
    g = torch.Generator().manual_seed(wl.seed + 7)
    return (torch.randn(wl.batch, wl.heads, wl.sq, wl.head_dim, generator=g) * 0.5).to(wl.dtype)
