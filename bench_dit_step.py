"""One denoising-step forward of the LongCat-Video DiT block stack with the drop-in block-sparse attention against the
reference's own attention, on the same GPU(s), same weights, same inputs.

    python bench_dit_step.py [--blocks 4] [--steps 5] [--warmup 2] [--grid 24 32 52]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_dit_step.py ...

The stack is the reference's ``LongCatSingleStreamBlock`` (longcat_video/modules/longcat_video_dit.py:21-121), unmodified,
loaded from ``baseline/_ref`` (baseline/install_reference.py): hidden 4096, 32 heads x 128, SwiGLU FFN x4, random bf16
weights, text cross-attention over 512 tokens, BSA (4x4x4 blocks, sparsity 0.9375) in every self-attention, the loop of
longcat_video_dit.py:336-346 over ``--blocks`` of the model's 48 blocks (the per-block time is what is reported; a
block's weights are 0.57 GB, so the count only bounds memory and run time).  ``diffusers`` is not needed by the block
itself; its three names that ``longcat_video_dit.py`` imports at module level are stubbed.

Two arms on identical modules:
  reference  ``Attention._process_attn`` as written: ulysses_wrapper(flash_attn_bsa_3d) with the Triton kernels
  drop-in    the module global ``longcat_video.modules.attention.flash_attn_bsa_3d`` rebound to this library's op
             (one GPU), or ``Attention._process_attn`` rebound to ``flash_attn_bsa_3d_ulysses`` (context parallel)
Rank 0 prints ONE JSON line: ms per block for both arms, the attention's share, and the difference of the outputs.
Latent grid: the reference-legal twin 24x32x52 of the 480p grid (the reference asserts divisibility by the block); under
context parallelism 24x32x64, whose H x W plane splits over 2, 4 and 8 ranks into parts that divide by the block.
Synthetic N(0,1) activations and N(0, 0.02) weights; no checkpoint or dataset is involved.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import types

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
REF_ROOT = os.path.join(ROOT, "baseline", "_ref")


def load_reference():
    """Import the reference's DiT block from baseline/_ref with the three diffusers names stubbed."""
    if not os.path.isdir(os.path.join(REF_ROOT, "longcat_video", "modules")):
        return None, "baseline/_ref/longcat_video/modules is absent (run baseline/install_reference.py where the reference checkout is)"
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    for name in ("diffusers", "diffusers.configuration_utils", "diffusers.models", "diffusers.models.modeling_utils"):
        sys.modules.setdefault(name, types.ModuleType(name))
    cu, mu = sys.modules["diffusers.configuration_utils"], sys.modules["diffusers.models.modeling_utils"]
    if not hasattr(cu, "ConfigMixin"):
        cu.ConfigMixin = type("ConfigMixin", (object,), {})
        cu.register_to_config = lambda f: f
    if not hasattr(mu, "ModelMixin"):
        mu.ModelMixin = type("ModelMixin", (torch.nn.Module,), {})
    try:
        with contextlib.redirect_stdout(sys.stderr):
            from longcat_video.modules import attention as ref_attention
            from longcat_video.modules import longcat_video_dit as ref_dit
            from longcat_video.context_parallel import context_parallel_util as ref_cp
    except Exception as e:  # noqa: BLE001
        return None, f"import failed: {e!r}"[:300]
    return (ref_attention, ref_dit, ref_cp), ""


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--blocks", type=int, default=4)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--grid", type=int, nargs=3, default=None,
                    help="latent grid; default 24 32 52 on one GPU (the legal twin of 480p), 24 32 64 under context parallelism "
                         "(every rank's part of the H x W plane must divide by the 4x4 block)")
    ap.add_argument("--sparsity", type=float, default=0.9375)
    ap.add_argument("--text-tokens", type=int, default=512)
    args = ap.parse_args()

    world, rank, local_rank = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    if args.grid is None:
        args.grid = [24, 32, 52] if world == 1 else [24, 32, 64]
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    mods, why = load_reference()
    if mods is None:
        if rank == 0:
            print(json.dumps({"bench": "dit_step", "unavailable": why}))
        return
    ref_attention, ref_dit, ref_cp = mods

    import torch.distributed as dist
    from longcat_video_b200.block_sparse_attention import bsa_interface as B
    from longcat_video_b200.context_parallel import context_parallel_util as our_cp
    from longcat_video_b200.context_parallel.bsa_context_parallel import flash_attn_bsa_3d_ulysses

    T, Hh, W = args.grid
    split = [1, 1]
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        ref_cp.init_context_parallel(context_parallel_size=world, global_rank=rank, world_size=world)
        our_cp.init_context_parallel(world, rank, world)
        split = list(our_cp.get_optimal_split(world))
    if Hh % split[0] or W % split[1] or (Hh // split[0]) % 4 or (W // split[1]) % 4 or T % 4:
        raise SystemExit(f"grid {args.grid} does not split {split} into parts that divide by the 4x4x4 block")
    n_local = T * (Hh // split[0]) * (W // split[1])
    hidden, heads, tdim = 4096, 32, 512
    bsa_params = dict(sparsity=args.sparsity, cdf_threshold=None, chunk_3d_shape_q=[4, 4, 4], chunk_3d_shape_k=[4, 4, 4])

    torch.manual_seed(1234)  # the same weights on every rank
    blocks = []
    with torch.device(dev):
        for _ in range(args.blocks):
            blk = ref_dit.LongCatSingleStreamBlock(hidden, heads, 4, tdim, enable_flashattn2=True, enable_bsa=True, bsa_params=bsa_params,
                                                   cp_split_hw=split)
            for p in blk.parameters():
                if p.dim() > 1:
                    torch.nn.init.normal_(p, std=0.02)
            blocks.append(blk.to(torch.bfloat16).eval())
    g = torch.Generator(device=dev).manual_seed(99 + rank)
    x0 = torch.randn(1, n_local, hidden, generator=g, device=dev, dtype=torch.bfloat16)
    g2 = torch.Generator(device=dev).manual_seed(7)
    y = torch.randn(1, args.text_tokens, hidden, generator=g2, device=dev, dtype=torch.bfloat16)
    t = torch.randn(1, T, tdim, generator=g2, device=dev, dtype=torch.float32)
    latent_shape = (T, Hh, W)

    def forward():
        x = x0
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            for blk in blocks:  # the loop of longcat_video_dit.py:336-346
                x = blk(x, y, t, [args.text_tokens], latent_shape)
        return x

    original_process = ref_attention.Attention._process_attn
    original_op = ref_attention.flash_attn_bsa_3d
    attn_events = []

    # The text cross-attention is not part of the path under test; it runs through flash_attn 2 as the reference has it
    # when that library has kernels for this GPU, else through torch's scaled_dot_product_attention, in BOTH arms.
    cross_note = "flash_attn 2 (as in the reference)"
    try:
        from flash_attn import flash_attn_varlen_func
        qq = torch.randn(64, 2, 128, device=dev, dtype=torch.bfloat16)
        cu = torch.tensor([0, 64], device=dev, dtype=torch.int32)
        flash_attn_varlen_func(q=qq, k=qq, v=qq, cu_seqlens_q=cu, cu_seqlens_k=cu, max_seqlen_q=64, max_seqlen_k=64)
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        cross_note = f"torch SDPA in both arms (flash_attn 2 unusable here: {e!r})"[:200]

        def sdpa_cross(self, x, cond, kv_seqlen):
            Bx, N, C = x.shape
            q = self.q_linear(x).view(Bx, N, self.num_heads, self.head_dim)
            kv = self.kv_linear(cond).view(Bx, -1, 2, self.num_heads, self.head_dim)
            k, v = kv.unbind(2)
            q, k = self.q_norm(q), self.k_norm(k)
            o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
            return self.proj(o.transpose(1, 2).reshape(Bx, N, C))

        ref_attention.MultiHeadCrossAttention._process_cross_attn = sdpa_cross

    def timed(fn):
        def wrapper(self, q, k, v, shape):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = fn(self, q, k, v, shape)
            b.record()
            attn_events.append((a, b))
            return out
        return wrapper

    def drop_in_process(self, q, k, v, shape):
        # context parallel: what ulysses_wrapper(Attention._process_attn) does (attention.py:49-67, ulysses_wrapper.py:108-116)
        # as this library's one op; q, k, v are this rank's [B, H, S/N, D] tensors
        _, Hs, Ws = shape
        Hl, Wl = Hs // self.cp_split_hw[0], Ws // self.cp_split_hw[1]
        return flash_attn_bsa_3d_ulysses(q.contiguous(), k.contiguous(), v.contiguous(), (world * (q.shape[2] // (Hl * Wl)), Hl, Wl),
                                         **self.bsa_params)

    def run_arm(drop_in):
        # one GPU: the drop-in is the rebound module global, exactly as INTEGRATION.md describes; the layer's own
        # _process_attn runs unchanged above it.  Context parallel: _process_attn itself is rebound.
        attn_events.clear()
        if drop_in and world == 1:
            ref_attention.flash_attn_bsa_3d = B.flash_attn_bsa_3d
        ref_attention.Attention._process_attn = timed(drop_in_process if (drop_in and world > 1) else original_process)
        try:
            with contextlib.redirect_stdout(sys.stderr):
                for _ in range(args.warmup):
                    out = forward()
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                attn_events.clear()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(args.steps):
                    out = forward()
                b.record()
                torch.cuda.synchronize()
            ms = a.elapsed_time(b) / args.steps / args.blocks
            ms_attn = sum(s.elapsed_time(e) for s, e in attn_events) / args.steps / args.blocks
            if world > 1:
                tt = torch.tensor([ms, ms_attn], device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                ms, ms_attn = float(tt[0]), float(tt[1])
            return out, ms, ms_attn
        finally:
            ref_attention.Attention._process_attn = original_process
            ref_attention.flash_attn_bsa_3d = original_op

    result = {"bench": "dit_step", "n_gpus": world, "blocks": args.blocks, "of_model_blocks": 48, "grid": list(args.grid),
              "tokens": T * Hh * W, "tokens_per_gpu": n_local, "hidden": hidden, "heads": heads, "text_tokens": args.text_tokens,
              "sparsity": args.sparsity, "steps": args.steps, "warmup": args.warmup, "dtype": "bf16", "data": "synthetic",
              "torch": torch.__version__}
    result["cross_attention"] = cross_note
    out_ours, ms_ours, attn_ours = run_arm(True)
    result["drop_in"] = {"ms_per_block": ms_ours, "ms_self_attention_op": attn_ours}
    try:
        out_ref, ms_ref, attn_ref = run_arm(False)
        diff = (out_ours.float() - out_ref.float())
        result["reference"] = {"ms_per_block": ms_ref, "ms_self_attention_op": attn_ref}
        result["speedup_per_block"] = ms_ref / ms_ours
        result["speedup_self_attention_op"] = attn_ref / attn_ours
        result["output_rel_l2_vs_reference"] = float(diff.norm() / out_ref.float().norm())
    except Exception as e:  # noqa: BLE001 - e.g. the reference's Triton kernels do not compile on this box
        result["reference"] = {"unavailable": f"{e!r}"[:300]}
    assert ref_attention.flash_attn_bsa_3d is original_op
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
