/*
 * lcbsa -- B200-native block-sparse attention (BSA) forward for LongCat-Video.
 *
 * C ABI of liblcbsa.so.  Every entry point takes plain pointers and sizes; all buffers
 * (inputs, outputs, workspace) are device memory owned by the caller; launches are
 * asynchronous on the stream that is passed in (a cudaStream_t cast to void*).
 *
 * Every function that returns int returns LCBSA_OK (0) or a negative LCBSA_E* code;
 * lcbsa_last_error() then gives a message for the calling thread.  Arguments are validated
 * on the host before anything is launched; no entry point aborts or traps the device.
 *
 * Citations name files of the LongCat-Video project that each entry point stands in for.
 */
#ifndef LCBSA_H_
#define LCBSA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LCBSA_VERSION 100

enum {
    LCBSA_OK = 0,
    LCBSA_EINVAL = -1,       /* bad argument (shape, dtype, alignment, null pointer) */
    LCBSA_EUNSUPPORTED = -2, /* valid request that no kernel here covers */
    LCBSA_EWORKSPACE = -3,   /* workspace smaller than lcbsa_*_workspace_bytes() says */
    LCBSA_ECUDA = -4,        /* a CUDA runtime / driver call failed */
    LCBSA_EDEVICE = -5       /* a kernel flagged a problem it met on the device: a bounded wait that ran out,
                                or a block list entry outside [0, Nk) (lcbsa_check_device_status) */
};

enum { LCBSA_BF16 = 0, LCBSA_FP16 = 1, LCBSA_FP32 = 2 };

/* Which attention kernel lcbsa_attn_fwd runs. */
enum {
    LCBSA_ATTN_AUTO = 0, /* tcgen05 kernel when the shape allows it, otherwise the generic one */
    LCBSA_ATTN_TC = 1,   /* TMA + tcgen05 + TMEM kernel (head_dim 128, 64-token blocks, bf16/fp16) */
    LCBSA_ATTN_MMA = 2   /* generic warp-level MMA kernel (other block sizes / head dims) */
};

/* A [B, H, S, D] tensor as the DiT's attention layer hands it over
 * (longcat_video/modules/attention.py:107-121): any B/H/S strides (in elements), D contiguous. */
typedef struct LcbsaTensor {
    void* data;
    int32_t dtype; /* LCBSA_BF16 | LCBSA_FP16 | LCBSA_FP32 */
    int32_t reserved;
    int64_t size[4];
    int64_t stride[4];
} LcbsaTensor;

/* Latent grid (T,H,W tokens, S = T*H*W) and the 3-D block ("chunk") that tiles it:
 * latent_shape_* and chunk_3d_shape_* of flash_attn_bsa_3d
 * (longcat_video/block_sparse_attention/bsa_interface.py:612-623). */
typedef struct LcbsaGrid {
    int32_t T, H, W;
    int32_t ct, ch, cw;
} LcbsaGrid;

int lcbsa_version(void);

/* Message of the last failing call made by this thread ("" if none). */
const char* lcbsa_last_error(void);

/* Number of 3-D blocks of a grid (partial edge blocks count). */
int lcbsa_num_blocks(const LcbsaGrid* g);

/* int((1 - sparsity) * n_k_blocks) evaluated in double precision, i.e. exactly what
 * bsa_interface.py:214 computes in Python. */
int lcbsa_num_selected(double sparsity, int n_k_blocks);

/*
 * Mean-pool x over every 3-D block without rearranging it first.
 * Stands in for rearrange_THW_to_3d_block + mean_pooling_compression
 * (bsa_interface.py:600-604, 168-178).
 * out: dense [B, H, Nblk, D], dtype of x.
 */
int lcbsa_pool(const LcbsaTensor* x, const LcbsaGrid* g, void* out, void* stream);

/*
 * lcbsa_pool for q and k of a context-parallel rank in ONE launch, with the pooled rows stored where the block-select
 * of the Ulysses-gathered tensors will read them: every rank of the group holds q, k as [1, H, S/N, D] (all heads, its
 * own tokens; longcat_video/context_parallel/ulysses_wrapper.py:86-95 would all-to-all them), pools the 3-D blocks of
 * ITS tokens for all heads and writes the rows of head h straight into the buffer of the rank that owns that head
 * (rank h / (H/N)): dst_q[r], dst_k[r] are that rank's buffers (this GPU's memory or a peer's, mapped into this
 * process), each [H/N][N source ranks][nblk][D] in the tensor dtype, and this call fills source slot `rank`.  Once
 * every rank has made the call (and the group has synchronised), each buffer is the dense pooled tensor
 * [H/N, N * nblk, D] of the gathered rank-major sequence.  The stores to peers are ordinary global stores issued by the
 * kernel.  No counterpart in the reference, which exchanges the full tensors first and pools afterwards
 * (bsa_interface.py:547-548).  Batch 1, up to 8 ranks.
 */
int lcbsa_pool_scatter(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk,
                       void* const* dst_q, void* const* dst_k, int n_ranks, int rank, void* stream);

/*
 * Block scores and per-row top-k from pooled tensors; the scores never reach HBM.
 * Stands in for cal_score + get_select_indices_topk_from_score (bsa_interface.py:180-184, 212-224).
 * q_cmp: dense [BH, Nq, D]; k_cmp: dense [BH, Nk, D]; dtype as given.
 * idx: int32 [BH, Nq, cap]; the first nsel entries of a row are the selected K-blocks in
 *      ascending block order, the rest are -1.   cnt: int32 [BH, Nq] (= nsel).
 * Ties: rows are ordered by (score descending, block index ascending).
 */
int lcbsa_score_topk(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D,
                     int nsel, int cap, int32_t* idx, int32_t* cnt, void* stream);

/*
 * lcbsa_score_topk with a workspace for the scores: with keys_bytes >= lcbsa_score_keys_bytes(...) (one 16-bit key
 * per score; 0 when the form does not apply: fp32, head_dim other than 64 or 128) the scores are computed by a
 * register-tiled GEMM kernel into the workspace and a second kernel selects per row; otherwise this is
 * lcbsa_score_topk.  Same results either way.
 */
size_t lcbsa_score_keys_bytes(int dtype, int BH, int Nq, int Nk, int D);
int lcbsa_score_topk_ws(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D, int nsel, int cap,
                        int32_t* idx, int32_t* cnt, void* keys_ws, size_t keys_bytes, void* stream);

/*
 * Bytes of workspace with which lcbsa_block_select takes its faster form: pooled Q and K plus one 16-bit key per
 * block score (B*H*Nq*Nk_padded*2 bytes), which lets the scores be computed by a register-tiled GEMM kernel and the
 * rows be selected by a second kernel.  Results are identical to the fused form.  Equal to
 * lcbsa_select_workspace_bytes when that form does not apply (fp32 inputs, head_dim other than 64 or 128).
 */
size_t lcbsa_select_workspace_bytes_fast(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq,
                                         const LcbsaGrid* gk);

/* Bytes of workspace lcbsa_block_select needs (pooled Q and pooled K). */
size_t lcbsa_select_workspace_bytes(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq,
                                    const LcbsaGrid* gk);

/*
 * A latent grid with a "first part": the conditioning frames of video continuation, which attend among themselves while
 * all other frames attend to everything (Attention.forward, longcat_video/modules/attention.py:124-137, where this
 * is two _process_attn calls on copies).  Blocks are numbered frame-major; a block is in the first part when
 * ((block / hw) % period) < split, with hw = blocks per frame-block plane, period = frame blocks of the whole grid
 * (or of one rank's share of the rank-major grid of a context-parallel group) and split = conditioning frame blocks.
 * Query blocks of the first part select nsel_first key blocks among the key blocks of the first part; every other
 * query block selects as usual among all key blocks.  One table holds both kinds of rows; rows of the first part are
 * padded with -1 beyond nsel_first.
 */
typedef struct LcbsaSplit {
    int32_t hw_q, period_q, split_q;
    int32_t hw_k, period_k, split_k;
    int32_t nsel_first;
} LcbsaSplit;

/* lcbsa_score_topk_ws for a grid with a first part; needs the key workspace (bf16 / fp16, head_dim 64 or 128, up to
 * 1536 key blocks). */
int lcbsa_score_topk_split(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D, const LcbsaSplit* split,
                           int nsel, int cap, int32_t* idx, int32_t* cnt, void* keys_ws, size_t keys_bytes, void* stream);

/* lcbsa_block_select for a grid with a first part (periods and splits in frame blocks); needs the workspace of
 * lcbsa_select_workspace_bytes_fast. */
int lcbsa_block_select_split(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk, int period_tq,
                             int split_tq, int period_tk, int split_tk, int nsel_first, int nsel, int cap, int32_t* idx,
                             int32_t* cnt, void* workspace, size_t workspace_bytes, void* stream);

/*
 * The whole block-select stage: pool Q and K, score, top-k.
 * Stands in for the gating part of _attention_bsa.forward (bsa_interface.py:547-549) with
 * cdf_threshold=None.  idx/cnt as in lcbsa_score_topk with BH = B*H.
 */
int lcbsa_block_select(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk,
                       int nsel, int cap, int32_t* idx, int32_t* cnt, void* workspace, size_t workspace_bytes,
                       void* stream);

/*
 * Block-sparse flash-attention forward over the listed K/V blocks, reading q/k/v and writing
 * out directly in T,H,W token order.
 * Stands in for the three rearrange_THW_to_3d_block copies, attn_fwd_bsa_varlen_triton and
 * rearrange_3d_block_to_THW (bsa_interface.py:650-659, 290-341) and the Triton kernels
 * _attn_fwd_bsa_varlen_align / _attn_fwd_bsa_varlen (flash_attn_bsa_varlen_mask.py:172-285, 35-153).
 * idx: int32 [B*H, Nq, cap], cnt: int32 [B*H, Nq] (entries beyond cnt are ignored; cnt is clamped to [0, cap]).
 *      An entry outside [0, Nk) is never turned into an address: the generic kernel skips that block, the tcgen05
 *      kernel reads zeros for it; either way the device status is flagged (lcbsa_check_device_status returns
 *      LCBSA_EDEVICE naming the entry) and the rows of that query block are finite but unspecified.
 * out: [B, H, Sq, D], dtype of q.   lse: nullable, fp32 dense [B*H, Sq], natural log.
 * impl: LCBSA_ATTN_*.
 */
int lcbsa_attn_fwd(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaTensor* v, const LcbsaGrid* gq,
                   const LcbsaGrid* gk, const int32_t* idx, const int32_t* cnt, int cap, float sm_scale,
                   const LcbsaTensor* out, float* lse, int impl, void* stream);

/*
 * lcbsa_attn_fwd for a context-parallel rank, with the return all-to-all folded into the kernel's output stores
 * (tcgen05 kernel: head_dim 128, 64-token blocks, bf16/fp16, batch 1, grid divisible by the block).  q, k, v are the
 * rank's heads of the Ulysses-gathered tensors, [1, h, S, D] over the rank-major grid gq (frames
 * [r * T/n, (r+1) * T/n) are the tokens of rank r; longcat_video/modules/attention.py:60-66).  Instead of writing
 * [1, h, S, D] and exchanging it back (ulysses_a2a_out, longcat_video/context_parallel/ulysses_wrapper.py:98-105), the
 * rows of rank r's tokens are stored straight into out_dst[r]: that rank's result for these h heads, a [1, h, S/n, D]
 * tensor (this GPU's memory or a peer's, mapped into this process) with the given head and token strides in
 * elements, head_dim contiguous.  The stores are TMA stores issued by the kernel; no load ever touches peer memory.
 * The caller synchronises the group before any rank reads its result.  No counterpart in the reference.
 */
int lcbsa_attn_fwd_scatter(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaTensor* v, const LcbsaGrid* gq,
                           const LcbsaGrid* gk, const int32_t* idx, const int32_t* cnt, int cap, float sm_scale,
                           void* const* out_dst, int n_dst, int64_t out_head_stride, int64_t out_token_stride, void* stream);

/*
 * Backward of lcbsa_attn_fwd for fixed block lists: dq, dk, dv from dout.  Replaces attn_bwd_bsa_varlen_triton and
 * its Triton kernels (longcat_video/block_sparse_attention/bsa_interface.py:343-461,
 * flash_attn_bsa_varlen_mask.py:289-945), i.e. the body of _attention_bsa.backward (bsa_interface.py:570-596).  No
 * gradient flows through the selection.  q, k, v, out, dout and the gradients are [B,H,S,D] descriptors with any
 * strides (T,H,W token order, D contiguous); idx, cnt, cap are the lists the forward ran with and lse is the
 * [B*H, Sq] fp32 log-sum-exp (natural log) that the forward returned.  bf16 or fp16, head_dim 64 or 128, block sizes
 * multiples of 64 tokens.  The workspace (lcbsa_attn_bwd_workspace_bytes, 256-byte aligned) holds delta =
 * rowsum(dout * out) and, for every key block, the ascending list of the query blocks that selected it (built through a
 * bitmap of (key block, query block) pairs; the entries of one list are taken as distinct); no atomics on the gradients,
 * so two calls give the same bits.  Every row of dq, dk, dv that exists is written (rows of blocks that nothing selected
 * get zeros).  head_dim 128 runs on tcgen05 (TMA tiles, accumulators in TMEM; a CTA owns a block of 64 or 128
 * tokens, larger blocks are taken as 64-token units; on ragged grids 64-token blocks in bf16); head_dim 64 and the
 * remaining ragged cases on warp-level MMAs, with the same bits for 64-token blocks (the environment
 * variable LCBSA_BWD_IMPL=mma keeps the warp-level kernels, for comparisons).
 */
size_t lcbsa_attn_bwd_workspace_bytes(const LcbsaTensor* q, const LcbsaGrid* gq, const LcbsaGrid* gk, int cap);
int lcbsa_attn_bwd(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaTensor* v, const LcbsaTensor* out, const LcbsaTensor* dout,
                   const LcbsaGrid* gq, const LcbsaGrid* gk, const int32_t* idx, const int32_t* cnt, int cap, float sm_scale,
                   const float* lse, const LcbsaTensor* dq, const LcbsaTensor* dk, const LcbsaTensor* dv, void* workspace,
                   size_t workspace_bytes, void* stream);

/*
 * lcbsa_block_select for callers that cannot allocate device memory for the workspace (a frozen
 * memory pool, a plugin that only receives its input and output buffers, code that must not touch the
 * CUDA allocator).  No counterpart in the reference: there the workspace is whatever PyTorch allocates.
 * The scratch is a device array built into the library, lcbsa_static_scratch_bytes() (32 MiB) per
 * GPU, reserved on every GPU that loads the library until the process exits.  Problems whose pooled Q
 * and K do not fit are refused with LCBSA_EWORKSPACE.  The call allocates nothing; it launches what
 * lcbsa_block_select launches on a workspace of that size: pool, score GEMM and top-k kernels with the
 * 16-bit score keys also in the array when lcbsa_select_workspace_bytes_fast() fits in it, else the pool
 * kernel and the fused score + top-k kernel.  All calls on one device share the array: calls that can
 * overlap on the GPU race and must be ordered by the caller.  The first call on a device resolves
 * the array's address and should be made outside stream capture.
 */
size_t lcbsa_static_scratch_bytes(void);
int lcbsa_block_select_static(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk,
                              int nsel, int cap, int32_t* idx, int32_t* cnt, void* stream);

/*
 * Number of SMs that lcbsa_attn_fwd leaves idle (0..64, default 0; process-wide).  The attention kernel is
 * persistent with one CTA per SM and all of an SM's shared memory, so nothing else can start beside it; a caller
 * that overlaps it with communication kernels on another stream (the all-to-all of
 * longcat_video/context_parallel/ulysses_wrapper.py:7-83) reserves a few SMs for them.  No counterpart in the
 * reference.  Returns the previous value, or LCBSA_EINVAL.
 */
int lcbsa_set_attn_sm_reserve(int n_sms);

/*
 * The cdf_threshold selectors: get_select_indices_cdf and get_select_indices_cdf_topk
 * (longcat_video/block_sparse_attention/bsa_interface.py:226-266) on pooled rows q_cmp [BH, Nq, D], k_cmp [BH, Nk, D]
 * (bf16 / fp16, head_dim 64 or 128, Nk <= 4096).  Per row of block scores: weights = softmax(score * sm_scale) in the
 * input dtype, the whole row sorted by descending weight (equal weights by ascending index; torch.sort leaves that
 * open), cdf = running sum of the sorted weights rounded to the dtype, count = number of entries with
 * cdf <= cdf_threshold, raised to nsel_min (0 for the cdf selector, int((1 - sparsity) * Nk) for the combined one).
 * idx: int32 [BH, Nq, Nk], the sorted index rows (the reference returns them as int64); cnt: int32 [BH, Nq]; both go to
 * lcbsa_attn_fwd with cap = Nk.  keys_ws: lcbsa_score_keys_bytes(...) bytes of scratch.
 */
int lcbsa_score_cdf(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D, float sm_scale, float cdf_threshold,
                    int nsel_min, int32_t* idx, int32_t* cnt, void* keys_ws, size_t keys_bytes, void* stream);

/*
 * The step in front of the BSA path, for q and for k (one call each): RMSNorm in fp32 over head_dim times the
 * learned weight, then the 3-D rotary embedding, in one pass from the strided [B, H, S, D] view of the fused qkv
 * projection into `out` (any B/H/S strides, e.g. the layout the attention or the Ulysses exchange reads).  Stands in
 * for q_norm / k_norm followed by rope_3d in Attention.forward (longcat_video/modules/attention.py:113-121), i.e.
 * RMSNorm_FP32.forward (longcat_video/modules/blocks.py:42-53) and RotaryPositionalEmbedding.forward
 * (longcat_video/modules/rope_3d.py:99-120).  bf16 / fp16, head_dim 64 or 128; weight: [D] in the tensor dtype, 16-byte aligned.
 * Only T, H, W of the grid are read (the chunk fields must still be positive).
 *
 * rope_tab is the reference's [S, D] cos / sin tables (rope_3d.py:62-97) in the separable form they are built
 * from, fp32, lcbsa_rope_table_floats(grid, D) floats (0 for a bad grid or odd D), with dh = 2 * (D / 6) and
 * dt = D - 2 * dh:  cos_t [T, dt]  sin_t [T, dt]  cos_h [H, dh]  sin_h [H, dh]  cos_w [W, dh]  sin_w [W, dh],
 * each entry repeated for the two elements of a rotation pair as in the reference's tables.
 */
size_t lcbsa_rope_table_floats(const LcbsaGrid* grid, int D);
int lcbsa_norm_rope(const LcbsaTensor* x, const void* weight, const LcbsaGrid* grid, const float* rope_tab, float eps,
                    const LcbsaTensor* out, void* stream);

/*
 * The same kernel with its parts switchable, for the KV-cache path (longcat_video/modules/attention.py:118-119 and
 * 149-171): weight == NULL skips the normalisation (keys that were cached after q_norm / k_norm and before rope_3d),
 * rope_tab == NULL skips the rotary embedding (what return_kv caches), and the token at grid position (t, h, w) takes
 * the angles of frame t + t_offset of a table built for table_T >= grid->T + t_offset frames (the new tokens behind
 * num_cond_latents cached frames, attention.py:165-169, without padding q).
 */
int lcbsa_norm_rope_ex(const LcbsaTensor* x, const void* weight, const LcbsaGrid* grid, const float* rope_tab, int table_T, int t_offset,
                       float eps, const LcbsaTensor* out, void* stream);

/*
 * Enqueue `count` device-to-device copies of `nbytes` each on `stream`: dst[i] <- src[i], one cudaMemcpyAsync per
 * slab, so the copy engines move them; a destination may be another GPU's memory mapped into this process
 * (symmetric memory, CUDA IPC).  The pointer arrays are host memory and are read before the call returns.
 * This is how the Ulysses exchange (longcat_video/context_parallel/ulysses_wrapper.py:7-83, NCCL all_to_all there)
 * moves its [S/N, D] slabs without taking an SM from the attention kernel.  No counterpart in the reference.
 */
int lcbsa_copy_slabs(void* const* dst, const void* const* src, size_t nbytes, int count, void* stream);

/*
 * Synchronise the current device and report whether any kernel of this library flagged a
 * bounded wait that ran out or a block list entry outside the key grid since the last call
 * (LCBSA_EDEVICE), clearing the flag.
 * Debug aid for tests; not part of the hot path.
 */
int lcbsa_check_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* LCBSA_H_ */
