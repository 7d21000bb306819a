// Shared host/device helpers for the lcbsa kernels (internal header).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lcbsa.h"

namespace lcbsa {

// Strided view of one [B,H,S,D] operand as the kernels see it (element strides, D contiguous).
struct View {
    const void* data;
    int64_t sb, sh, ss;  // batch, head, token strides in elements
};

// Block geometry of a latent grid, precomputed on the host.
struct Geom {
    int T, H, W;     // grid
    int ct, ch, cw;  // block shape
    int Nt, Nh, Nw;  // blocks per axis (ceil)
    int nblk;        // Nt*Nh*Nw
    int bs;          // ct*ch*cw
    int ragged;      // 1 when some axis does not divide
};

inline Geom make_geom(const LcbsaGrid& g) {
    Geom r;
    r.T = g.T; r.H = g.H; r.W = g.W;
    r.ct = g.ct; r.ch = g.ch; r.cw = g.cw;
    r.Nt = (g.T + g.ct - 1) / g.ct;
    r.Nh = (g.H + g.ch - 1) / g.ch;
    r.Nw = (g.W + g.cw - 1) / g.cw;
    r.nblk = r.Nt * r.Nh * r.Nw;
    r.bs = g.ct * g.ch * g.cw;
    r.ragged = (g.T % g.ct != 0) || (g.H % g.ch != 0) || (g.W % g.cw != 0);
    return r;
}

template <typename T> struct DType;
template <> struct DType<__nv_bfloat16> {
    static constexpr int code = LCBSA_BF16;
    __device__ static __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct DType<__half> {
    static constexpr int code = LCBSA_FP16;
    __device__ static __forceinline__ float to_f32(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct DType<float> {
    static constexpr int code = LCBSA_FP32;
    __device__ static __forceinline__ float to_f32(float v) { return v; }
    __device__ static __forceinline__ float from_f32(float v) { return v; }
};

// Slot r of a block -> (lt, lh, lw) and the token offset relative to the block's first token.
__device__ __forceinline__ void slot_coords(const Geom& g, int r, int& lt, int& lh, int& lw) {
    lw = r % g.cw;
    int q = r / g.cw;
    lh = q % g.ch;
    lt = q / g.ch;
}

__device__ __forceinline__ void block_coords(const Geom& g, int blk, int& bt, int& bh, int& bw) {
    bw = blk % g.Nw;
    int q = blk / g.Nw;
    bh = q % g.Nh;
    bt = q / g.Nh;
}

// Device status word [0]: 1 = shared memory base not 1024-byte aligned, 2 = a block list entry outside [0, Nk)
// (words 1..3: batch*head, query block, list position), >= 10 = a bounded wait ran out (words 1..3: CTA, thread, iteration).
constexpr unsigned kStatusBadBlockIndex = 2u;

// Message returned by lcbsa_last_error() for the calling thread (api.cu owns the buffer).
void set_last_error(const char* msg);

// Launchers implemented in the .cu files (host side). All return a cudaError_t from the launch.
cudaError_t launch_pool(int dtype, const View& x, int B, int H, int D, const Geom& g, void* out, cudaStream_t st);
// One launch that pools one or two tensors (x1 may be null).  Each has its destination: dense rows at dst[0], or rows
// scattered by head over up to kPoolMaxDst buffers (see pool.cu).
constexpr int kPoolMaxDst = 8;
struct PoolDst {
    void* dst[kPoolMaxDst];
    int n_dst;          // 0: dense [B*H, nblk, D] at dst[0]
    int heads_per_dst;  // scatter: heads per destination buffer
    int src_rank;       // scatter: which source slot of the destination layout this call fills
};
cudaError_t launch_pool2(int dtype, const View& x0, const Geom& g0, const PoolDst& d0, const View* x1, const Geom* g1, const PoolDst* d1,
                         int B, int H, int D, cudaStream_t st);

// two-kernel form of the same stage (select_gemm.cu): bytes of key workspace it needs (0: does not apply) and launch
size_t score_keys_bytes(int dtype, int BH, int Nq, int Nk, int D);
// A grid with a "first part" (conditioning frames): blocks are numbered frame-major and a block is in the first part when
// ((block / hw) % period) < split, hw = blocks per frame-block plane.  Query blocks of the first part select nsel_first
// key blocks among the key blocks of the first part; the others select among all key blocks.
struct SelectSplit {
    int hw_q, period_q, split_q;
    int hw_k, period_k, split_k;
    int nsel_first;
};
cudaError_t launch_score_gemm_topk(int dtype, const void* qc, const void* kc, int BH, int Nq, int Nk, int D, int nsel, int cap,
                                   int32_t* idx, int32_t* cnt, void* keys_ws, cudaStream_t st, const char** why,
                                   const SelectSplit* split = nullptr);
cudaError_t launch_score_topk(int dtype, const void* qc, const void* kc, int BH, int Nq, int Nk, int D, int nsel,
                              int cap, int32_t* idx, int32_t* cnt, cudaStream_t st, const char** why);

struct AttnArgs {
    int dtype;
    View q, k, v, o;
    int B, H, D;
    Geom gq, gk;
    const int32_t* idx;
    const int32_t* cnt;
    int cap;
    float sm_scale;
    float* lse;  // nullable, [B*H, Sq]
    unsigned int* status;  // device status words
    // Scattered output (tcgen05 kernel only): with n_out_dst > 0 the query grid is rank-major over n_out_dst ranks
    // (frames split evenly) and the rows of rank r's frames go to out_dst[r], a [1, H, Sq / n, D] tensor with the
    // head and token strides of `o` (o.data is then unused).
    int n_out_dst = 0;
    void* out_dst[8] = {};
};

cudaError_t launch_attn_mma(const AttnArgs& a, cudaStream_t st, const char** why);
cudaError_t launch_attn_tc(const AttnArgs& a, cudaStream_t st, const char** why);
bool attn_tc_supported(const AttnArgs& a, const char** why);
// Backward (attn_bwd.cu): dq, dk, dv for fixed block lists.
struct BwdArgs {
    int dtype, D;
    View q, k, v, o, dout, dq, dk, dv;
    int B, H;
    Geom gq, gk;
    const int32_t* idx;   // [B*H, Nq, cap]
    const int32_t* cnt;   // [B*H, Nq]
    int cap;
    float sm_scale;
    const float* lse;     // [B*H, Sq] natural log, from the forward
    unsigned int* status;
    // carved out of the workspace by launch_attn_bwd:
    float* delta;         // [B*H, Sq]
    int32_t* tcnt;        // [B*H, Nk]       query blocks per key block
    int32_t* toff;        // [B*H, Nk + 1]   exclusive prefix of tcnt
    int32_t* tidx;        // [B*H, Nq * cap] query blocks of key block j at toff[j] .. toff[j + 1], ascending
    uint32_t* bitmap;     // [B*H, Nk, ceil(Nq / 32)] bit i of row j: query block i selected key block j
    float* stats;         // [B*H, Sq * 2] per 64-token query block: lse * log2(e) [64], delta [64] (tcgen05 passes)
    int32_t* idx_u;       // [B*H, Nq_u, cap * Uk] rewritten lists of the dQ pass (tcgen05 passes, blocks split into units)
    int32_t* cnt_u;       // [B*H, Nq_u]
    int32_t* idx_t;       // the same for the lists that are transposed for the dK/dV pass
    int32_t* cnt_t;
};
bool attn_bwd_supported(const BwdArgs& a, const char** why);
size_t attn_bwd_workspace_bytes(long long BH, const Geom& gq, const Geom& gk, int cap);
cudaError_t launch_attn_bwd(BwdArgs a, void* workspace, cudaStream_t st, const char** why);
// the dQ and dK/dV passes on tcgen05 (attn_bwd_tc.cu): head_dim 128.  A CTA owns a block of 64 or 128
// tokens and streams 64-token units; the plan names the grids and the lists in those terms.
struct BwdTcPlan {
    Geom own_q, own_k;        // blocks of the CTAs of the dQ pass and of the dK/dV pass (64 or 128 tokens)
    Geom unit_q, unit_k;      // the 64-token grids of the streamed tiles (query units in the dK/dV pass, key units in the dQ pass)
    const int32_t* list_q;    // [B*H, own_q.nblk, cap_q] key units of every own query block
    const int32_t* cnt_q;     // [B*H, own_q.nblk]
    int cap_q;
    const int32_t* toff;      // [B*H, own_k.nblk + 1]
    const int32_t* tidx;      // [B*H, tidx_stride] query units of own key block j at toff[j] .. toff[j + 1]
    long long tidx_stride;
};
bool attn_bwd_tc_supported(const BwdArgs& a, const BwdTcPlan& p);
cudaError_t launch_attn_bwd_tc(const BwdArgs& a, const BwdTcPlan& p, cudaStream_t st, const char** why);

// the same for 128-token query and key blocks (attn_tc128.cu)
cudaError_t launch_attn_tc128(const AttnArgs& a, cudaStream_t st, const char** why);
bool attn_tc128_supported(const AttnArgs& a, const char** why);
cudaError_t launch_score_keys(int dtype, const void* qc, const void* kc, int BH, int Nq, int Nk, int D, void* keys_ws, cudaStream_t st,
                              const char** why);
// cdf_threshold selectors on the keys of launch_score_keys (select_cdf.cu): idx [rows, Nk] sorted by descending weight, cnt [rows]
cudaError_t launch_cdf_rows(int dtype, const void* keys, long long rows, int Nk, float sm_scale, float threshold, int nsel_min,
                            int32_t* idx, int32_t* cnt, cudaStream_t st, const char** why);
int set_attn_sm_reserve(int n_sms);  // SMs the tcgen05 attention kernel leaves idle; returns the previous value

// q/k RMSNorm + 3-D rotary embedding in one pass (norm_rope.cu).  The table is the packed separable form
// cos_t [T, dt] sin_t [T, dt] cos_h [H, dh] sin_h [H, dh] cos_w [W, dh] sin_w [W, dh], dh = 2 * (D / 6), dt = D - 2 * dh.
size_t rope_table_floats(int Tg, int Hg, int Wg, int D);
cudaError_t launch_norm_rope(int dtype, const View& x, int B, int H, int S, int D, int tab_t, int t_off, int Hg, int Wg, const void* weight,
                             const float* tab, float eps, void* out, long long osb, long long osh, long long oss, cudaStream_t st,
                             const char** why);

}  // namespace lcbsa
