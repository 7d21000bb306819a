// Block-sparse attention backward for sm_100a: dq, dk, dv for fixed block lists.
//
// Stands in for attn_bwd_bsa_varlen_triton and its Triton kernels (longcat_video/block_sparse_attention/
// bsa_interface.py:343-461, flash_attn_bsa_varlen_mask.py:289-945; the autograd contract is _attention_bsa.backward,
// bsa_interface.py:570-596): the block lists are constants of the backward (no gradient flows through the selection),
// q, k, v, o, do are [B, H, S, D] tensors in T,H,W token order and the 3-D blocks are addressed in place.
//
// Per (query block i, selected key block j), with scale = sm_scale and lse the forward's row log-sum-exp:
//   S = Q_i K_j^T * scale          P = exp(S - lse_i)              dV_j += P^T dO_i
//   dP = dO_i V_j^T                dS = P o (dP - delta_i) * scale  dQ_i += dS K_j        dK_j += dS^T Q_i
//   delta_i = rowsum(dO_i o O_i)
//
// No atomics on the gradients, every sum in a fixed order:
//   bwd_delta_kernel      delta for every query row (fp32), one pass over dO and O;
//   bwd_mark / count / scan / emit   for every key block the query blocks that selected it, in ascending order (the
//                         lists hold for every query block its key blocks), through a bitmap: four small launches;
//   bwd_dq_mma_kernel     one CTA per 64 query rows, walks the forward lists;
//   bwd_dkdv_mma_kernel   one CTA per 64 keys, walks the transposed lists.
// Tiles are 64 x 64 whatever the block sizes (multiples of 64 tokens): a block of 128 or more tokens is a run of
// 64-row tiles in slot order.  The contractions run on the tensor cores through warp-level mma (mma.sync m16n8k16 fed by
// ldmatrix, fp32 accumulation); P and dS are rounded to the input dtype before they enter a contraction, as in the
// forward.  The two passes of this file serve every supported shape; head_dim 128 is taken by the tcgen05 passes of
// attn_bwd_tc.cu instead (same delta kernel, same transposition; blocks above 64 tokens as 64-token units), except for
// ragged grids in fp16 or with blocks above 64 tokens.
#include "mma_common.cuh"

namespace lcbsa {

namespace {

constexpr int kTile = 64;      // rows and keys per tile
constexpr int kBwdThreads = 128;

// ------------------------------------------------------------------------------------------ delta

template <typename T, int D>
__global__ void __launch_bounds__(256) bwd_delta_kernel(View o, View dout, float* delta, int H, long long Sq, long long rows) {
    // eight lanes per row: a lane reads D/8 consecutive elements of o and do
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long row = gid >> 3;
    const int part = (int)(gid & 7);
    float acc = 0.f;
    if (row < rows) {
        const long long bh = row / Sq, s = row % Sq;
        const long long b = bh / H, h = bh % H;
        const T* po = reinterpret_cast<const T*>(o.data) + b * o.sb + h * o.sh + s * o.ss + part * (D / 8);
        const T* pd = reinterpret_cast<const T*>(dout.data) + b * dout.sb + h * dout.sh + s * dout.ss + part * (D / 8);
#pragma unroll
        for (int c = 0; c < D / 8; c += 8) {
            const uint4 a = *reinterpret_cast<const uint4*>(po + c), d = *reinterpret_cast<const uint4*>(pd + c);
            const T* a8 = reinterpret_cast<const T*>(&a);
            const T* d8 = reinterpret_cast<const T*>(&d);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc = fmaf(DType<T>::to_f32(a8[e]), DType<T>::to_f32(d8[e]), acc);
        }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (row < rows && part == 0) delta[row] = acc;
}

// ------------------------------------------------------------------------------------------ transposed lists

// The lists hold for every query block its key blocks; the dK/dV pass needs for every key block its query blocks, in a
// fixed order.  Four small launches: mark (one bit per (key block, query block) pair in a zeroed bitmap), count (a warp
// per key block adds up the population counts of its bitmap row), scan (exclusive prefix of the counts per head) and emit
// (a warp per key block turns its bitmap row into the ascending list of its query blocks).  Entries outside [0, Nk) are
// skipped and flagged; the entries of one list are taken as distinct.
__global__ void __launch_bounds__(256) bwd_mark_kernel(const int32_t* idx, const int32_t* cnt, int cap, int Nq, int Nk, int Wq, long long total,
                                                       uint32_t* bitmap, unsigned int* status) {
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= total) return;
    const int e = (int)(p % cap);
    const long long row = p / cap;  // bh * Nq + i
    const int i = (int)(row % Nq);
    const long long bh = row / Nq;
    if (e >= min(max(cnt[row], 0), cap)) return;
    const int j = idx[p];
    if ((unsigned)j < (unsigned)Nk) atomicOr(&bitmap[(bh * Nk + j) * Wq + (i >> 5)], 1u << (i & 31));
    else if (atomicCAS(status, 0u, kStatusBadBlockIndex) == 0u) {
        status[1] = (unsigned)bh;
        status[2] = i;
        status[3] = e;
    }
}

__global__ void __launch_bounds__(256) bwd_count_kernel(const uint32_t* bitmap, int Wq, long long rows, int32_t* tcnt) {
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // bh * Nk + j
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    int n = 0;
    for (int w = lane; w < Wq; w += 32) n += __popc(bitmap[row * Wq + w]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    if (lane == 0) tcnt[row] = n;
}

// one CTA per (batch, head): toff[j] = sum of tcnt[0 .. j), toff[Nk] = the total
__global__ void __launch_bounds__(256) bwd_scan_kernel(const int32_t* tcnt, int Nk, int32_t* toff) {
    __shared__ int part[256];
    const int bh = blockIdx.x, tid = threadIdx.x;
    const int32_t* c = tcnt + (long long)bh * Nk;
    int32_t* o = toff + (long long)bh * (Nk + 1);
    const int per = (Nk + 255) / 256, lo = tid * per, hi = min(lo + per, Nk);
    int sum = 0;
    for (int j = lo; j < hi; ++j) sum += c[j];
    part[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int t = 0; t < 256; ++t) {
            const int v = part[t];
            part[t] = run;
            run += v;
        }
        o[Nk] = run;
    }
    __syncthreads();
    int run = part[tid];
    for (int j = lo; j < hi; ++j) {
        o[j] = run;
        run += c[j];
    }
}

__global__ void __launch_bounds__(256) bwd_emit_kernel(const uint32_t* bitmap, int Wq, int Nk, int Nq, int cap, long long rows, const int32_t* toff,
                                                       int32_t* tidx) {
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // bh * Nk + j
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const long long bh = row / Nk;
    const int j = (int)(row % Nk);
    int32_t* out = tidx + bh * Nq * cap;
    int base = toff[bh * (Nk + 1) + j];
    for (int w0 = 0; w0 < Wq; w0 += 32) {
        const int w = w0 + lane;
        uint32_t bits = w < Wq ? bitmap[row * Wq + w] : 0u;
        const int n = __popc(bits);
        int incl = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        int pos = base + incl - n;
        while (bits) {
            const int b = __ffs(bits) - 1;
            out[pos++] = 32 * w + b;
            bits &= bits - 1;
        }
        base += __shfl_sync(0xffffffffu, incl, 31);
    }
}

// ------------------------------------------------------------------------------------------ dQ and dK/dV
//
// Both passes run on mma.sync m16n8k16 with ldmatrix from 128-byte-row swizzled tiles (the machinery of the generic
// forward, attn_mma.cu).  S, dP, P and dS never leave registers: the accumulator layout of one contraction is
// the A-operand layout of the next (as P is for P V in the forward).  64 x 64 tiles, four warps of 16 rows, the
// streamed tiles double-buffered with cp.async, two CTAs per SM.

// 16 rows x 64 columns (fp32 accumulators, 8 n-tiles) = A[16 x D] * B[64 x D]^T with A already in registers
template <typename T, int D>
__device__ __forceinline__ void mma_abt(float (&acc)[8][4], const uint32_t (&af)[D / 16][4], uint32_t b_tile, int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            const int mid = lane >> 3;
            const int row = np * 16 + (lane & 7) + (mid >> 1) * 8;
            const int c = 2 * ks + (mid & 1);
            uint32_t bf[4];
            mm::ldsm_x4(bf, b_tile + row * (D * 2) + ((c ^ (row & 7)) << 4));
            mm::mma16816<T>(acc[2 * np], af[ks], bf[0], bf[1]);
            mm::mma16816<T>(acc[2 * np + 1], af[ks], bf[2], bf[3]);
        }
    }
}

// Two such products at once (S and dP of the same tile pair): two independent accumulation chains in one instruction
// stream, which is what hides the ldmatrix -> mma latency with only two warps per scheduler.
template <typename T, int D>
__device__ __forceinline__ void mma_abt2(float (&acc0)[8][4], float (&acc1)[8][4], const uint32_t (&a0)[D / 16][4],
                                         const uint32_t (&a1)[D / 16][4], uint32_t b0_tile, uint32_t b1_tile, int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        acc0[i][0] = acc0[i][1] = acc0[i][2] = acc0[i][3] = 0.f;
        acc1[i][0] = acc1[i][1] = acc1[i][2] = acc1[i][3] = 0.f;
    }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            const int mid = lane >> 3;
            const int row = np * 16 + (lane & 7) + (mid >> 1) * 8;
            const int c = 2 * ks + (mid & 1);
            const uint32_t off = row * (D * 2) + ((c ^ (row & 7)) << 4);
            uint32_t bf0[4], bf1[4];
            mm::ldsm_x4(bf0, b0_tile + off);
            mm::ldsm_x4(bf1, b1_tile + off);
            mm::mma16816<T>(acc0[2 * np], a0[ks], bf0[0], bf0[1]);
            mm::mma16816<T>(acc1[2 * np], a1[ks], bf1[0], bf1[1]);
            mm::mma16816<T>(acc0[2 * np + 1], a0[ks], bf0[2], bf0[3]);
            mm::mma16816<T>(acc1[2 * np + 1], a1[ks], bf1[2], bf1[3]);
        }
    }
}

// The same with the A operands read from shared tiles step by step (this warp's 16 rows of a0_tile and a1_tile)
template <typename T, int D>
__device__ __forceinline__ void mma_abt2_sa(float (&acc0)[8][4], float (&acc1)[8][4], uint32_t a0_tile, uint32_t a1_tile, uint32_t b0_tile,
                                            uint32_t b1_tile, int warp, int lane) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        acc0[i][0] = acc0[i][1] = acc0[i][2] = acc0[i][3] = 0.f;
        acc1[i][0] = acc1[i][1] = acc1[i][2] = acc1[i][3] = 0.f;
    }
    const int arow = warp * 16 + (lane & 15);
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a0[4], a1[4];
        {
            const int c = 2 * ks + (lane >> 4);
            const uint32_t off = arow * (D * 2) + ((c ^ (arow & 7)) << 4);
            mm::ldsm_x4(a0, a0_tile + off);
            mm::ldsm_x4(a1, a1_tile + off);
        }
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            const int mid = lane >> 3;
            const int row = np * 16 + (lane & 7) + (mid >> 1) * 8;
            const int c = 2 * ks + (mid & 1);
            const uint32_t off = row * (D * 2) + ((c ^ (row & 7)) << 4);
            uint32_t bf0[4], bf1[4];
            mm::ldsm_x4(bf0, b0_tile + off);
            mm::ldsm_x4(bf1, b1_tile + off);
            mm::mma16816<T>(acc0[2 * np], a0, bf0[0], bf0[1]);
            mm::mma16816<T>(acc1[2 * np], a1, bf1[0], bf1[1]);
            mm::mma16816<T>(acc0[2 * np + 1], a0, bf0[2], bf0[3]);
            mm::mma16816<T>(acc1[2 * np + 1], a1, bf1[2], bf1[3]);
        }
    }
}

// A fragments (16 rows of this warp, all of D) of a swizzled [64][D] tile
template <int D>
__device__ __forceinline__ void load_a_frags(uint32_t (&af)[D / 16][4], uint32_t tile, int warp, int lane) {
    const int row = warp * 16 + (lane & 15);
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int c = 2 * ks + (lane >> 4);
        mm::ldsm_x4(af[ks], tile + row * (D * 2) + ((c ^ (row & 7)) << 4));
    }
}

// out[16 x D] += X[16 x 64] * B[64 x D], X given as fp32 accumulators of the layout mma_abt produces (rounded to T here)
template <typename T, int D>
__device__ __forceinline__ void mma_xb(float (&out)[D / 8][4], const float (&x)[8][4], uint32_t b_tile, int lane) {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        uint32_t pa[4];
        pa[0] = mm::pack2(T(), x[2 * kk][0], x[2 * kk][1]);
        pa[1] = mm::pack2(T(), x[2 * kk][2], x[2 * kk][3]);
        pa[2] = mm::pack2(T(), x[2 * kk + 1][0], x[2 * kk + 1][1]);
        pa[3] = mm::pack2(T(), x[2 * kk + 1][2], x[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            const int mid = lane >> 3;
            const int row = kk * 16 + (lane & 7) + (mid & 1) * 8;
            const int c = 2 * dp + (mid >> 1);
            uint32_t bf[4];
            mm::ldsm_x4_t(bf, b_tile + row * (D * 2) + ((c ^ (row & 7)) << 4));
            mm::mma16816<T>(out[2 * dp], pa, bf[0], bf[1]);
            mm::mma16816<T>(out[2 * dp + 1], pa, bf[2], bf[3]);
        }
    }
}

// Two of those at once: out0 += X0 * B0 and out1 += X1 * B1 (dV and dK of one tile pair)
template <typename T, int D>
__device__ __forceinline__ void mma_xb2(float (&out0)[D / 8][4], const float (&x0)[8][4], uint32_t b0_tile, float (&out1)[D / 8][4],
                                        const float (&x1)[8][4], uint32_t b1_tile, int lane) {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        uint32_t pa0[4], pa1[4];
        pa0[0] = mm::pack2(T(), x0[2 * kk][0], x0[2 * kk][1]);
        pa0[1] = mm::pack2(T(), x0[2 * kk][2], x0[2 * kk][3]);
        pa0[2] = mm::pack2(T(), x0[2 * kk + 1][0], x0[2 * kk + 1][1]);
        pa0[3] = mm::pack2(T(), x0[2 * kk + 1][2], x0[2 * kk + 1][3]);
        pa1[0] = mm::pack2(T(), x1[2 * kk][0], x1[2 * kk][1]);
        pa1[1] = mm::pack2(T(), x1[2 * kk][2], x1[2 * kk][3]);
        pa1[2] = mm::pack2(T(), x1[2 * kk + 1][0], x1[2 * kk + 1][1]);
        pa1[3] = mm::pack2(T(), x1[2 * kk + 1][2], x1[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            const int mid = lane >> 3;
            const int row = kk * 16 + (lane & 7) + (mid & 1) * 8;
            const int c = 2 * dp + (mid >> 1);
            const uint32_t off = row * (D * 2) + ((c ^ (row & 7)) << 4);
            uint32_t bf0[4], bf1[4];
            mm::ldsm_x4_t(bf0, b0_tile + off);
            mm::ldsm_x4_t(bf1, b1_tile + off);
            mm::mma16816<T>(out0[2 * dp], pa0, bf0[0], bf0[1]);
            mm::mma16816<T>(out1[2 * dp], pa1, bf1[0], bf1[1]);
            mm::mma16816<T>(out0[2 * dp + 1], pa0, bf0[2], bf0[3]);
            mm::mma16816<T>(out1[2 * dp + 1], pa1, bf1[2], bf1[3]);
        }
    }
}

// fp32 accumulators of this warp's 16 rows (all of D) -> a swizzled [64][D] tile in T
template <typename T, int D>
__device__ __forceinline__ void stage_rows(unsigned char* tile, const float (&o)[D / 8][4], int warp, int lane) {
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        const int col = i * 8 + 2 * (lane & 3);
        const int c = col >> 3, within = (col & 7) * 2;
        *reinterpret_cast<uint32_t*>(tile + r0 * (D * 2) + ((c ^ (r0 & 7)) << 4) + within) = mm::pack2(T(), o[i][0], o[i][1]);
        *reinterpret_cast<uint32_t*>(tile + r1 * (D * 2) + ((c ^ (r1 & 7)) << 4) + within) = mm::pack2(T(), o[i][2], o[i][3]);
    }
}

// rows of a swizzled [64][D] tile -> the rows of the block that exist
template <typename T, int D>
__device__ __forceinline__ void write_rows(const unsigned char* tile, T* head, long long ss, const Geom& g, const mm::SlotEntry* tab, int blk,
                                           int slot0, int tid) {
    constexpr int CPR = D * 2 / 16;
    int bt, bh, bw;
    block_coords(g, blk, bt, bh, bw);
    const int t0 = bt * g.ct, h0 = bh * g.ch, w0 = bw * g.cw;
    const long long origin = ((long long)t0 * g.H + h0) * g.W + w0;
    for (int v = tid; v < kTile * CPR; v += kBwdThreads) {
        const int row = v / CPR, c = v % CPR;
        const mm::SlotEntry e = tab[slot0 + row];
        if (g.ragged && !mm::slot_present(g, e.packed, t0, h0, w0)) continue;
        *reinterpret_cast<uint4*>(head + (origin + e.off) * ss + c * 8) =
            *reinterpret_cast<const uint4*>(tile + row * (D * 2) + ((c ^ (row & 7)) << 4));
    }
}

// lse (scaled to log2), delta and presence of 64 rows of a query block -> shared arrays
__device__ __forceinline__ void load_q_scalars(float* lse2, float* delta, unsigned char* ok, const float* lse_head, const float* delta_head,
                                               const Geom& g, const mm::SlotEntry* tab, int blk, int slot0, int tid) {
    int bt, bh, bw;
    block_coords(g, blk, bt, bh, bw);
    const int t0 = bt * g.ct, h0 = bh * g.ch, w0 = bw * g.cw;
    const long long origin = ((long long)t0 * g.H + h0) * g.W + w0;
    for (int r = tid; r < kTile; r += kBwdThreads) {
        const mm::SlotEntry e = tab[slot0 + r];
        const bool p = !g.ragged || mm::slot_present(g, e.packed, t0, h0, w0);
        lse2[r] = p ? lse_head[origin + e.off] * 1.4426950408889634f : 0.f;
        delta[r] = p ? delta_head[origin + e.off] : 0.f;
        ok[r] = p ? 1 : 0;
    }
}

__device__ __forceinline__ void fill_slots(mm::SlotEntry* tab, const Geom& g, int tid) {
    for (int r = tid; r < g.bs; r += kBwdThreads) {
        int lt, lh, lw;
        slot_coords(g, r, lt, lh, lw);
        tab[r] = mm::SlotEntry{(lt * g.H + lh) * g.W + lw, lt | (lh << 10) | (lw << 20)};
    }
}

template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads, 2) bwd_dq_mma_kernel(const __grid_constant__ BwdArgs a) {
    constexpr int kTB = kTile * D * 2;  // bytes of a tile
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                 // Q rows, later the staged dQ
    unsigned char* do_s = q_s + kTB;
    unsigned char* k_s = do_s + kTB;           // [2]
    unsigned char* v_s = k_s + 2 * kTB;        // [2]
    unsigned char* k_ok = v_s + 2 * kTB;       // [2][64] presence of the keys of a tile
    mm::SlotEntry* qtab = reinterpret_cast<mm::SlotEntry*>(k_ok + 2 * kTile);
    mm::SlotEntry* ktab = qtab + a.gq.bs;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tiles_q = a.gq.bs / kTile, tiles_k = a.gk.bs / kTile;
    const int qb = blockIdx.x / tiles_q, qsub = blockIdx.x % tiles_q;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    fill_slots(qtab, a.gq, tid);
    fill_slots(ktab, a.gk, tid);
    __syncthreads();

    const long long Sq = (long long)a.gq.T * a.gq.H * a.gq.W;
    const T* qh = reinterpret_cast<const T*>(a.q.data) + (long long)b * a.q.sb + (long long)h * a.q.sh;
    const T* kh = reinterpret_cast<const T*>(a.k.data) + (long long)b * a.k.sb + (long long)h * a.k.sh;
    const T* vh = reinterpret_cast<const T*>(a.v.data) + (long long)b * a.v.sb + (long long)h * a.v.sh;
    const T* doh = reinterpret_cast<const T*>(a.dout.data) + (long long)b * a.dout.sb + (long long)h * a.dout.sh;
    T* dqh = reinterpret_cast<T*>(const_cast<void*>(a.dq.data)) + (long long)b * a.dq.sb + (long long)h * a.dq.sh;

    const int32_t* list = a.idx + ((long long)bh * a.gq.nblk + qb) * a.cap;
    const int n_list = min(max(a.cnt[(long long)bh * a.gq.nblk + qb], 0), a.cap);
    const int n_tiles = n_list * tiles_k;

    // presence of the keys of a tile (all absent for a list entry outside [0, Nk), which the mark kernel has flagged)
    auto key_flags = [&](unsigned char* dst, int blk, int slot0) {
        const bool blk_ok = (unsigned)blk < (unsigned)a.gk.nblk;
        int bt, bhh, bw;
        block_coords(a.gk, blk_ok ? blk : 0, bt, bhh, bw);
        const int t0 = bt * a.gk.ct, h0 = bhh * a.gk.ch, w0 = bw * a.gk.cw;
        for (int r = tid; r < kTile; r += kBwdThreads)
            dst[r] = (blk_ok && (!a.gk.ragged || mm::slot_present(a.gk, ktab[slot0 + r].packed, t0, h0, w0))) ? 1 : 0;
    };

    mm::load_tile<T, D, kTile, kBwdThreads>(q_s, qh, a.q.ss, a.gq, qtab, qb, qsub * kTile, tid);
    mm::load_tile<T, D, kTile, kBwdThreads>(do_s, doh, a.dout.ss, a.gq, qtab, qb, qsub * kTile, tid);
    mm::cp_async_commit();
    if (n_tiles > 0) {
        mm::load_tile<T, D, kTile, kBwdThreads>(k_s, kh, a.k.ss, a.gk, ktab, list[0], 0, tid);
        mm::load_tile<T, D, kTile, kBwdThreads>(v_s, vh, a.v.ss, a.gk, ktab, list[0], 0, tid);
        key_flags(k_ok, list[0], 0);
    }
    mm::cp_async_commit();
    mm::cp_async_wait<1>();
    __syncthreads();

    uint32_t qf[D / 16][4], dof[D / 16][4];
    load_a_frags<D>(qf, mm::smem_u32(q_s), warp, lane);
    load_a_frags<D>(dof, mm::smem_u32(do_s), warp, lane);

    // per-row constants of this thread's two rows
    float lse2[2], dl[2];
    bool rok[2];
    {
        int bt, bhh, bw;
        block_coords(a.gq, qb, bt, bhh, bw);
        const int t0 = bt * a.gq.ct, h0 = bhh * a.gq.ch, w0 = bw * a.gq.cw;
        const long long origin = ((long long)t0 * a.gq.H + h0) * a.gq.W + w0;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const mm::SlotEntry se = qtab[qsub * kTile + warp * 16 + (lane >> 2) + 8 * e];
            rok[e] = !a.gq.ragged || mm::slot_present(a.gq, se.packed, t0, h0, w0);
            lse2[e] = rok[e] ? a.lse[(long long)bh * Sq + origin + se.off] * 1.4426950408889634f : 0.f;
            dl[e] = rok[e] ? a.delta[(long long)bh * Sq + origin + se.off] : 0.f;
        }
    }
    const float scale2 = a.sm_scale * 1.4426950408889634f;

    float dq[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;

    for (int it = 0; it < n_tiles; ++it) {
        const int buf = it & 1;
        if (it + 1 < n_tiles) {
            const int nblk = list[(it + 1) / tiles_k], nsub = (it + 1) % tiles_k;
            mm::load_tile<T, D, kTile, kBwdThreads>(k_s + (buf ^ 1) * kTB, kh, a.k.ss, a.gk, ktab, nblk, nsub * kTile, tid);
            mm::load_tile<T, D, kTile, kBwdThreads>(v_s + (buf ^ 1) * kTB, vh, a.v.ss, a.gk, ktab, nblk, nsub * kTile, tid);
            key_flags(k_ok + (buf ^ 1) * kTile, nblk, nsub * kTile);
        }
        mm::cp_async_commit();
        mm::cp_async_wait<1>();
        __syncthreads();
        const uint32_t kt = mm::smem_u32(k_s) + buf * kTB, vt = mm::smem_u32(v_s) + buf * kTB;
        const unsigned char* kok = k_ok + buf * kTile;

        float s[8][4], dp[8][4];
        mma_abt2<T, D>(s, dp, qf, dof, kt, vt, lane);
        // dS in place of dP: ds = p * (dp - delta) * scale, p = 2^(s * scale2 - lse2); absent keys and rows give 0
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int col = nt * 8 + 2 * (lane & 3) + (e & 1), r = e >> 1;
                const bool ok = rok[r] && kok[col];
                const float p = ok ? mm::ex2(fmaf(s[nt][e], scale2, -lse2[r])) : 0.f;
                dp[nt][e] = p * (dp[nt][e] - dl[r]) * a.sm_scale;
            }
        }
        mma_xb<T, D>(dq, dp, kt, lane);  // dQ += dS K
        __syncthreads();
    }
    mm::cp_async_wait<0>();
    __syncthreads();
    stage_rows<T, D>(q_s, dq, warp, lane);
    __syncthreads();
    write_rows<T, D>(q_s, dqh, a.dq.ss, a.gq, qtab, qb, qsub * kTile, tid);
}

template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads, 2) bwd_dkdv_mma_kernel(const __grid_constant__ BwdArgs a) {
    constexpr int kTB = kTile * D * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* k_s = smem;                 // K rows of this tile, later the staged dK
    unsigned char* v_s = k_s + kTB;            // V rows, later the staged dV
    unsigned char* q_s = v_s + kTB;            // [2]
    unsigned char* do_s = q_s + 2 * kTB;       // [2]
    float* lse2 = reinterpret_cast<float*>(do_s + 2 * kTB);  // [2][64]
    float* delta = lse2 + 2 * kTile;                         // [2][64]
    unsigned char* q_ok = reinterpret_cast<unsigned char*>(delta + 2 * kTile);  // [2][64]
    mm::SlotEntry* qtab = reinterpret_cast<mm::SlotEntry*>(q_ok + 2 * kTile);
    mm::SlotEntry* ktab = qtab + a.gq.bs;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tiles_q = a.gq.bs / kTile, tiles_k = a.gk.bs / kTile;
    const int kb = blockIdx.x / tiles_k, ksub = blockIdx.x % tiles_k;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    fill_slots(qtab, a.gq, tid);
    fill_slots(ktab, a.gk, tid);
    __syncthreads();

    const long long Sq = (long long)a.gq.T * a.gq.H * a.gq.W;
    const T* qh = reinterpret_cast<const T*>(a.q.data) + (long long)b * a.q.sb + (long long)h * a.q.sh;
    const T* kh = reinterpret_cast<const T*>(a.k.data) + (long long)b * a.k.sb + (long long)h * a.k.sh;
    const T* vh = reinterpret_cast<const T*>(a.v.data) + (long long)b * a.v.sb + (long long)h * a.v.sh;
    const T* doh = reinterpret_cast<const T*>(a.dout.data) + (long long)b * a.dout.sb + (long long)h * a.dout.sh;
    T* dkh = reinterpret_cast<T*>(const_cast<void*>(a.dk.data)) + (long long)b * a.dk.sb + (long long)h * a.dk.sh;
    T* dvh = reinterpret_cast<T*>(const_cast<void*>(a.dv.data)) + (long long)b * a.dv.sb + (long long)h * a.dv.sh;
    const float* lse_h = a.lse + (long long)bh * Sq;
    const float* delta_h = a.delta + (long long)bh * Sq;

    const int32_t* tl = a.tidx + (long long)bh * a.gq.nblk * a.cap;
    const int t_lo = a.toff[(long long)bh * (a.gk.nblk + 1) + kb], t_hi = a.toff[(long long)bh * (a.gk.nblk + 1) + kb + 1];
    const int n_tiles = (t_hi - t_lo) * tiles_q;

    mm::load_tile<T, D, kTile, kBwdThreads>(k_s, kh, a.k.ss, a.gk, ktab, kb, ksub * kTile, tid);
    mm::load_tile<T, D, kTile, kBwdThreads>(v_s, vh, a.v.ss, a.gk, ktab, kb, ksub * kTile, tid);
    mm::cp_async_commit();
    if (n_tiles > 0) {
        const int qb0 = tl[t_lo];
        mm::load_tile<T, D, kTile, kBwdThreads>(q_s, qh, a.q.ss, a.gq, qtab, qb0, 0, tid);
        mm::load_tile<T, D, kTile, kBwdThreads>(do_s, doh, a.dout.ss, a.gq, qtab, qb0, 0, tid);
        load_q_scalars(lse2, delta, q_ok, lse_h, delta_h, a.gq, qtab, qb0, 0, tid);
    }
    mm::cp_async_commit();
    mm::cp_async_wait<1>();
    __syncthreads();

    // presence of this thread's two key rows
    bool kok[2];
    {
        int bt, bhh, bw;
        block_coords(a.gk, kb, bt, bhh, bw);
        const int t0 = bt * a.gk.ct, h0 = bhh * a.gk.ch, w0 = bw * a.gk.cw;
#pragma unroll
        for (int e = 0; e < 2; ++e)
            kok[e] = !a.gk.ragged || mm::slot_present(a.gk, ktab[ksub * kTile + warp * 16 + (lane >> 2) + 8 * e].packed, t0, h0, w0);
    }
    const float scale2 = a.sm_scale * 1.4426950408889634f;

    float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
        dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
        dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
    }

    for (int it = 0; it < n_tiles; ++it) {
        const int buf = it & 1;
        if (it + 1 < n_tiles) {
            const int nqb = tl[t_lo + (it + 1) / tiles_q], nsub = (it + 1) % tiles_q;
            mm::load_tile<T, D, kTile, kBwdThreads>(q_s + (buf ^ 1) * kTB, qh, a.q.ss, a.gq, qtab, nqb, nsub * kTile, tid);
            mm::load_tile<T, D, kTile, kBwdThreads>(do_s + (buf ^ 1) * kTB, doh, a.dout.ss, a.gq, qtab, nqb, nsub * kTile, tid);
            load_q_scalars(lse2 + (buf ^ 1) * kTile, delta + (buf ^ 1) * kTile, q_ok + (buf ^ 1) * kTile, lse_h, delta_h, a.gq, qtab, nqb,
                           nsub * kTile, tid);
        }
        mm::cp_async_commit();
        mm::cp_async_wait<1>();
        __syncthreads();
        const uint32_t qt = mm::smem_u32(q_s) + buf * kTB, dot = mm::smem_u32(do_s) + buf * kTB;
        const float* l2 = lse2 + buf * kTile;
        const float* dl = delta + buf * kTile;
        const unsigned char* qok = q_ok + buf * kTile;

        // S^T = K Q^T and dP^T = V dO^T for this warp's 16 keys: rows are keys, columns are the 64 query rows of the tile
        float st[8][4], dpt[8][4];
        mma_abt2_sa<T, D>(st, dpt, mm::smem_u32(k_s), mm::smem_u32(v_s), qt, dot, warp, lane);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int col = nt * 8 + 2 * (lane & 3) + (e & 1), r = e >> 1;
                const float p = (kok[r] && qok[col]) ? mm::ex2(fmaf(st[nt][e], scale2, -l2[col])) : 0.f;  // P^T
                st[nt][e] = p;
                dpt[nt][e] = p * (dpt[nt][e] - dl[col]) * a.sm_scale;                                       // dS^T
            }
        }
        mma_xb2<T, D>(dv, st, dot, dk, dpt, qt, lane);  // dV += P^T dO,  dK += dS^T Q
        __syncthreads();
    }
    mm::cp_async_wait<0>();
    __syncthreads();
    stage_rows<T, D>(k_s, dk, warp, lane);
    stage_rows<T, D>(v_s, dv, warp, lane);
    __syncthreads();
    write_rows<T, D>(k_s, dkh, a.dk.ss, a.gk, ktab, kb, ksub * kTile, tid);
    write_rows<T, D>(v_s, dvh, a.dv.ss, a.gk, ktab, kb, ksub * kTile, tid);
}

// ------------------------------------------------------------------------------------------ blocks as 64-token units
//
// The backward has no per-block state (no running maximum: lse is given), so a block of 128, 256 or 512 tokens is just
// the union of 64-token pieces, and on whole grids those pieces are the blocks of a finer grid over the same tokens.
// The tcgen05 passes stream 64-token tiles and own tiles of 64 or 128 tokens; the lists are rewritten in those terms: on
// the row side a query unit takes the list of its block, on the value side a selected key block becomes its units.

struct UnitSplit {
    Geom gu;         // the grid with the unit as block
    int rt, rh, rw;  // units per block along t, h, w
    int units;
};

// halves the block (w first, then h, then t) until 64 tokens are left; false when that cannot be done
bool split_units64(const Geom& g, UnitSplit* out) {
    if (g.bs < kTile || (g.ragged && g.bs != kTile)) return false;  // partial blocks are only taken whole
    int ut = g.ct, uh = g.ch, uw = g.cw;
    while (ut * uh * uw > kTile) {
        if (uw % 2 == 0) uw /= 2;
        else if (uh % 2 == 0) uh /= 2;
        else if (ut % 2 == 0) ut /= 2;
        else return false;
    }
    if (ut * uh * uw != kTile) return false;
    LcbsaGrid lg;
    lg.T = g.T; lg.H = g.H; lg.W = g.W;
    lg.ct = ut; lg.ch = uh; lg.cw = uw;
    out->gu = make_geom(lg);
    out->rt = g.ct / ut; out->rh = g.ch / uh; out->rw = g.cw / uw;
    out->units = out->rt * out->rh * out->rw;
    return true;
}

// one thread per (batch*head, query unit, list position): the units of that key block, in (t, h, w) order
__global__ void __launch_bounds__(256) bwd_expand_lists_kernel(const int32_t* idx, const int32_t* cnt, int cap, Geom gq, UnitSplit sq, Geom gk,
                                                               UnitSplit sk, long long total, int32_t* idx_u, int32_t* cnt_u) {
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= total) return;
    const int e = (int)(p % cap);
    const long long rest = p / cap;
    const int qu = (int)(rest % sq.gu.nblk);
    const long long bh = rest / sq.gu.nblk;
    int ut, uh, uw;
    block_coords(sq.gu, qu, ut, uh, uw);
    const int q = ((ut / sq.rt) * gq.Nh + uh / sq.rh) * gq.Nw + uw / sq.rw;
    const int n = min(max(cnt[bh * gq.nblk + q], 0), cap);
    if (e == 0) cnt_u[bh * sq.gu.nblk + qu] = n * sk.units;
    if (e >= n) return;
    const int j = idx[(bh * gq.nblk + q) * cap + e];
    int32_t* dst = idx_u + ((bh * sq.gu.nblk + qu) * cap + e) * sk.units;
    const bool in_grid = (unsigned)j < (unsigned)gk.nblk;  // an entry outside the grid stays outside: flagged later, never an address
    int bt, bhh, bw;
    block_coords(gk, in_grid ? j : 0, bt, bhh, bw);
    for (int u = 0; u < sk.units; ++u) {
        const int sw = u % sk.rw, sh = (u / sk.rw) % sk.rh, stt = u / (sk.rw * sk.rh);
        dst[u] = in_grid ? ((bt * sk.rt + stt) * sk.gu.Nh + (bhh * sk.rh + sh)) * sk.gu.Nw + (bw * sk.rw + sw) : -1;
    }
}

template <typename T, int D>
cudaError_t run_bwd(const BwdArgs& a, cudaStream_t st, const char** why) {
    const long long Sq = (long long)a.gq.T * a.gq.H * a.gq.W;
    const long long rows = (long long)a.B * a.H * Sq;
    const int BH = a.B * a.H;
    if (rows == 0 || a.gk.nblk == 0) return cudaSuccess;
    {
        const long long threads = rows * 8;
        bwd_delta_kernel<T, D><<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(a.o, a.dout, a.delta, a.H, Sq, rows);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    // head_dim 128: the tcgen05 passes.  Their CTAs own a block of 64 or 128 tokens and stream 64-token
    // units, so the lists are rewritten in those terms: for the dQ pass (own query block -> key units) and for the dK/dV
    // pass (query unit -> own key block, which is then transposed).
    BwdTcPlan plan{};
    bool use_tc = false;
    const int32_t* t_idx = a.idx;  // the lists to transpose
    const int32_t* t_cnt = a.cnt;
    int t_cap = a.cap, t_nq = a.gq.nblk, t_nk = a.gk.nblk;
    if (D == 128) {
        UnitSplit sq, sk;
        if (split_units64(a.gq, &sq) && split_units64(a.gk, &sk)) {
            const UnitSplit idq{a.gq, 1, 1, 1, 1}, idk{a.gk, 1, 1, 1, 1};
            const UnitSplit& q1 = a.gq.bs == 128 ? idq : sq;  // own blocks of the dQ pass
            const UnitSplit& k2 = a.gk.bs == 128 ? idk : sk;  // own blocks of the dK/dV pass
            plan.own_q = q1.gu; plan.unit_k = sk.gu;
            plan.unit_q = sq.gu; plan.own_k = k2.gu;
            const bool rewrite1 = q1.units * sk.units > 1, rewrite2 = sq.units * k2.units > 1;
            const bool same = q1.units == sq.units && k2.units == sk.units;  // one rewriting serves both passes
            plan.list_q = rewrite1 ? a.idx_u : a.idx;
            plan.cnt_q = rewrite1 ? a.cnt_u : a.cnt;
            plan.cap_q = a.cap * sk.units;
            use_tc = attn_bwd_tc_supported(a, plan);
            if (use_tc) {
                if (rewrite1) {
                    const long long total = (long long)BH * q1.gu.nblk * a.cap;
                    bwd_expand_lists_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a.idx, a.cnt, a.cap, a.gq, q1, a.gk, sk, total, a.idx_u,
                                                                                           a.cnt_u);
                }
                if (rewrite2 && !same) {
                    const long long total = (long long)BH * sq.gu.nblk * a.cap;
                    bwd_expand_lists_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a.idx, a.cnt, a.cap, a.gq, sq, a.gk, k2, total, a.idx_t,
                                                                                           a.cnt_t);
                }
                cudaError_t e = cudaGetLastError();
                if (e != cudaSuccess) return e;
                if (rewrite2) {
                    t_idx = same ? a.idx_u : a.idx_t;
                    t_cnt = same ? a.cnt_u : a.cnt_t;
                }
                t_cap = a.cap * k2.units;
                t_nq = sq.gu.nblk;
                t_nk = k2.gu.nblk;
            }
        }
    }
    {
        const int Nq = t_nq, Nk = t_nk, Wq = (Nq + 31) / 32;
        const long long rows_k = (long long)BH * Nk, entries = (long long)BH * Nq * t_cap;
        cudaError_t e = cudaMemsetAsync(a.bitmap, 0, (size_t)rows_k * Wq * sizeof(uint32_t), st);
        if (e != cudaSuccess) return e;
        bwd_mark_kernel<<<(unsigned)((entries + 255) / 256), 256, 0, st>>>(t_idx, t_cnt, t_cap, Nq, Nk, Wq, entries, a.bitmap, a.status);
        bwd_count_kernel<<<(unsigned)((rows_k * 32 + 255) / 256), 256, 0, st>>>(a.bitmap, Wq, rows_k, a.tcnt);
        bwd_scan_kernel<<<BH, 256, 0, st>>>(a.tcnt, Nk, a.toff);
        bwd_emit_kernel<<<(unsigned)((rows_k * 32 + 255) / 256), 256, 0, st>>>(a.bitmap, Wq, Nk, Nq, t_cap, rows_k, a.toff, a.tidx);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    if (use_tc) {
        plan.toff = a.toff;
        plan.tidx = a.tidx;
        plan.tidx_stride = (long long)t_nq * t_cap;
        return launch_attn_bwd_tc(a, plan, st, why);
    }
    const size_t tabs = (size_t)(a.gq.bs + a.gk.bs) * sizeof(mm::SlotEntry);
    const size_t smem_dq = 6 * (size_t)kTile * D * 2 + 2 * kTile + tabs;
    const size_t smem_kv = 6 * (size_t)kTile * D * 2 + 2 * 2 * kTile * sizeof(float) + 2 * kTile + tabs;
    if (smem_kv > 227 * 1024) { *why = "block sizes too large for the backward's slot tables"; return cudaErrorInvalidValue; }
    // the attribute is per device and per kernel; setting it on every call costs a microsecond and keeps this stateless
    cudaError_t e = cudaFuncSetAttribute(bwd_dq_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(bwd_dkdv_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
    if (e != cudaSuccess) return e;
    bwd_dq_mma_kernel<T, D><<<dim3((unsigned)(a.gq.nblk * (a.gq.bs / kTile)), (unsigned)BH), kBwdThreads, smem_dq, st>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    bwd_dkdv_mma_kernel<T, D><<<dim3((unsigned)(a.gk.nblk * (a.gk.bs / kTile)), (unsigned)BH), kBwdThreads, smem_kv, st>>>(a);
    return cudaGetLastError();
}

}  // namespace

bool attn_bwd_supported(const BwdArgs& a, const char** why) {
    if (a.dtype != LCBSA_BF16 && a.dtype != LCBSA_FP16) { *why = "needs bf16 or fp16"; return false; }
    if (a.D != 64 && a.D != 128) { *why = "needs head_dim 64 or 128"; return false; }
    if (a.gq.bs % kTile != 0 || a.gk.bs % kTile != 0) { *why = "needs query and key blocks that are multiples of 64 tokens"; return false; }
    if (a.gq.T > 1023 || a.gq.H > 1023 || a.gq.W > 1023 || a.gk.T > 1023 || a.gk.H > 1023 || a.gk.W > 1023) {
        *why = "grid axis above 1023 tokens (slot coordinates are packed into 10-bit fields)";
        return false;
    }
    return true;
}

namespace {

// The workspace is laid out for the finest form the lists can take: 64-token units (a block of 64 * U tokens counts U times).
struct BwdLayout {
    size_t delta, tcnt, toff, tidx, bitmap, stats, idx_u, cnt_u, idx_t, cnt_t, total;
};

BwdLayout bwd_layout(long long BH, const Geom& gq, const Geom& gk, int cap) {
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t Sq = (size_t)gq.T * gq.H * gq.W;
    const size_t Uq = gq.bs >= kTile ? gq.bs / kTile : 1, Uk = gk.bs >= kTile ? gk.bs / kTile : 1;
    const size_t Nq = (size_t)gq.nblk * Uq, Nk = (size_t)gk.nblk * Uk, capu = (size_t)cap * Uk;
    BwdLayout l;
    size_t off = 0;
    l.delta = off;  off += up((size_t)BH * Sq * sizeof(float));
    l.tcnt = off;   off += up((size_t)BH * Nk * sizeof(int32_t));
    l.toff = off;   off += up((size_t)BH * (Nk + 1) * sizeof(int32_t));
    l.tidx = off;   off += up((size_t)BH * Nq * capu * sizeof(int32_t));
    l.bitmap = off; off += up((size_t)BH * Nk * ((Nq + 31) / 32) * sizeof(uint32_t));
    l.stats = off;  off += up((size_t)BH * Sq * 2 * sizeof(float));
    const size_t rewritten = Uq * Uk > 1 ? 1 : 0;  // 64-token blocks on both sides: the lists are used as they are
    l.idx_u = off;  off += up(rewritten * BH * Nq * capu * sizeof(int32_t));
    l.cnt_u = off;  off += up(rewritten * BH * Nq * sizeof(int32_t));
    l.idx_t = off;  off += up(rewritten * BH * Nq * capu * sizeof(int32_t));
    l.cnt_t = off;  off += up(rewritten * BH * Nq * sizeof(int32_t));
    l.total = off;
    return l;
}

}  // namespace

size_t attn_bwd_workspace_bytes(long long BH, const Geom& gq, const Geom& gk, int cap) { return bwd_layout(BH, gq, gk, cap).total; }

cudaError_t launch_attn_bwd(BwdArgs a, void* workspace, cudaStream_t st, const char** why) {
    const BwdLayout l = bwd_layout((long long)a.B * a.H, a.gq, a.gk, a.cap);
    unsigned char* w = static_cast<unsigned char*>(workspace);
    a.delta = reinterpret_cast<float*>(w + l.delta);
    a.tcnt = reinterpret_cast<int32_t*>(w + l.tcnt);
    a.toff = reinterpret_cast<int32_t*>(w + l.toff);
    a.tidx = reinterpret_cast<int32_t*>(w + l.tidx);
    a.bitmap = reinterpret_cast<uint32_t*>(w + l.bitmap);
    a.stats = reinterpret_cast<float*>(w + l.stats);
    a.idx_u = reinterpret_cast<int32_t*>(w + l.idx_u);
    a.cnt_u = reinterpret_cast<int32_t*>(w + l.cnt_u);
    a.idx_t = reinterpret_cast<int32_t*>(w + l.idx_t);
    a.cnt_t = reinterpret_cast<int32_t*>(w + l.cnt_t);
    if (a.dtype == LCBSA_BF16) return a.D == 128 ? run_bwd<__nv_bfloat16, 128>(a, st, why) : run_bwd<__nv_bfloat16, 64>(a, st, why);
    return a.D == 128 ? run_bwd<__half, 128>(a, st, why) : run_bwd<__half, 64>(a, st, why);
}

}  // namespace lcbsa
