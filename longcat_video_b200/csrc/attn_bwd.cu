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
//   bwd_dq_kernel         one CTA per 64 query rows, walks the forward lists;
//   bwd_dkdv_kernel       one CTA per 64 keys, walks the transposed lists.
// Tiles are 64 x 64 whatever the block sizes (multiples of 64 tokens): a block of 128 or more tokens is a run of
// 64-row tiles in slot order.  The contractions run on the tensor cores through warp-level mma (wmma, fp32
// accumulation); P and dS are rounded to the input dtype before they enter a contraction, as in the forward.
// This is the first, plain version of the backward: its roofline is the mma.sync rate, not tcgen05's.
#include <mma.h>

#include "common.cuh"

namespace lcbsa {

namespace {

using namespace nvcuda;

constexpr int kTile = 64;      // rows and keys per tile
constexpr int kBwdThreads = 128;

struct BwdSlot {
    int off;     // token offset of the slot relative to the block's first token
    int packed;  // lt | lh << 10 | lw << 20
};

template <typename T> struct Wm;
template <> struct Wm<__nv_bfloat16> { using type = __nv_bfloat16; };
template <> struct Wm<__half> { using type = half; };

__device__ __forceinline__ bool slot_in_grid(const Geom& g, int packed, int t0, int h0, int w0) {
    return (t0 + (packed & 1023) < g.T) && (h0 + ((packed >> 10) & 1023) < g.H) && (w0 + (packed >> 20) < g.W);
}

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

// ------------------------------------------------------------------------------------------ tile helpers

// Gather 64 slots (slot0 ..) of block `blk` of a [S, D] head into a [64][LD] shared tile; absent tokens read as zero.
// present[r] says whether row r exists.  Called by all threads of the CTA.
template <typename T, int D, int LD>
__device__ __forceinline__ void load_rows(T* tile, unsigned char* present, const T* head, long long ss, const Geom& g, const BwdSlot* tab, int blk,
                                          int slot0, int tid) {
    constexpr int CPR = D / 8;                           // 16-byte chunks per row
    constexpr int kPer = kTile * CPR / kBwdThreads;      // chunks per thread: all of them in flight before the first store
    int bt, bh, bw;
    block_coords(g, blk, bt, bh, bw);
    const int t0 = bt * g.ct, h0 = bh * g.ch, w0 = bw * g.cw;
    const long long origin = ((long long)t0 * g.H + h0) * g.W + w0;
    uint4 val[kPer];
    bool ok[kPer];
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
        const int v = tid + u * kBwdThreads, row = v / CPR, c = v % CPR;
        const BwdSlot e = tab[slot0 + row];
        ok[u] = !g.ragged || slot_in_grid(g, e.packed, t0, h0, w0);
        val[u] = make_uint4(0u, 0u, 0u, 0u);
        if (ok[u]) val[u] = __ldg(reinterpret_cast<const uint4*>(head + (origin + e.off) * ss + c * 8));
    }
#pragma unroll
    for (int u = 0; u < kPer; ++u) {
        const int v = tid + u * kBwdThreads, row = v / CPR, c = v % CPR;
        *reinterpret_cast<uint4*>(tile + row * LD + c * 8) = val[u];
        if (c == 0 && present != nullptr) present[row] = ok[u] ? 1 : 0;
    }
}

// Two tensors that share geometry and slots (K and V of a key tile), in two steps: fetch_rows2 issues every load of the
// thread into registers, commit_rows2 writes them to the shared tiles.  The dQ kernel fetches tile i + 1 before it
// computes on tile i, so the global-memory latency is spent under the contractions.  valid == false: a tile of zeros.
template <int D>
struct RowRegs2 {
    static constexpr int kPer = kTile * (D / 8) / kBwdThreads;
    uint4 a[kPer], b[kPer];
    bool ok[kPer];
};
template <typename T, int D>
__device__ __forceinline__ void fetch_rows2(RowRegs2<D>& r, const T* head0, long long ss0, const T* head1, long long ss1, const Geom& g,
                                            const BwdSlot* tab, int blk, int slot0, bool valid, int tid) {
    constexpr int CPR = D / 8;
    int bt, bh, bw;
    block_coords(g, valid ? blk : 0, bt, bh, bw);
    const int t0 = bt * g.ct, h0 = bh * g.ch, w0 = bw * g.cw;
    const long long origin = ((long long)t0 * g.H + h0) * g.W + w0;
#pragma unroll
    for (int u = 0; u < RowRegs2<D>::kPer; ++u) {
        const int v = tid + u * kBwdThreads, row = v / CPR, c = v % CPR;
        const BwdSlot e = tab[slot0 + row];
        r.ok[u] = valid && (!g.ragged || slot_in_grid(g, e.packed, t0, h0, w0));
        r.a[u] = r.b[u] = make_uint4(0u, 0u, 0u, 0u);
        if (r.ok[u]) {
            r.a[u] = __ldg(reinterpret_cast<const uint4*>(head0 + (origin + e.off) * ss0 + c * 8));
            r.b[u] = __ldg(reinterpret_cast<const uint4*>(head1 + (origin + e.off) * ss1 + c * 8));
        }
    }
}
template <typename T, int D, int LD>
__device__ __forceinline__ void commit_rows2(const RowRegs2<D>& r, T* tile0, T* tile1, unsigned char* present, int tid) {
    constexpr int CPR = D / 8;
#pragma unroll
    for (int u = 0; u < RowRegs2<D>::kPer; ++u) {
        const int v = tid + u * kBwdThreads, row = v / CPR, c = v % CPR;
        *reinterpret_cast<uint4*>(tile0 + row * LD + c * 8) = r.a[u];
        *reinterpret_cast<uint4*>(tile1 + row * LD + c * 8) = r.b[u];
        if (c == 0) present[row] = r.ok[u] ? 1 : 0;
    }
}

// fp32 per-row values (lse or delta) of the same 64 slots; absent rows read as zero.
__device__ __forceinline__ void load_row_scalars(float* dst, const float* src, const Geom& g, const BwdSlot* tab, int blk, int slot0, int tid) {
    int bt, bh, bw;
    block_coords(g, blk, bt, bh, bw);
    const int t0 = bt * g.ct, h0 = bh * g.ch, w0 = bw * g.cw;
    const long long origin = ((long long)t0 * g.H + h0) * g.W + w0;
    for (int r = tid; r < kTile; r += kBwdThreads) {
        const BwdSlot e = tab[slot0 + r];
        const bool ok = !g.ragged || slot_in_grid(g, e.packed, t0, h0, w0);
        dst[r] = ok ? src[origin + e.off] : 0.f;
    }
}

// Write a [64][D] fp32 tile (leading dimension LDF) as T into the rows of the block that exist.
template <typename T, int D, int LDF>
__device__ __forceinline__ void store_rows(const float* tile, T* head, long long ss, const Geom& g, const BwdSlot* tab, int blk, int slot0, int tid) {
    constexpr int CPR = D / 8;
    int bt, bh, bw;
    block_coords(g, blk, bt, bh, bw);
    const int t0 = bt * g.ct, h0 = bh * g.ch, w0 = bw * g.cw;
    const long long origin = ((long long)t0 * g.H + h0) * g.W + w0;
    for (int v = tid; v < kTile * CPR; v += kBwdThreads) {
        const int row = v / CPR, c = v % CPR;
        const BwdSlot e = tab[slot0 + row];
        if (g.ragged && !slot_in_grid(g, e.packed, t0, h0, w0)) continue;
        uint4 val;
        T* v8 = reinterpret_cast<T*>(&val);
#pragma unroll
        for (int x = 0; x < 8; ++x) v8[x] = DType<T>::from_f32(tile[row * LDF + c * 8 + x]);
        *reinterpret_cast<uint4*>(head + (origin + e.off) * ss + c * 8) = val;
    }
}

__device__ __forceinline__ void fill_slot_table(BwdSlot* tab, const Geom& g, int tid) {
    for (int r = tid; r < g.bs; r += kBwdThreads) {
        int lt, lh, lw;
        slot_coords(g, r, lt, lh, lw);
        tab[r] = BwdSlot{(lt * g.H + lh) * g.W + lw, lt | (lh << 10) | (lw << 20)};
    }
}

// One warp: C[16 x 64] (fp32, into `out` with leading dimension LDO) = A[16 x D] * B[64 x D]^T.
template <typename T, int D, int LDA, int LDB, int LDO>
__device__ __forceinline__ void warp_abt_16x64(float* out, const T* a_rows, const T* b_rows) {
    using W = typename Wm<T>::type;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[4];
#pragma unroll
    for (int n = 0; n < 4; ++n) wmma::fill_fragment(acc[n], 0.f);
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::row_major> fa;
        wmma::load_matrix_sync(fa, reinterpret_cast<const W*>(a_rows) + kk * 16, LDA);
#pragma unroll
        for (int n = 0; n < 4; ++n) {
            wmma::fragment<wmma::matrix_b, 16, 16, 16, W, wmma::col_major> fb;  // B(k, n) = b_rows[n][k]
            wmma::load_matrix_sync(fb, reinterpret_cast<const W*>(b_rows) + n * 16 * LDB + kk * 16, LDB);
            wmma::mma_sync(acc[n], fa, fb, acc[n]);
        }
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) wmma::store_matrix_sync(out + n * 16, acc[n], LDO, wmma::mem_row_major);
}

// ------------------------------------------------------------------------------------------ shared-memory plan

// About 106 KB for head_dim 128, so that two CTAs share an SM.  P and dS (input dtype) are written over the rows of S and
// dP (fp32) they were computed from, and the fp32 staging of a finished [64][D] result lies over the two operand tiles
// that are dead by then.
template <typename T, int D>
struct BwdSmem {
    static constexpr int LD = D + 8;        // operand tiles, in elements (row stride 16 bytes off a bank period)
    static constexpr int LDF = kTile + 4;   // fp32 S / dP tiles
    static constexpr int LDP = 2 * LDF;     // the same rows seen as T: P / dS in place
    static constexpr int LDO = D + 4;       // fp32 staging of a [64][D] result
    static constexpr size_t tile_bytes = (size_t)kTile * LD * sizeof(T);
    static constexpr size_t f_bytes = (size_t)kTile * LDF * sizeof(float);
    static constexpr size_t stage_bytes = (size_t)kTile * LDO * sizeof(float);
    static_assert(stage_bytes <= 2 * tile_bytes, "the staging tile lies over operand tiles c and d");
    // a, b, c, d: four operand tiles; sf, dpf: fp32 (then P, dS); scalars: lse, delta (fp32 x 64 each), flags (2 x 64 bytes)
    static constexpr size_t off_a = 0, off_b = tile_bytes, off_c = 2 * tile_bytes, off_d = 3 * tile_bytes;
    static constexpr size_t off_sf = 4 * tile_bytes;
    static constexpr size_t off_dpf = off_sf + f_bytes;
    static constexpr size_t off_sc = off_dpf + f_bytes;
    static constexpr size_t off_stage = off_c;
    static constexpr size_t bytes_no_tab = off_sc + 2 * kTile * sizeof(float) + 2 * kTile;
};

// P and dS of the 16 query rows of one warp from its S and dP rows (fp32) -> T, written over the same rows.  A lane owns
// half a row (32 keys): it reads its 32 values of S and of dP into registers, the warp synchronises (the bytes a lane
// writes belong to the span its neighbour reads), then it writes 32 values of P and of dS.
template <typename T, int LDF, int LDP>
__device__ __forceinline__ void warp_softmax_grad_rows(float* sf, float* dpf, const float* lse, const float* delta, const unsigned char* q_ok,
                                                       const unsigned char* k_ok, float sm_scale, int row0, int lane) {
    const float scale2 = sm_scale * 1.4426950408889634f;
    const int r = row0 + (lane >> 1), c0 = (lane & 1) * 32;
    float sv[32], dv[32];
#pragma unroll
    for (int x = 0; x < 8; ++x) {
        const float4 a = *reinterpret_cast<const float4*>(sf + r * LDF + c0 + 4 * x);
        const float4 b = *reinterpret_cast<const float4*>(dpf + r * LDF + c0 + 4 * x);
        sv[4 * x] = a.x; sv[4 * x + 1] = a.y; sv[4 * x + 2] = a.z; sv[4 * x + 3] = a.w;
        dv[4 * x] = b.x; dv[4 * x + 1] = b.y; dv[4 * x + 2] = b.z; dv[4 * x + 3] = b.w;
    }
    const float l2 = lse[r] * 1.4426950408889634f, dl = delta[r];
    const bool row_ok = q_ok[r] != 0;
    uint32_t kf[8];  // presence flags of this lane's 32 keys, four per word
#pragma unroll
    for (int x = 0; x < 8; ++x) kf[x] = *reinterpret_cast<const uint32_t*>(k_ok + c0 + 4 * x);
    __syncwarp();
    T* ps = reinterpret_cast<T*>(sf) + r * LDP + c0;
    T* dss = reinterpret_cast<T*>(dpf) + r * LDP + c0;
#pragma unroll
    for (int x = 0; x < 4; ++x) {
        uint4 pw, dw;
        T* p8 = reinterpret_cast<T*>(&pw);
        T* d8 = reinterpret_cast<T*>(&dw);
#pragma unroll
        for (int y = 0; y < 8; ++y) {
            const int c = 8 * x + y;
            const bool ok = row_ok && ((kf[c >> 2] >> (8 * (c & 3))) & 0xffu) != 0;
            const float p = ok ? exp2f(sv[c] * scale2 - l2) : 0.f;
            p8[y] = DType<T>::from_f32(p);
            d8[y] = DType<T>::from_f32(p * (dv[c] - dl) * sm_scale);
        }
        *reinterpret_cast<uint4*>(ps + 8 * x) = pw;
        *reinterpret_cast<uint4*>(dss + 8 * x) = dw;
    }
    __syncwarp();
}

// ------------------------------------------------------------------------------------------ dQ

template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads) bwd_dq_kernel(const __grid_constant__ BwdArgs a) {
    using SM = BwdSmem<T, D>;
    using W = typename Wm<T>::type;
    extern __shared__ __align__(128) unsigned char smem[];
    T* qs = reinterpret_cast<T*>(smem + SM::off_a);
    T* dos = reinterpret_cast<T*>(smem + SM::off_b);
    T* ks = reinterpret_cast<T*>(smem + SM::off_c);
    T* vs = reinterpret_cast<T*>(smem + SM::off_d);
    float* sf = reinterpret_cast<float*>(smem + SM::off_sf);
    float* dpf = reinterpret_cast<float*>(smem + SM::off_dpf);
    T* ps = reinterpret_cast<T*>(sf);     // P and dS replace S and dP row by row
    T* dss = reinterpret_cast<T*>(dpf);
    float* lse = reinterpret_cast<float*>(smem + SM::off_sc);
    float* delta = lse + kTile;
    unsigned char* q_ok = reinterpret_cast<unsigned char*>(delta + kTile);
    unsigned char* k_ok = q_ok + kTile;
    float* stage = reinterpret_cast<float*>(smem + SM::off_stage);
    BwdSlot* qtab = reinterpret_cast<BwdSlot*>(smem + SM::bytes_no_tab);
    BwdSlot* ktab = qtab + a.gq.bs;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tiles_q = a.gq.bs / kTile, tiles_k = a.gk.bs / kTile;
    const int qb = blockIdx.x / tiles_q, qsub = blockIdx.x % tiles_q;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    fill_slot_table(qtab, a.gq, tid);
    fill_slot_table(ktab, a.gk, tid);
    __syncthreads();

    const long long Sq = (long long)a.gq.T * a.gq.H * a.gq.W;
    const T* qh = reinterpret_cast<const T*>(a.q.data) + (long long)b * a.q.sb + (long long)h * a.q.sh;
    const T* kh = reinterpret_cast<const T*>(a.k.data) + (long long)b * a.k.sb + (long long)h * a.k.sh;
    const T* vh = reinterpret_cast<const T*>(a.v.data) + (long long)b * a.v.sb + (long long)h * a.v.sh;
    const T* doh = reinterpret_cast<const T*>(a.dout.data) + (long long)b * a.dout.sb + (long long)h * a.dout.sh;
    T* dqh = reinterpret_cast<T*>(const_cast<void*>(a.dq.data)) + (long long)b * a.dq.sb + (long long)h * a.dq.sh;

    load_rows<T, D, SM::LD>(qs, q_ok, qh, a.q.ss, a.gq, qtab, qb, qsub * kTile, tid);
    load_rows<T, D, SM::LD>(dos, nullptr, doh, a.dout.ss, a.gq, qtab, qb, qsub * kTile, tid);
    load_row_scalars(lse, a.lse + (long long)bh * Sq, a.gq, qtab, qb, qsub * kTile, tid);
    load_row_scalars(delta, a.delta + (long long)bh * Sq, a.gq, qtab, qb, qsub * kTile, tid);

    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[D / 16];  // dQ rows 16 * warp .. of this tile
#pragma unroll
    for (int n = 0; n < D / 16; ++n) wmma::fill_fragment(acc[n], 0.f);

    const int32_t* list = a.idx + ((long long)bh * a.gq.nblk + qb) * a.cap;
    const int n_list = min(max(a.cnt[(long long)bh * a.gq.nblk + qb], 0), a.cap);
    // tiles of the listed key blocks, one after the other; tile it + 1 is fetched into registers while tile it is
    // computed on.  An entry outside [0, Nk) (flagged by the mark kernel) is a tile of absent keys.
    const int n_tiles = n_list * tiles_k;
    RowRegs2<D> regs;
    auto fetch = [&](int it) {
        const int kb = list[it / tiles_k];
        fetch_rows2<T, D>(regs, kh, a.k.ss, vh, a.v.ss, a.gk, ktab, kb, (it % tiles_k) * kTile, (unsigned)kb < (unsigned)a.gk.nblk, tid);
    };
    if (n_tiles > 0) fetch(0);
    for (int it = 0; it < n_tiles; ++it) {
        __syncthreads();  // the previous tile's K and V have been read by every warp
        commit_rows2<T, D, SM::LD>(regs, ks, vs, k_ok, tid);
        __syncthreads();
        if (it + 1 < n_tiles) fetch(it + 1);
        {
            const int row0 = 16 * warp;
            warp_abt_16x64<T, D, SM::LD, SM::LD, SM::LDF>(sf + row0 * SM::LDF, qs + row0 * SM::LD, ks);
            warp_abt_16x64<T, D, SM::LD, SM::LD, SM::LDF>(dpf + row0 * SM::LDF, dos + row0 * SM::LD, vs);
            __syncwarp();
            warp_softmax_grad_rows<T, SM::LDF, SM::LDP>(sf, dpf, lse, delta, q_ok, k_ok, a.sm_scale, row0, lane);
            __syncwarp();
            // dQ[16 x D] += dS[16 x 64] * K[64 x D]
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::row_major> fa;
                wmma::load_matrix_sync(fa, reinterpret_cast<const W*>(dss) + row0 * SM::LDP + kk * 16, SM::LDP);
#pragma unroll
                for (int n = 0; n < D / 16; ++n) {
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, W, wmma::row_major> fb;
                    wmma::load_matrix_sync(fb, reinterpret_cast<const W*>(ks) + kk * 16 * SM::LD + n * 16, SM::LD);
                    wmma::mma_sync(acc[n], fa, fb, acc[n]);
                }
            }
        }
    }
    // every warp stages its 16 rows (its own region of the staging tile, which lies over the K and V tiles), then the
    // CTA writes the rows that exist
    __syncthreads();
#pragma unroll
    for (int n = 0; n < D / 16; ++n) wmma::store_matrix_sync(stage + 16 * warp * SM::LDO + n * 16, acc[n], SM::LDO, wmma::mem_row_major);
    __syncthreads();
    store_rows<T, D, SM::LDO>(stage, dqh, a.dq.ss, a.gq, qtab, qb, qsub * kTile, tid);
}

// ------------------------------------------------------------------------------------------ dK, dV

template <typename T, int D>
__global__ void __launch_bounds__(kBwdThreads) bwd_dkdv_kernel(const __grid_constant__ BwdArgs a) {
    using SM = BwdSmem<T, D>;
    using W = typename Wm<T>::type;
    extern __shared__ __align__(128) unsigned char smem[];
    T* ks = reinterpret_cast<T*>(smem + SM::off_a);
    T* vs = reinterpret_cast<T*>(smem + SM::off_b);
    T* qs = reinterpret_cast<T*>(smem + SM::off_c);
    T* dos = reinterpret_cast<T*>(smem + SM::off_d);
    float* sf = reinterpret_cast<float*>(smem + SM::off_sf);
    float* dpf = reinterpret_cast<float*>(smem + SM::off_dpf);
    T* ps = reinterpret_cast<T*>(sf);     // P and dS replace S and dP row by row
    T* dss = reinterpret_cast<T*>(dpf);
    float* lse = reinterpret_cast<float*>(smem + SM::off_sc);
    float* delta = lse + kTile;
    unsigned char* q_ok = reinterpret_cast<unsigned char*>(delta + kTile);
    unsigned char* k_ok = q_ok + kTile;
    float* stage = reinterpret_cast<float*>(smem + SM::off_stage);
    BwdSlot* qtab = reinterpret_cast<BwdSlot*>(smem + SM::bytes_no_tab);
    BwdSlot* ktab = qtab + a.gq.bs;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tiles_q = a.gq.bs / kTile, tiles_k = a.gk.bs / kTile;
    const int kb = blockIdx.x / tiles_k, ksub = blockIdx.x % tiles_k;
    const int bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    fill_slot_table(qtab, a.gq, tid);
    fill_slot_table(ktab, a.gk, tid);
    __syncthreads();

    const long long Sq = (long long)a.gq.T * a.gq.H * a.gq.W;
    const T* qh = reinterpret_cast<const T*>(a.q.data) + (long long)b * a.q.sb + (long long)h * a.q.sh;
    const T* kh = reinterpret_cast<const T*>(a.k.data) + (long long)b * a.k.sb + (long long)h * a.k.sh;
    const T* vh = reinterpret_cast<const T*>(a.v.data) + (long long)b * a.v.sb + (long long)h * a.v.sh;
    const T* doh = reinterpret_cast<const T*>(a.dout.data) + (long long)b * a.dout.sb + (long long)h * a.dout.sh;
    T* dkh = reinterpret_cast<T*>(const_cast<void*>(a.dk.data)) + (long long)b * a.dk.sb + (long long)h * a.dk.sh;
    T* dvh = reinterpret_cast<T*>(const_cast<void*>(a.dv.data)) + (long long)b * a.dv.sb + (long long)h * a.dv.sh;

    load_rows<T, D, SM::LD>(ks, k_ok, kh, a.k.ss, a.gk, ktab, kb, ksub * kTile, tid);
    load_rows<T, D, SM::LD>(vs, nullptr, vh, a.v.ss, a.gk, ktab, kb, ksub * kTile, tid);

    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc_k[D / 16], acc_v[D / 16];  // key rows 16 * warp .. of this tile
#pragma unroll
    for (int n = 0; n < D / 16; ++n) {
        wmma::fill_fragment(acc_k[n], 0.f);
        wmma::fill_fragment(acc_v[n], 0.f);
    }
    const int32_t* tl = a.tidx + (long long)bh * a.gq.nblk * a.cap;
    const int t_lo = a.toff[(long long)bh * (a.gk.nblk + 1) + kb], t_hi = a.toff[(long long)bh * (a.gk.nblk + 1) + kb + 1];
    for (int t = t_lo; t < t_hi; ++t) {
        const int qb = tl[t];
        for (int qsub = 0; qsub < tiles_q; ++qsub) {
            __syncthreads();  // the previous tile's Q, dO, P and dS have been read by every warp
            load_rows<T, D, SM::LD>(qs, q_ok, qh, a.q.ss, a.gq, qtab, qb, qsub * kTile, tid);
            load_rows<T, D, SM::LD>(dos, nullptr, doh, a.dout.ss, a.gq, qtab, qb, qsub * kTile, tid);
            load_row_scalars(lse, a.lse + (long long)bh * Sq, a.gq, qtab, qb, qsub * kTile, tid);
            load_row_scalars(delta, a.delta + (long long)bh * Sq, a.gq, qtab, qb, qsub * kTile, tid);
            __syncthreads();
            const int row0 = 16 * warp;  // query rows of this warp for S, dP, P, dS
            warp_abt_16x64<T, D, SM::LD, SM::LD, SM::LDF>(sf + row0 * SM::LDF, qs + row0 * SM::LD, ks);
            warp_abt_16x64<T, D, SM::LD, SM::LD, SM::LDF>(dpf + row0 * SM::LDF, dos + row0 * SM::LD, vs);
            __syncwarp();
            warp_softmax_grad_rows<T, SM::LDF, SM::LDP>(sf, dpf, lse, delta, q_ok, k_ok, a.sm_scale, row0, lane);
            __syncthreads();  // all 64 query rows of P and dS are needed by every warp now
            // key rows 16 * warp ..:  dV += P^T dO,  dK += dS^T Q   (A = P^T: column-major view of the [q][k] tile)
#pragma unroll
            for (int kk = 0; kk < kTile / 16; ++kk) {
                wmma::fragment<wmma::matrix_a, 16, 16, 16, W, wmma::col_major> fp, fs;
                wmma::load_matrix_sync(fp, reinterpret_cast<const W*>(ps) + kk * 16 * SM::LDP + row0, SM::LDP);
                wmma::load_matrix_sync(fs, reinterpret_cast<const W*>(dss) + kk * 16 * SM::LDP + row0, SM::LDP);
#pragma unroll
                for (int n = 0; n < D / 16; ++n) {
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, W, wmma::row_major> fb;
                    wmma::load_matrix_sync(fb, reinterpret_cast<const W*>(dos) + kk * 16 * SM::LD + n * 16, SM::LD);
                    wmma::mma_sync(acc_v[n], fp, fb, acc_v[n]);
                    wmma::load_matrix_sync(fb, reinterpret_cast<const W*>(qs) + kk * 16 * SM::LD + n * 16, SM::LD);
                    wmma::mma_sync(acc_k[n], fs, fb, acc_k[n]);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int n = 0; n < D / 16; ++n) wmma::store_matrix_sync(stage + 16 * warp * SM::LDO + n * 16, acc_k[n], SM::LDO, wmma::mem_row_major);
    __syncthreads();
    store_rows<T, D, SM::LDO>(stage, dkh, a.dk.ss, a.gk, ktab, kb, ksub * kTile, tid);
    __syncthreads();
#pragma unroll
    for (int n = 0; n < D / 16; ++n) wmma::store_matrix_sync(stage + 16 * warp * SM::LDO + n * 16, acc_v[n], SM::LDO, wmma::mem_row_major);
    __syncthreads();
    store_rows<T, D, SM::LDO>(stage, dvh, a.dv.ss, a.gk, ktab, kb, ksub * kTile, tid);
}

template <typename T, int D>
cudaError_t run_bwd(const BwdArgs& a, cudaStream_t st, const char** why) {
    using SM = BwdSmem<T, D>;
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
    {
        const int Nq = a.gq.nblk, Nk = a.gk.nblk, Wq = (Nq + 31) / 32;
        const long long rows_k = (long long)BH * Nk, entries = (long long)BH * Nq * a.cap;
        cudaError_t e = cudaMemsetAsync(a.bitmap, 0, (size_t)rows_k * Wq * sizeof(uint32_t), st);
        if (e != cudaSuccess) return e;
        bwd_mark_kernel<<<(unsigned)((entries + 255) / 256), 256, 0, st>>>(a.idx, a.cnt, a.cap, Nq, Nk, Wq, entries, a.bitmap, a.status);
        bwd_count_kernel<<<(unsigned)((rows_k * 32 + 255) / 256), 256, 0, st>>>(a.bitmap, Wq, rows_k, a.tcnt);
        bwd_scan_kernel<<<BH, 256, 0, st>>>(a.tcnt, Nk, a.toff);
        bwd_emit_kernel<<<(unsigned)((rows_k * 32 + 255) / 256), 256, 0, st>>>(a.bitmap, Wq, Nk, Nq, a.cap, rows_k, a.toff, a.tidx);
        e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    const size_t smem = SM::bytes_no_tab + (size_t)(a.gq.bs + a.gk.bs) * sizeof(BwdSlot);
    if (smem > 227 * 1024) { *why = "block sizes too large for the backward's slot tables"; return cudaErrorInvalidValue; }
    // the attribute is per device and per kernel; setting it on every call costs a microsecond and keeps this stateless
    cudaError_t e = cudaFuncSetAttribute(bwd_dq_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(bwd_dkdv_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    bwd_dq_kernel<T, D><<<dim3((unsigned)(a.gq.nblk * (a.gq.bs / kTile)), (unsigned)BH), kBwdThreads, smem, st>>>(a);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    bwd_dkdv_kernel<T, D><<<dim3((unsigned)(a.gk.nblk * (a.gk.bs / kTile)), (unsigned)BH), kBwdThreads, smem, st>>>(a);
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

size_t attn_bwd_workspace_bytes(long long BH, long long Sq, int Nq, int Nk, int cap) {
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    return up((size_t)BH * Sq * sizeof(float)) + up((size_t)BH * Nk * sizeof(int32_t)) + up((size_t)BH * (Nk + 1) * sizeof(int32_t)) +
           up((size_t)BH * Nq * cap * sizeof(int32_t)) + up((size_t)BH * Nk * ((Nq + 31) / 32) * sizeof(uint32_t));
}

cudaError_t launch_attn_bwd(BwdArgs a, void* workspace, cudaStream_t st, const char** why) {
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    const long long BH = (long long)a.B * a.H, Sq = (long long)a.gq.T * a.gq.H * a.gq.W;
    unsigned char* w = static_cast<unsigned char*>(workspace);
    a.delta = reinterpret_cast<float*>(w);
    w += up((size_t)BH * Sq * sizeof(float));
    a.tcnt = reinterpret_cast<int32_t*>(w);
    w += up((size_t)BH * a.gk.nblk * sizeof(int32_t));
    a.toff = reinterpret_cast<int32_t*>(w);
    w += up((size_t)BH * (a.gk.nblk + 1) * sizeof(int32_t));
    a.tidx = reinterpret_cast<int32_t*>(w);
    w += up((size_t)BH * a.gq.nblk * a.cap * sizeof(int32_t));
    a.bitmap = reinterpret_cast<uint32_t*>(w);
    if (a.dtype == LCBSA_BF16) return a.D == 128 ? run_bwd<__nv_bfloat16, 128>(a, st, why) : run_bwd<__nv_bfloat16, 64>(a, st, why);
    return a.D == 128 ? run_bwd<__half, 128>(a, st, why) : run_bwd<__half, 64>(a, st, why);
}

}  // namespace lcbsa
