// Block-sparse attention backward on TMA + tcgen05 + TMEM for head_dim 128: the dQ pass and the dK/dV pass, after the delta
// kernel and the transposition of the block lists of attn_bwd.cu (which keeps head_dim 64, and ragged grids in fp16 or with
// blocks above 64 tokens, on warp-level MMAs).  A CTA owns a block of 64 or 128 tokens (kM rows: M=64 or M=128 MMAs) and
// streams 64-token tiles; attn_bwd.cu writes the lists in those terms (larger blocks are taken as 64-token units).
// Stands in for the Triton kernels _attn_bwd_dq_bsa_varlen_align and _attn_bwd_dkdv_bsa_varlen_align
// (longcat_video/block_sparse_attention/flash_attn_bsa_varlen_mask.py:289-945).
//
// Both passes are one kernel with the roles of the operands exchanged.  A CTA owns one tile pair (A1, A2) of kM rows and
// walks a list of 64-row tile pairs (B1, B2); per list entry
//
//   dQ pass   (CTA = query block i, list = its key blocks j):  A1 = Q_i  A2 = dO_i  B1 = K_j  B2 = V_j
//       S  = A1 B1^T        dP  = A2 B2^T        dS  = P o (dP - delta_i) * scale        dQ_i += dS B1
//   dK/dV pass (CTA = key block j, list = the query blocks i that selected it):  A1 = K_j  A2 = V_j  B1 = Q_i  B2 = dO_i
//       S^T = A1 B1^T       dP^T = A2 B2^T       P^T, dS^T as above, transposed          dV_j += P^T B2   dK_j += dS^T B1
//
// with P = exp2(S * scale * log2(e) - lse * log2(e)).  S and dP are (M = kM) N64 K128 MMAs with both operands in shared
// memory (fp32 in TMEM); P and dS are written back to TMEM in the input dtype and are the A operands of the N128 K64 MMAs
// that accumulate the gradients in TMEM over the whole list, with the streamed tile as MN-major B operand: a tile is
// loaded once (two 5-D TMA boxes of 64 columns, 128-byte swizzle) and serves as K-major operand of the first
// contraction and as MN-major operand of the last.  Nothing is recomputed within a pass, nothing goes through shared
// memory between the contractions, and no gradient is accumulated with atomics.
//
// Ragged grids (64-token blocks, bf16): the boxes of partial blocks are zero-filled by TMA outside the grid; a key outside
// the grid then has K = V = 0 and a query row outside has Q = dO = 0, so every term they enter is a finite number times
// zero and needs no mask (P of such a key is 2^(-lse * log2 e), finite in fp32 and bf16; fp16 could overflow, so fp16 keeps
// ragged grids on the warp-level kernels); rows outside the grid are not stored.
//
//   warps 0-7 : arithmetic.  A thread serves one TMEM lane = one row of the kM x 64 tile (an M=128 accumulator has row r in
//               lane r, an M=64 one occupies lanes 0-15 of every 32-lane quadrant)
//   warp 8    : TMA producer: the CTA's own tiles once, then a ring of five (four for kM = 128) (B1, B2) slots; in the
//               dK/dV pass also the query block's 64 (lse * log2 e) and 64 delta values per slot, by a bulk copy onto the
//               same barrier (bwd_stats_kernel lays them out per block)
//   warp 9    : issues every MMA, one elected lane
//
// TMEM and the order of the MMAs.  P and dS (16-bit pairs) have columns of their own, twice, in both passes: the values
// of entry s + 2 go where those of entry s were and are written after s_full(s + 2), a commit the issuer makes behind
// TS(s), so no buffer is rewritten while an MMA may still read it.
//   dQ pass (448 columns): S and dP have two buffers; warps 0-3 take the even entries, warps 4-7 the odd ones.
//       SS(0) SS(1) | TS(0) SS(2) | TS(1) SS(3) | ...        TS(s) after x_full(s), which also frees S/dP of entry s
//   dK/dV pass (512 columns, two accumulators): S^T and dP^T have ONE buffer; all eight warps work on every entry (warps
//       0-3 columns 0-31, warps 4-7 columns 32-63) and release the buffer as soon as they hold it in registers (s_free).
//       SS(0) | SS(1) TS(0) | SS(2) TS(1) | ...               SS(s+1) after s_free(s),  TS(s) after x_full(s)
// Every mbarrier wait is bounded; when one runs out the CTA flags the status word, drains its copies, frees TMEM, returns.
#include <cstdlib>
#include <cstring>

#include "tc_common.cuh"

namespace lcbsa {

namespace {

using namespace tc;

constexpr int kD = 128;
constexpr int kBlk = 64;
constexpr int kTileBytes = kBlk * kD * 2;   // 16 KiB
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column half: 64 rows x 128 B, 128B-swizzled
constexpr int kSlotBytes = 2 * kTileBytes;  // a ring slot: the (B1, B2) tiles of one list entry
constexpr int kStatsFloats = 2 * kBlk;      // per 64-token query block: lse * log2(e) [64], delta [64]
constexpr int kStatsBytes = kStatsFloats * 4;
constexpr int kThreads = 384;
constexpr int kRegsMath = 208, kRegsOther = 88;  // setmaxnreg: (208 + 208 + 88) * 128 <= 64 K registers

// Shared memory, for own tiles of kM = 64 or 128 rows (the streamed tiles always have 64).
template <int kM> struct Lay {
    static constexpr int aTile = kM * kD * 2;        // 16 or 32 KiB: A1, A2
    static constexpr int aHalf = aTile / 2;          // one 64-column half: kM rows x 128 B, 128B-swizzled
    static constexpr int slots = kM == 64 ? 5 : 4;   // ring of (B1, B2) tile pairs
    static constexpr int offA = 0;
    static constexpr int offB = offA + 2 * aTile;
    static constexpr int offStats = offB + slots * kSlotBytes;  // per slot: lse2[64], delta[64] of the streamed query block
    static constexpr int offBar = offStats + slots * kStatsBytes;
    // barriers: a_full, full[slots], empty[slots], s_full[2], s_free, x_full[2], acc_done
    static constexpr int numBars = 1 + 2 * slots + 2 + 1 + 2 + 1;
    static constexpr int offMisc = offBar + numBars * 8;  // abort flag, TMEM base
    static constexpr int smem = offMisc + 64;
};

// TMEM columns.  dQ pass: dQ 0..127, S[buf] 128 + 128 buf, dP[buf] 192 + 128 buf, dS[buf] 384 + 32 buf.
// dK/dV pass: dK 0..127, dV 128..255, S^T 256..319, dP^T 320..383, P^T[buf] 384 + 64 buf, dS^T[buf] 416 + 64 buf.
template <int kMode> struct Cols;
template <> struct Cols<0> {
    static constexpr uint32_t acc1 = 0, acc2 = 0;
    __device__ static __forceinline__ uint32_t s(int buf) { return 128u + 128u * buf; }
    __device__ static __forceinline__ uint32_t dp(int buf) { return 192u + 128u * buf; }
    __device__ static __forceinline__ uint32_t xp(int buf) { return 384u + 32u * buf; }  // unused in this pass
    __device__ static __forceinline__ uint32_t xd(int buf) { return 384u + 32u * buf; }
};
template <> struct Cols<1> {
    static constexpr uint32_t acc1 = 0, acc2 = 128;
    __device__ static __forceinline__ uint32_t s(int) { return 256u; }
    __device__ static __forceinline__ uint32_t dp(int) { return 320u; }
    __device__ static __forceinline__ uint32_t xp(int buf) { return 384u + 64u * buf; }
    __device__ static __forceinline__ uint32_t xd(int buf) { return 416u + 64u * buf; }
};

struct BwdTcParams {
    CUtensorMap tm_a1, tm_a2, tm_b1, tm_b2;
    const int32_t* list;   // dQ pass: [BH][n_own][cap] key units per own block; dK/dV pass: [BH][list_stride] query units, by toff
    const int32_t* cnt;    // dQ pass: [BH][n_own]
    const int32_t* toff;   // dK/dV pass: [BH][n_own + 1]
    long long list_stride;
    const float* stats;    // dK/dV pass: [BH][n_stream][2][64] of the streamed 64-token query blocks
    const float* lse;      // dQ pass: [BH][Sq] natural log, of the own rows
    const float* delta;    // dQ pass: [BH][Sq]
    long long Sq;
    unsigned int* status;
    void* out1;            // dQ pass: dq; dK/dV pass: dk
    void* out2;            // dK/dV pass: dv
    long long o1_sb, o1_sh, o1_ss, o2_sb, o2_sh, o2_ss;  // element strides
    int cap, n_own, n_stream, heads;
    int merge_a1, merge_a2, merge_b1, merge_b2;  // how the batch axis is folded into each map
    Geom ga, gb;           // grid of the CTA's own tiles (blocks of 64 or 128 tokens), grid of the streamed 64-token tiles
    float scale, scale2;   // sm_scale, sm_scale * log2(e)
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// the two 64-column boxes of one [64 tokens x 128] tile
__device__ __forceinline__ void load_tile_pair(uint32_t dst, const CUtensorMap* tm, uint32_t bar, const Coord& c) {
    tma_load_5d(dst, tm, bar, 0, c.c1, c.c2, c.c3, c.c4);
    tma_load_5d(dst + kHalfBytes, tm, bar, 64, c.c1, c.c2, c.c3, c.c4);
}

// lse * log2(e) and delta of every query row, laid out per 64-token block in slot order, so that a block's 128 values are
// one contiguous 512-byte piece.  Slots of a partial block that lie outside the grid get zeros (their q and dO rows are
// zero-filled by TMA, so every term they enter is a finite number times zero).
__global__ void __launch_bounds__(256) bwd_stats_kernel(const float* lse, const float* delta, Geom g, long long Sq, long long total,
                                                        float* stats) {
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= total) return;
    const int r = (int)(p % kBlk);
    const long long rest = p / kBlk;
    const int blk = (int)(rest % g.nblk);
    const long long bh = rest / g.nblk;
    int lt, lh, lw, bt, bhh, bw;
    slot_coords(g, r, lt, lh, lw);
    block_coords(g, blk, bt, bhh, bw);
    const int tt = bt * g.ct + lt, hh = bhh * g.ch + lh, ww = bw * g.cw + lw;
    const bool inside = tt < g.T && hh < g.H && ww < g.W;
    const long long tok = ((long long)tt * g.H + hh) * g.W + ww;
    float* dst = stats + (bh * g.nblk + blk) * kStatsFloats;
    dst[r] = inside ? lse[bh * Sq + tok] * 1.4426950408889634f : 0.f;
    dst[kBlk + r] = inside ? delta[bh * Sq + tok] : 0.f;
}

// 32 columns of this thread's accumulator row -> 64 bytes of the row in global memory (input dtype)
template <bool kBf16>
__device__ __forceinline__ void store_row32(unsigned char* row_ptr, int col0, const uint32_t (&r)[32]) {
#pragma unroll
    for (int q8 = 0; q8 < 4; ++q8) {
        uint4 pk;
        pk.x = pack2(kBf16, __uint_as_float(r[q8 * 8 + 0]), __uint_as_float(r[q8 * 8 + 1]));
        pk.y = pack2(kBf16, __uint_as_float(r[q8 * 8 + 2]), __uint_as_float(r[q8 * 8 + 3]));
        pk.z = pack2(kBf16, __uint_as_float(r[q8 * 8 + 4]), __uint_as_float(r[q8 * 8 + 5]));
        pk.w = pack2(kBf16, __uint_as_float(r[q8 * 8 + 6]), __uint_as_float(r[q8 * 8 + 7]));
        *reinterpret_cast<uint4*>(row_ptr + (col0 + q8 * 8) * 2) = pk;
    }
}

// kMode 0: dQ pass, 1: dK/dV pass.  Grid: (blocks of the CTA's own grid, batch * heads).
template <bool kBf16, int kMode, int kM>
__global__ void __launch_bounds__(kThreads, 1) bwd_tc_kernel(const __grid_constant__ BwdTcParams P) {
    using C = Cols<kMode>;
    using Ly = Lay<kM>;
    constexpr int kSlots = Ly::slots, kOffA = Ly::offA, kOffB = Ly::offB, kOffStats = Ly::offStats, kOffBar = Ly::offBar, kOffMisc = Ly::offMisc;
    constexpr int kATile = Ly::aTile, kAHalf = Ly::aHalf;
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kOffBar;
    const uint32_t bar_a_full = bar0;
    auto bar_full = [&](int s) { return bar0 + 8u * (1 + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (1 + kSlots + s); };
    auto bar_s_full = [&](int buf) { return bar0 + 8u * (1 + 2 * kSlots + (kMode == 0 ? buf : 0)); };
    const uint32_t bar_s_free = bar0 + 8u * (3 + 2 * kSlots);
    auto bar_x_full = [&](int buf) { return bar0 + 8u * (4 + 2 * kSlots + buf); };
    const uint32_t bar_acc_done = bar0 + 8u * (6 + 2 * kSlots);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffMisc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffMisc + 8);
    const Ctl ctl{abort_flag, P.status};

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // provably warp-uniform
    const int own = blockIdx.x;                              // block of the CTA's own grid
    const int bh = blockIdx.y, b = bh / P.heads, h = bh % P.heads;

    // this CTA's list
    const int32_t* list;
    int n;
    if (kMode == 0) {
        list = P.list + ((long long)bh * P.n_own + own) * P.cap;
        n = min(max(P.cnt[(long long)bh * P.n_own + own], 0), P.cap);
    } else {
        const int lo = P.toff[(long long)bh * (P.n_own + 1) + own], hi = P.toff[(long long)bh * (P.n_own + 1) + own + 1];
        list = P.list + (long long)bh * P.list_stride + lo;
        n = max(hi - lo, 0);
    }

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar_a_full, 1);
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        mbar_init(bar0 + 8u * (1 + 2 * kSlots), 1);  // s_full[0], s_full[1]
        mbar_init(bar0 + 8u * (2 + 2 * kSlots), 1);
        mbar_init(bar_s_free, 8);  // one elected arrival per arithmetic warp
        mbar_init(bar_x_full(0), kMode == 0 ? 4 : 8);  // the warps that work on an entry
        mbar_init(bar_x_full(1), kMode == 0 ? 4 : 8);
        mbar_init(bar_acc_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the tiles are 128B-swizzled, which ties their layout to address bits 7-9: refuse to run on an unaligned base
        if (sbase & 1023u) {
            *abort_flag = 1;
            if (atomicCAS(P.status, 0u, 1u) == 0u) {
                P.status[1] = blockIdx.x;
                P.status[2] = sbase;
                P.status[3] = 0;
            }
        }
    }
    if (warp == 9) {  // TMEM: all 512 columns, allocated and freed by the issuing warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    if (*abort_flag != 0) n = -1;  // nothing runs, nothing is written

    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (warp == 8 && n > 0) {
            // ================================================================== TMA producer
            if (lane == 0) {
                // one box of kM rows per 64-column half (the own grid's block is the box)
                mbar_arrive_tx(bar_a_full, 2 * kATile);
                const Coord c1 = block_coord(P.ga, own, b, h, P.heads, P.merge_a1, P.ga.T), c2 = block_coord(P.ga, own, b, h, P.heads, P.merge_a2, P.ga.T);
                tma_load_5d(sbase + kOffA, &P.tm_a1, bar_a_full, 0, c1.c1, c1.c2, c1.c3, c1.c4);
                tma_load_5d(sbase + kOffA + kAHalf, &P.tm_a1, bar_a_full, 64, c1.c1, c1.c2, c1.c3, c1.c4);
                tma_load_5d(sbase + kOffA + kATile, &P.tm_a2, bar_a_full, 0, c2.c1, c2.c2, c2.c3, c2.c4);
                tma_load_5d(sbase + kOffA + kATile + kAHalf, &P.tm_a2, bar_a_full, 64, c2.c1, c2.c2, c2.c3, c2.c4);
            }
            bool ok = true;
            int win = 0, issued = 0;
            for (int s = 0; s < n; ++s) {
                if ((s & 31) == 0) win = (s + lane < n) ? list[s + lane] : 0;
                const int blk = __shfl_sync(0xffffffffu, win, s & 31);
                const int slot = s % kSlots;
                ok = mbar_wait_warp(bar_empty(slot), ((s / kSlots) & 1) ^ 1, ctl, 210 + kMode, s);
                if (!ok) break;
                ++issued;
                if (lane == 0) {
                    mbar_arrive_tx(bar_full(slot), 2 * kTileBytes + (kMode == 1 ? kStatsBytes : 0));
                    Coord c1, c2;
                    if ((unsigned)blk < (unsigned)P.gb.nblk) {
                        c1 = block_coord(P.gb, blk, b, h, P.heads, P.merge_b1, P.gb.T);
                        c2 = block_coord(P.gb, blk, b, h, P.heads, P.merge_b2, P.gb.T);
                    } else {
                        // an entry outside the grid never becomes an address: the box is placed at w = W, wholly outside
                        // the map, and TMA fills the tiles with zeros (the list transposition has flagged the call)
                        c1 = Coord{P.gb.W, 0, 0, 0};
                        c2 = c1;
                    }
                    const uint32_t dst = sbase + kOffB + slot * kSlotBytes;
                    load_tile_pair(dst, &P.tm_b1, bar_full(slot), c1);
                    load_tile_pair(dst + kTileBytes, &P.tm_b2, bar_full(slot), c2);
                    if (kMode == 1)  // transposed lists only hold blocks of the grid
                        bulk_load(sbase + kOffStats + slot * kStatsBytes, P.stats + ((long long)bh * P.n_stream + blk) * kStatsFloats, kStatsBytes,
                                  bar_full(slot));
                }
                __syncwarp();
            }
            if (!ok && lane == 0) {
                // drain: give the copies this warp issued a bounded time to land before the CTA exits
                const long long t0 = clock64();
                while (!mbar_try(bar_a_full, 0) && clock64() - t0 < 40000000ll) {
                }
                for (int r = issued > kSlots ? issued - kSlots : 0; r < issued; ++r)
                    while (!mbar_try(bar_full(r % kSlots), (r / kSlots) & 1) && clock64() - t0 < 40000000ll) {
                    }
            }
        } else if (warp == 9 && n > 0) {
            // ================================================================== MMA issuer
            const uint32_t idesc_ss = instr_desc(kBf16, kM, 64, 0), idesc_ts = instr_desc(kBf16, kM, 128, 1);
            const uint64_t a1d = smem_desc(sbase + kOffA, 16, 1024), a2d = smem_desc(sbase + kOffA + kATile, 16, 1024);
            bool ok = mbar_wait_warp(bar_a_full, 0, ctl, 220 + kMode, 0);
            // S (or S^T) and dP (or dP^T) of entry s
            auto issue_ss = [&](int s) -> bool {
                const int slot = s % kSlots, buf = s & 1;
                if (!mbar_wait_warp(bar_full(slot), (s / kSlots) & 1, ctl, 222 + kMode, s)) return false;
                // dK/dV pass: the arithmetic warps hold S^T and dP^T of entry s - 1 in registers.  (dQ pass: the buffer
                // was entry s - 2's, whose x_full the issuer has seen before TS(s - 2).)
                if (kMode == 1 && s > 0 && !mbar_wait_warp(bar_s_free, (s - 1) & 1, ctl, 226, s)) return false;
                tc_fence_after();
                const uint32_t tile = sbase + kOffB + slot * kSlotBytes;
                const uint64_t b1d = smem_desc(tile, 16, 1024), b2d = smem_desc(tile + kTileBytes, 16, 1024);
#pragma unroll
                for (int j = 0; j < kD / 16; ++j) {
                    // 32 bytes per 16-column step inside a 64-column half; the halves are kM x 128 B (own tile) and 8 KiB
                    // (streamed tile) apart
                    const uint64_t aoff = (uint64_t)(((j >> 2) * kAHalf + (j & 3) * 32) >> 4);
                    const uint64_t off = (uint64_t)(((j >> 2) * kHalfBytes + (j & 3) * 32) >> 4);
                    tc_mma(tmem + C::s(buf), a1d + aoff, b1d + off, idesc_ss, j > 0);
                }
#pragma unroll
                for (int j = 0; j < kD / 16; ++j) {
                    const uint64_t aoff = (uint64_t)(((j >> 2) * kAHalf + (j & 3) * 32) >> 4);
                    const uint64_t off = (uint64_t)(((j >> 2) * kHalfBytes + (j & 3) * 32) >> 4);
                    tc_mma(tmem + C::dp(buf), a2d + aoff, b2d + off, idesc_ss, j > 0);
                }
                tc_commit(bar_s_full(buf));
                return true;
            };
            // the gradient MMAs of entry e: A from TMEM (8 columns per 16-row step), B the streamed tile, MN-major
            // (64-column halves 8 KiB apart = LBO, 8-row groups 1 KiB apart = SBO, 16 rows = 2 KiB per step)
            auto issue_ts = [&](int e) -> bool {
                const int slot = e % kSlots, buf = e & 1;
                if (!mbar_wait_warp(bar_x_full(buf), (e >> 1) & 1, ctl, 224 + kMode, e)) return false;
                tc_fence_after();
                const uint32_t tile = sbase + kOffB + slot * kSlotBytes;
                const uint64_t b1m = smem_desc(tile, kHalfBytes, 1024), b2m = smem_desc(tile + kTileBytes, kHalfBytes, 1024);
                if (kMode == 1) {
#pragma unroll
                    for (int j = 0; j < kBlk / 16; ++j)  // dV += P^T dO
                        tc_mma_ts(tmem + C::acc2, tmem + C::xp(buf) + 8u * j, b2m + (uint64_t)((j * 2048) >> 4), idesc_ts, (e > 0 || j > 0) ? 1u : 0u);
                }
#pragma unroll
                for (int j = 0; j < kBlk / 16; ++j)  // dQ += dS K, or dK += dS^T Q
                    tc_mma_ts(tmem + C::acc1, tmem + C::xd(buf) + 8u * j, b1m + (uint64_t)((j * 2048) >> 4), idesc_ts, (e > 0 || j > 0) ? 1u : 0u);
                tc_commit(bar_empty(slot));  // the streamed tiles are free once these MMAs have read them
                if (e == n - 1) tc_commit(bar_acc_done);
                return true;
            };
            if (ok) ok = issue_ss(0);
            if (kMode == 0) {
                if (ok && n > 1) ok = issue_ss(1);
                for (int i = 0; i < n && ok; ++i) {
                    ok = issue_ts(i);
                    if (ok && i + 2 < n) ok = issue_ss(i + 2);
                }
            } else {
                for (int i = 0; i < n && ok; ++i) {
                    if (i + 1 < n) ok = issue_ss(i + 1);
                    if (ok) ok = issue_ts(i);
                }
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsMath));
        // ================================================================== arithmetic warps
        const int wg = warp >> 2;  // dQ pass: entries wg, wg + 2, ...; dK/dV pass: columns 32 wg .. 32 wg + 31 of every entry
        const int wq = warp & 3;   // TMEM quadrant of this warp
        // row of the own tile = TMEM lane.  An M=128 accumulator has row r in lane r; an M=64 one occupies lanes 0-15 of every
        // 32-lane quadrant (lanes 16-31 of a warp then shadow lanes 0-15 on TMEM lanes that nothing reads)
        const int row = kM == 128 ? wq * 32 + lane : wq * 16 + (lane & 15);
        const uint32_t t_lane = (uint32_t)(wq * 32) << 16;
        // the token of this row (rows of a block are its tokens in t, h, w order)
        // A row of a partial block that lies outside the grid is computed on zero-filled operands and never stored.
        long long tok;
        bool row_inside;
        {
            int lt, lh, lw, bt, bhh, bw;
            slot_coords(P.ga, row, lt, lh, lw);
            block_coords(P.ga, own, bt, bhh, bw);
            const int tt = bt * P.ga.ct + lt, hh = bhh * P.ga.ch + lh, ww = bw * P.ga.cw + lw;
            row_inside = tt < P.ga.T && hh < P.ga.H && ww < P.ga.W;
            tok = ((long long)tt * P.ga.H + hh) * P.ga.W + ww;
        }
        // dQ pass: this thread's query row has one lse and one delta for the whole list
        float my_l2 = 0.f, my_dl = 0.f;
        if (kMode == 0 && n > 0 && row_inside) {
            my_l2 = P.lse[(long long)bh * P.Sq + tok] * 1.4426950408889634f;
            my_dl = P.delta[(long long)bh * P.Sq + tok];
        }
        // 32 columns of S and dP -> 16 columns of P and of dS in the input dtype.  st4: the slot's lse and delta values
        // of those 32 columns (dK/dV pass, where columns are query rows)
        auto columns32 = [&](const uint32_t (&sr)[32], const uint32_t (&dr)[32], const float4* l4, const float4* d4, uint32_t* xp, uint32_t* xd) {
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
                float4 l2 = make_float4(my_l2, my_l2, my_l2, my_l2), dl = make_float4(my_dl, my_dl, my_dl, my_dl);
                if (kMode == 1) {
                    l2 = l4[c4];
                    dl = d4[c4];
                }
                const float p0 = ex2(fmaf(__uint_as_float(sr[4 * c4 + 0]), P.scale2, -l2.x));
                const float p1 = ex2(fmaf(__uint_as_float(sr[4 * c4 + 1]), P.scale2, -l2.y));
                const float p2 = ex2(fmaf(__uint_as_float(sr[4 * c4 + 2]), P.scale2, -l2.z));
                const float p3 = ex2(fmaf(__uint_as_float(sr[4 * c4 + 3]), P.scale2, -l2.w));
                const float g0 = p0 * (__uint_as_float(dr[4 * c4 + 0]) - dl.x) * P.scale;
                const float g1 = p1 * (__uint_as_float(dr[4 * c4 + 1]) - dl.y) * P.scale;
                const float g2 = p2 * (__uint_as_float(dr[4 * c4 + 2]) - dl.z) * P.scale;
                const float g3 = p3 * (__uint_as_float(dr[4 * c4 + 3]) - dl.w) * P.scale;
                if (kMode == 1) {
                    xp[2 * c4] = pack2(kBf16, p0, p1);
                    xp[2 * c4 + 1] = pack2(kBf16, p2, p3);
                }
                xd[2 * c4] = pack2(kBf16, g0, g1);
                xd[2 * c4 + 1] = pack2(kBf16, g2, g3);
            }
        };
        bool ok = true;
        if (kMode == 0) {
            unsigned r = 0;
            for (int i = wg; i < n && ok; i += 2, ++r) {  // buffer i & 1 = wg
                ok = mbar_wait_warp(bar_s_full(wg), r & 1, ctl, 230 + wg, i);
                if (!ok) break;
                tc_fence_after();
                uint32_t xd[32];
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    uint32_t sr[32], dr[32];
                    tc_ld32(tmem + C::s(wg) + 32u * half + t_lane, sr);
                    tc_ld32(tmem + C::dp(wg) + 32u * half + t_lane, dr);
                    tc_wait_ld();
                    columns32(sr, dr, nullptr, nullptr, nullptr, xd + 16 * half);
                }
                tc_st32(tmem + C::xd(wg) + t_lane, xd);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive_elect(bar_x_full(wg));
            }
        } else {
            for (int i = 0; i < n && ok; ++i) {
                const int slot = i % kSlots, buf = i & 1;
                ok = mbar_wait_warp(bar_s_full(0), i & 1, ctl, 232 + wg, i);
                // the slot's lse and delta values came with its tiles (a completed phase answers at once)
                if (ok) ok = mbar_wait_warp(bar_full(slot), (i / kSlots) & 1, ctl, 234 + wg, i);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[32], dr[32];
                tc_ld32(tmem + C::s(0) + 32u * wg + t_lane, sr);
                tc_ld32(tmem + C::dp(0) + 32u * wg + t_lane, dr);
                tc_wait_ld();
                tc_fence_before();
                mbar_arrive_elect(bar_s_free);  // S^T and dP^T may be overwritten by the next entry's
                const float4* st4 = reinterpret_cast<const float4*>(smem + kOffStats + slot * kStatsBytes);
                uint32_t xp[16], xd[16];
                columns32(sr, dr, st4 + wg * 8, st4 + 16 + wg * 8, xp, xd);
                // 32 columns of the tile are 16 columns of 16-bit pairs
                tc_st16(tmem + C::xp(buf) + 16u * wg + t_lane, xp);
                tc_st16(tmem + C::xd(buf) + 16u * wg + t_lane, xd);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive_elect(bar_x_full(buf));
            }
        }

        // ---- the accumulated gradients of the CTA's 64 rows: TMEM -> registers -> global memory (rows in T,H,W order)
        if (n >= 0) {
            if (n > 0 && ok) {
                ok = mbar_wait_warp(bar_acc_done, 0, ctl, 240 + kMode, n);
                tc_fence_after();
            }
            if (ok) {
                // dQ pass: warpgroup g stores columns 64 g .. 64 g + 63 of dQ; dK/dV pass: warpgroup 0 stores dK, 1 dV
                const bool second = kMode == 1 && wg == 1;
                unsigned char* base = static_cast<unsigned char*>(second ? P.out2 : P.out1);
                const long long sb = second ? P.o2_sb : P.o1_sb, sh = second ? P.o2_sh : P.o1_sh, ss = second ? P.o2_ss : P.o1_ss;
                unsigned char* row_ptr = base + ((long long)b * sb + (long long)h * sh + tok * ss) * 2;
                const uint32_t t_acc = tmem + (second ? C::acc2 : C::acc1) + t_lane;
                const int col_lo = kMode == 0 ? 64 * wg : 0, n_chunks = kMode == 0 ? 2 : 4;
#pragma unroll 1
                for (int ch = 0; ch < n_chunks; ++ch) {
                    uint32_t acc[32];
                    if (n > 0) {
                        tc_ld32(t_acc + col_lo + 32 * ch, acc);
                        tc_wait_ld();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) acc[j] = 0u;  // nothing selected this block: its gradient is zero
                    }
                    if ((kM == 128 || lane < 16) && row_inside) store_row32<kBf16>(row_ptr, col_lo + 32 * ch, acc);
                }
            }
        }
    }

    // ---- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}

template <bool kBf16, int kMode, int kM>
cudaError_t launch_pass(const BwdTcParams& P, unsigned own_blocks, unsigned BH, cudaStream_t st) {
    // the attribute is per device and per kernel; setting it on every call costs a microsecond and keeps this stateless
    cudaError_t e = cudaFuncSetAttribute(bwd_tc_kernel<kBf16, kMode, kM>, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay<kM>::smem);
    if (e != cudaSuccess) return e;
    bwd_tc_kernel<kBf16, kMode, kM><<<dim3(own_blocks, BH), kThreads, Lay<kM>::smem, st>>>(P);
    return cudaGetLastError();
}

template <int kMode>
cudaError_t launch_pass_any(bool bf16, int rows, const BwdTcParams& P, unsigned own_blocks, unsigned BH, cudaStream_t st) {
    if (rows == 128) return bf16 ? launch_pass<true, kMode, 128>(P, own_blocks, BH, st) : launch_pass<false, kMode, 128>(P, own_blocks, BH, st);
    return bf16 ? launch_pass<true, kMode, 64>(P, own_blocks, BH, st) : launch_pass<false, kMode, 64>(P, own_blocks, BH, st);
}

bool grid_fits(const Geom& g, int rows) { return g.bs == rows && g.ct <= 256 && g.ch <= 256 && g.cw <= 256; }

}  // namespace

bool attn_bwd_tc_supported(const BwdArgs& a, const BwdTcPlan& p) {
    const char* force = std::getenv("LCBSA_BWD_IMPL");  // "mma" keeps the warp-level kernels (for comparisons)
    if (force && std::strcmp(force, "mma") == 0) return false;
    if (a.dtype != LCBSA_BF16 && a.dtype != LCBSA_FP16) return false;
    if (a.D != kD) return false;
    if (!grid_fits(p.unit_q, 64) || !grid_fits(p.unit_k, 64)) return false;
    if ((p.unit_q.ragged || p.unit_k.ragged) && a.dtype != LCBSA_BF16) return false;  // see the note on ragged grids above
    if (!grid_fits(p.own_q, 64) && !grid_fits(p.own_q, 128)) return false;
    if (!grid_fits(p.own_k, 64) && !grid_fits(p.own_k, 128)) return false;
    if (encode_fn() == nullptr) return false;
    const View* vs[4] = {&a.q, &a.dout, &a.k, &a.v};
    const Geom* gs[8] = {&p.own_q, &p.own_q, &p.own_k, &p.own_k, &p.unit_q, &p.unit_q, &p.unit_k, &p.unit_k};
    for (int i = 0; i < 8; ++i) {
        const View& v = *vs[i % 4];
        if (merge_mode(v, a.B, a.H, *gs[i]) < 0) return false;
        if (v.ss * 2 >= (1ll << 40) || v.sh * 2 >= (1ll << 40)) return false;
    }
    return true;
}

// a.delta, the lists of the plan and (for the dK/dV pass) their transposition are ready on the stream; a.stats is scratch
// of B*H*Sq*2 floats
cudaError_t launch_attn_bwd_tc(const BwdArgs& a, const BwdTcPlan& p, cudaStream_t st, const char** why) {
    const long long Sq = (long long)a.gq.T * a.gq.H * a.gq.W;
    const long long BH = (long long)a.B * a.H;
    {
        const long long total = BH * p.unit_q.nblk * kBlk;  // every slot of every 64-token query unit
        bwd_stats_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(a.lse, a.delta, p.unit_q, Sq, total, a.stats);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    // maps: q and dout with the boxes of the dQ pass's own blocks and of the streamed query units; k and v likewise
    const int m_q_own = merge_mode(a.q, a.B, a.H, p.own_q), m_do_own = merge_mode(a.dout, a.B, a.H, p.own_q);
    const int m_q_u = merge_mode(a.q, a.B, a.H, p.unit_q), m_do_u = merge_mode(a.dout, a.B, a.H, p.unit_q);
    const int m_k_own = merge_mode(a.k, a.B, a.H, p.own_k), m_v_own = merge_mode(a.v, a.B, a.H, p.own_k);
    const int m_k_u = merge_mode(a.k, a.B, a.H, p.unit_k), m_v_u = merge_mode(a.v, a.B, a.H, p.unit_k);
    BwdTcParams P;
    std::memset(&P, 0, sizeof(P));
    P.stats = a.stats;
    P.lse = a.lse;
    P.delta = a.delta;
    P.Sq = Sq;
    P.status = a.status;
    P.heads = a.H;
    P.scale = a.sm_scale;
    P.scale2 = a.sm_scale * 1.4426950408889634f;
    const bool bf16 = a.dtype == LCBSA_BF16;

    // dQ pass: own tiles Q_i, dO_i (a query block of 64 or 128 tokens); streamed K_j, V_j (64-token units)
    if (!make_map(&P.tm_a1, a.dtype, a.q, a.B, a.H, p.own_q, m_q_own) || !make_map(&P.tm_a2, a.dtype, a.dout, a.B, a.H, p.own_q, m_do_own) ||
        !make_map(&P.tm_b1, a.dtype, a.k, a.B, a.H, p.unit_k, m_k_u) || !make_map(&P.tm_b2, a.dtype, a.v, a.B, a.H, p.unit_k, m_v_u)) {
        *why = "cuTensorMapEncodeTiled rejected a tensor";
        return cudaErrorInvalidValue;
    }
    P.merge_a1 = m_q_own; P.merge_a2 = m_do_own; P.merge_b1 = m_k_u; P.merge_b2 = m_v_u;
    P.ga = p.own_q; P.gb = p.unit_k;
    P.list = p.list_q; P.cnt = p.cnt_q; P.cap = p.cap_q; P.toff = nullptr; P.list_stride = 0;
    P.n_own = p.own_q.nblk; P.n_stream = p.unit_k.nblk;
    P.out1 = const_cast<void*>(a.dq.data); P.o1_sb = a.dq.sb; P.o1_sh = a.dq.sh; P.o1_ss = a.dq.ss;
    P.out2 = nullptr;
    cudaError_t e = launch_pass_any<0>(bf16, p.own_q.bs, P, (unsigned)p.own_q.nblk, (unsigned)BH, st);
    if (e != cudaSuccess) return e;

    // dK/dV pass: own tiles K_j, V_j (a key block of 64 or 128 tokens); streamed Q_i, dO_i (64-token units)
    if (!make_map(&P.tm_a1, a.dtype, a.k, a.B, a.H, p.own_k, m_k_own) || !make_map(&P.tm_a2, a.dtype, a.v, a.B, a.H, p.own_k, m_v_own) ||
        !make_map(&P.tm_b1, a.dtype, a.q, a.B, a.H, p.unit_q, m_q_u) || !make_map(&P.tm_b2, a.dtype, a.dout, a.B, a.H, p.unit_q, m_do_u)) {
        *why = "cuTensorMapEncodeTiled rejected a tensor";
        return cudaErrorInvalidValue;
    }
    P.merge_a1 = m_k_own; P.merge_a2 = m_v_own; P.merge_b1 = m_q_u; P.merge_b2 = m_do_u;
    P.ga = p.own_k; P.gb = p.unit_q;
    P.list = p.tidx; P.cnt = nullptr; P.cap = 0; P.toff = p.toff; P.list_stride = p.tidx_stride;
    P.n_own = p.own_k.nblk; P.n_stream = p.unit_q.nblk;
    P.out1 = const_cast<void*>(a.dk.data); P.o1_sb = a.dk.sb; P.o1_sh = a.dk.sh; P.o1_ss = a.dk.ss;
    P.out2 = const_cast<void*>(a.dv.data); P.o2_sb = a.dv.sb; P.o2_sh = a.dv.sh; P.o2_ss = a.dv.ss;
    return launch_pass_any<1>(bf16, p.own_k.bs, P, (unsigned)p.own_k.nblk, (unsigned)BH, st);
}

}  // namespace lcbsa
