// Block-sparse flash-attention forward for sm_100a, 128-token blocks: TMA + tcgen05 + TMEM.
//
// The block shape that flash_attn_bsa_3d takes by default (chunk_3d_shape = [4, 4, 8], bsa_interface.py:619-622),
// for which the reference launches _attn_fwd_bsa_varlen_align with BLOCK_M = BLOCK_N_LG = 128
// (flash_attn_bsa_varlen_mask.py:172-285, launcher bsa_interface.py:290-341).  Same contract as attn_tc.cu (the
// 64-token kernel): q, k, v are read and the output is written straight from / to T,H,W order by 5-D TMA boxes.
//
// Shape handled: head_dim 128, query blocks of 128 tokens, key blocks of 128, 256 or 512 tokens (for which the
// reference switches to _attn_fwd_bsa_varlen, flash_attn_bsa_varlen_mask.py:37-153, bsa_interface.py:309-315), bf16 or fp16.
//
// One persistent CTA per SM.  A work item is ONE query block of one head: a 128-row tile, i.e. M=128 tcgen05 MMAs
// that run the tensor pipe at its full rate (the 64-row tiles of the other kernel occupy it like 128-row ones).  A
// selected key block is processed as 2, 4 or 8 units of 64 keys (sub-boxes of the block, cut along its outermost even
// axes), which keeps the S tile at 64 TMEM columns, so that every warpgroup has two S/P buffers beside its O
// accumulator, exactly as in the 64-token kernel:
//
//   warps 0-3, 4-7 : softmax warpgroups 0 and 1 (units of even / odd number; thread = one query row)
//   warp 8 : TMA producer (Q tile, K ring, V ring)   warp 9 : S = Q K^T issuer   warp 10 : O += P V issuer
//   warp 11: output TMA stores
//
// Per unit i (warpgroup g = i & 1, its round r = i >> 1):  S = Q K^T (M128 N64 K128, buffer r & 1 of the warpgroup)
// -> tcgen05.ld, exp2 online softmax in registers, P in the input dtype over the first half of the same buffer ->
// O_g += P V (M128 N128 K64, A from TMEM).  The two warpgroups keep separate maxima, row sums and accumulators and
// are merged once per work item.  K and V rings: six slots of one 64-key tile (16 KiB) each.  The finished O
// (128 rows x 256 B) is staged in the V slots of the item's last two units and leaves by TMA store.
//
// Every wait on an mbarrier is bounded, as in attn_tc.cu.
#include "tc_common.cuh"


namespace lcbsa {

namespace {

using namespace tc;

constexpr int kD = 128;
constexpr int kQRows = 128;                        // tokens per query block: one M=128 tile
constexpr int kBlk = 64;                           // keys per unit: a key block is 2, 4 or 8 units
constexpr int kQTileBytes = kQRows * kD * 2;       // 32 KiB: the Q tile, and the staged O tile
constexpr int kQHalfBytes = kQTileBytes / 2;       // one 64-column half of it: 128 rows x 128 B, 128B-swizzled
constexpr int kTileBytes = kBlk * kD * 2;          // 16 KiB: one K or V tile of 64 keys
constexpr int kHalfBytes = kTileBytes / 2;         // one 64-column half: 64 rows x 128 B
constexpr int kSlotBytes = kTileBytes;             // a ring slot holds one unit's tile
constexpr int kMaxUnits = 8;                       // units of 64 keys per key block: blocks of up to 512 tokens
constexpr int kKSlots = 6, kVSlots = 6;            // even, like the number of units of an item: the last two units sit in a slot pair
constexpr int kKLead = 4;                          // K units requested ahead of V: S runs two rounds of each warpgroup ahead
constexpr int kThreads = 384;
// setmaxnreg per warpgroup: (208 + 208 + 88) * 128 threads <= the 64 K registers of the SM
constexpr int kRegsSoftmax = 208, kRegsOther = 88;

// TMEM columns of warpgroup g: base 256 * g
constexpr uint32_t kTmWg = 256, kTmS = 0, kTmO = 128;

// shared memory map (offsets from the 1024-byte aligned base of dynamic shared memory)
constexpr int kOffQ = 0;
constexpr int kOffK = kOffQ + kQTileBytes;
constexpr int kOffV = kOffK + kKSlots * kSlotBytes;
constexpr int kOffBar = kOffV + kVSlots * kSlotBytes;
// barriers: k_full[6] k_empty[6] v_full[6] v_empty[6] q_full q_empty s_full[2][2] p_full[2][2] pv_done[2][2]
//           ml_ready o_free o_staged
constexpr int kNumBars = 2 * kKSlots + 2 * kVSlots + 2 + 12 + 3;
constexpr int kOffMisc = kOffBar + kNumBars * 8;      // abort flag, TMEM base
constexpr int kOffMl = kOffMisc + 64;                 // [2 warpgroups][128 lanes] (maximum, row sum)
constexpr int kSmemBytes = kOffMl + 2 * 128 * 8;

struct TcParams {
    CUtensorMap tm_q, tm_k, tm_v;
    // Output maps.  Normally one (tm_o[0]).  With o_frames > 0 the query grid is the rank-major grid of a
    // context-parallel group: frames [r * o_frames, (r + 1) * o_frames) are the tokens of rank r, and the rows of a
    // query block are stored straight into rank r's result buffer (its own map, over this GPU's or a peer's memory).
    CUtensorMap tm_o[kMaxOutDst];
    int o_frames;
    const int32_t* idx;
    const int32_t* cnt;
    float* lse;
    unsigned int* status;
    int cap;
    int nq;         // query blocks per head
    int bh_total;   // B*H
    int heads;      // H
    int merge_q, merge_k, merge_v, merge_o;  // 0: batch folded into the head axis of the map, 1: into the T axis
    int Tq, Tk;     // frames (for merge == 1 coordinates)
    Geom gq, gk;
    float scale2;   // sm_scale * log2(e)
    int is_bf16;
    // A key block of 128, 256 or 512 tokens is cut into 2, 4 or 8 units of 64 keys: unit u of a block starts
    // (sub_t[u], sub_h[u], sub_w[u]) tokens into it.  lg_units = log2 of the units per block.
    int lg_units;
    int sub_t[kMaxUnits], sub_h[kMaxUnits], sub_w[kMaxUnits];
    Geom gu;                // the key geometry with the block shape replaced by the unit's: slot order inside a unit
};

// ------------------------------------------------------------------------------------------ kernel

__device__ __forceinline__ int clamp_cnt(const TcParams& P, int bh, int qt) {
    return qt < P.nq ? min(max(P.cnt[(long long)bh * P.nq + qt], 0), P.cap) : 0;
}

// kRagged: the key grid has partial blocks.  The masking code exists only in that instantiation, which keeps the
// instruction stream of the softmax loop of whole grids short (the loop is sensitive to instruction fetch).
template <bool kBf16, bool kRagged>
__global__ void __launch_bounds__(kThreads, 1) attn_tc128_kernel(const __grid_constant__ TcParams P) {
    extern __shared__ __align__(1024) unsigned char smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kOffBar;
    auto bar_k_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_k_empty = [&](int s) { return bar0 + 8u * (kKSlots + s); };
    auto bar_v_full = [&](int s) { return bar0 + 8u * (2 * kKSlots + s); };
    auto bar_v_empty = [&](int s) { return bar0 + 8u * (2 * kKSlots + kVSlots + s); };
    constexpr int kB0 = 2 * kKSlots + 2 * kVSlots;
    const uint32_t bar_q_full = bar0 + 8u * kB0, bar_q_empty = bar0 + 8u * (kB0 + 1);
    auto bar_s_full = [&](int wg, int buf) { return bar0 + 8u * (kB0 + 2 + 2 * wg + buf); };
    auto bar_p_full = [&](int wg, int buf) { return bar0 + 8u * (kB0 + 6 + 2 * wg + buf); };
    auto bar_pv_done = [&](int wg, int buf) { return bar0 + 8u * (kB0 + 10 + 2 * wg + buf); };
    const uint32_t bar_ml_ready = bar0 + 8u * (kB0 + 14), bar_o_free = bar0 + 8u * (kB0 + 15), bar_o_staged = bar0 + 8u * (kB0 + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffMisc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffMisc + 8);
    float2* ml = reinterpret_cast<float2*>(smem + kOffMl);  // [2][128]
    const Ctl ctl{abort_flag, P.status};

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // the same value, but provably warp-uniform

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kKSlots; ++s) {
            mbar_init(bar_k_full(s), 1);
            mbar_init(bar_k_empty(s), 1);
        }
        for (int s = 0; s < kVSlots; ++s) {
            mbar_init(bar_v_full(s), 1);
            mbar_init(bar_v_empty(s), 1);
        }
        mbar_init(bar_q_full, 1);
        mbar_init(bar_q_empty, 1);
        for (int g = 0; g < 2; ++g)
            for (int b = 0; b < 2; ++b) {
                mbar_init(bar_s_full(g, b), 1);
                mbar_init(bar_p_full(g, b), 4);  // one elected arrival per softmax warp
                mbar_init(bar_pv_done(g, b), 1);
            }
        mbar_init(bar_ml_ready, 8);
        mbar_init(bar_o_free, 8);
        mbar_init(bar_o_staged, 8);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The tiles are 128B-swizzled, which ties their layout to address bits 7-9: without a 1024-byte aligned
        // base nothing below is valid.  The declaration asks for it; refuse to run if it was not honoured.
        if (sbase & 1023u) {
            *abort_flag = 1;
            if (atomicCAS(P.status, 0u, 1u) == 0u) {
                P.status[1] = blockIdx.x;
                P.status[2] = sbase;
                P.status[3] = 0;
            }
        }
    }
    if (warp == 9) {  // TMEM: all 512 columns, allocated and freed by the S issuer
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    const bool start_ok = *abort_flag == 0;

    const int groups = P.nq;  // one work item per query block
    const long long total_work = start_ok ? (long long)P.bh_total * groups : 0;
    constexpr bool bf16 = kBf16;

    // All roles walk the same list of work items and units.  Unit number gb (counted over the whole kernel)
    // uses K slot gb % 6 and V slot gb % 6; warpgroup g numbers its own rounds rr[g] over the whole kernel and
    // round rr uses S/P buffer rr & 1.  Within an item unit i belongs to warpgroup i & 1.
    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
      if (warp == 8) {
        // ================================================================== TMA producer
        unsigned gk = 0, gv = 0, wk = 0, nq_issued = 0;
        bool ok = true;
        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), qb = (int)(w % groups);
            const int b = bh / P.heads, h = bh % P.heads;
            const int cnt = clamp_cnt(P, bh, qb);
            const int n_act = cnt << P.lg_units;  // units that exist: 2, 4 or 8 per listed key block
            const int n_iter = max(2, n_act);     // an empty list still goes through one (masked) pair of units
            // Q tile: the buffer is free once the last S of the previous item has been computed
            ok = mbar_wait_warp(bar_q_empty, (wk & 1) ^ 1, ctl, 10, wk);
            if (!ok) break;
            ++nq_issued;
            if (lane == 0) {
                mbar_arrive_tx(bar_q_full, kQTileBytes);
                const Coord cc = block_coord(P.gq, qb, b, h, P.heads, P.merge_q, P.Tq);
                tma_load_5d(sbase + kOffQ, &P.tm_q, bar_q_full, 0, cc.c1, cc.c2, cc.c3, cc.c4);
                tma_load_5d(sbase + kOffQ + kQHalfBytes, &P.tm_q, bar_q_full, 64, cc.c1, cc.c2, cc.c3, cc.c4);
            }
            // Block coordinates are fetched and decoded by the whole warp: lane L holds list entry win + L as the
            // block's first token packed t << 20 | h << 10 | w.  `prv` holds the window of thirty-two entries before
            // (V trails K by kKLead units).
            const int32_t* my_l = P.idx + ((long long)bh * P.nq + qb) * P.cap;
            auto fetch = [&](int e) {
                if (e >= cnt) return 0;
                const int blk = my_l[e];
                if ((unsigned)blk >= (unsigned)P.gk.nblk) {
                    // A list entry outside [0, Nk) never becomes an address: its box is placed at w = W, wholly
                    // outside the tensor map, so TMA fills the tile with zeros; the call is flagged.
                    if (atomicCAS(P.status, 0u, kStatusBadBlockIndex) == 0u) {
                        P.status[1] = bh;
                        P.status[2] = qb;
                        P.status[3] = e;
                    }
                    return P.gk.W;
                }
                int bt, bhh, bw;
                block_coords(P.gk, blk, bt, bhh, bw);
                return ((bt * P.gk.ct) << 20) | ((bhh * P.gk.ch) << 10) | (bw * P.gk.cw);
            };
            int win = 0, prv = 0;
            int cur = fetch(lane);
            const int c3k = P.merge_k ? b * P.Tk : 0, c4k = P.merge_k ? h : b * P.heads + h;
            const int c3v = P.merge_v ? b * P.Tk : 0, c4v = P.merge_v ? h : b * P.heads + h;
            // coordinates of unit u: those of its block plus the offset of the unit inside the block
            auto unit_coords = [&](int pk, int u, int& cw, int& chh, int& ctt) {
                cw = pk & 1023;
                chh = (pk >> 10) & 1023;
                ctt = pk >> 20;
                const int sub = u & ((1 << P.lg_units) - 1);
                ctt += P.sub_t[sub];
                chh += P.sub_h[sub];
                cw += P.sub_w[sub];
            };
            for (int j = 0; j < n_iter + kKLead && ok; ++j) {
                if (j >= kKLead) {  // V(j - kKLead)
                    const int jj = j - kKLead, e = jj >> P.lg_units;
                    const int pk = __shfl_sync(0xffffffffu, e >= win ? cur : prv, e >= win ? e - win : e - (win - 32));
                    const bool act = jj < n_act;
                    const int slot = gv % kVSlots;
                    ok = mbar_wait_warp(bar_v_empty(slot), ((gv / kVSlots) & 1) ^ 1, ctl, 22, gv);
                    if (!ok) break;
                    ++gv;
                    if (lane == 0) {
                        mbar_arrive_tx(bar_v_full(slot), act ? kTileBytes : 0);
                        if (act) {
                            int cw, chh, ctt;
                            unit_coords(pk, jj, cw, chh, ctt);
                            const uint32_t dst = sbase + kOffV + slot * kSlotBytes;
                            tma_load_5d(dst, &P.tm_v, bar_v_full(slot), 0, cw, chh, ctt + c3v, c4v);
                            tma_load_5d(dst + kHalfBytes, &P.tm_v, bar_v_full(slot), 64, cw, chh, ctt + c3v, c4v);
                        }
                    }
                }
                if (j < n_iter) {  // K(j)
                    const int e = j >> P.lg_units;
                    while (e >= win + 32) {
                        win += 32;
                        prv = cur;
                        cur = fetch(win + lane);
                    }
                    const int pk = __shfl_sync(0xffffffffu, cur, e - win);
                    const bool act = j < n_act;
                    const int slot = gk % kKSlots;
                    ok = mbar_wait_warp(bar_k_empty(slot), ((gk / kKSlots) & 1) ^ 1, ctl, 20, gk);
                    if (!ok) break;
                    ++gk;
                    if (lane == 0) {
                        mbar_arrive_tx(bar_k_full(slot), act ? kTileBytes : 0);
                        if (act) {
                            int cw, chh, ctt;
                            unit_coords(pk, j, cw, chh, ctt);
                            const uint32_t dst = sbase + kOffK + slot * kSlotBytes;
                            tma_load_5d(dst, &P.tm_k, bar_k_full(slot), 0, cw, chh, ctt + c3k, c4k);
                            tma_load_5d(dst + kHalfBytes, &P.tm_k, bar_k_full(slot), 64, cw, chh, ctt + c3k, c4k);
                        }
                    }
                }
            }
        }
        if (!ok && lane == 0) {
            // drain: give the copies this warp issued a bounded time to land before the CTA exits
            const long long t0 = clock64();
            for (unsigned r = gk > kKSlots ? gk - kKSlots : 0; r < gk; ++r)
                while (!mbar_try(bar_k_full(r % kKSlots), (r / kKSlots) & 1) && clock64() - t0 < 40000000ll) {
                }
            for (unsigned r = gv > kVSlots ? gv - kVSlots : 0; r < gv; ++r)
                while (!mbar_try(bar_v_full(r % kVSlots), (r / kVSlots) & 1) && clock64() - t0 < 40000000ll) {
                }
            if (nq_issued > 0)
                while (!mbar_try(bar_q_full, (nq_issued - 1) & 1) && clock64() - t0 < 40000000ll) {
                }
        }
      } else if (warp == 9) {
        // ================================================================== S = Q K^T issuer
        const uint32_t idesc_s = instr_desc(bf16, kQRows, kBlk, 0);
        const uint64_t qd = smem_desc(sbase + kOffQ, 16, 1024);
        unsigned gb = 0, wk = 0, rr0 = 0, rr1 = 0;
        bool ok = true;
        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), qb = (int)(w % groups);
            const int n_act = clamp_cnt(P, bh, qb) << P.lg_units;
            const int n_iter = max(2, n_act);
            ok = mbar_wait_warp(bar_q_full, wk & 1, ctl, 30, wk);
            bool pre = false;
            for (int i = 0; i < n_iter && ok; ++i, ++gb) {
                const int wg = i & 1;
                const unsigned rr = wg ? rr1 : rr0;
                const int slot = gb % kKSlots, buf = rr & 1;
                if (!pre) {  // not already seen ready by the look-ahead of the unit before
                    ok = mbar_wait_warp(bar_k_full(slot), (gb / kKSlots) & 1, ctl, 40, gb);
                    // the buffer held P of the warpgroup's round rr - 2: that PV has to be finished
                    if (ok) ok = mbar_wait_warp(bar_pv_done(wg, buf), ((rr >> 1) & 1) ^ 1, ctl, 34 + wg, rr);
                    if (!ok) break;
                }
                // look ahead: probe the two barriers of the item's next unit now, read the answer after the MMAs
                bool nk = false, np = false;
                if (i + 1 < n_iter) {
                    const int wg2 = wg ^ 1;
                    const unsigned rr2 = wg2 ? rr1 : rr0;  // that warpgroup's next round
                    nk = mbar_test(bar_k_full((gb + 1) % kKSlots), ((gb + 1) / kKSlots) & 1);
                    np = mbar_test(bar_pv_done(wg2, rr2 & 1), ((rr2 >> 1) & 1) ^ 1);
                }
                tc_fence_after();
                if (i < n_act) {
                    const uint64_t kd = smem_desc(sbase + kOffK + slot * kSlotBytes, 16, 1024);
                    const uint32_t d = tmem + kTmWg * wg + kTmS + 64u * buf;
#pragma unroll
                    for (int j = 0; j < kD / 16; ++j) {
                        // 32 bytes per 16-column step inside a 64-column half; the halves are 16 KiB (Q) and
                        // 8 KiB (K) apart
                        const uint64_t qoff = (uint64_t)(((j >> 2) * kQHalfBytes + (j & 3) * 32) >> 4);
                        const uint64_t koff = (uint64_t)(((j >> 2) * kHalfBytes + (j & 3) * 32) >> 4);
                        tc_mma(d, qd + qoff, kd + koff, idesc_s, j > 0);
                    }
                }
                tc_commit(bar_k_empty(slot));  // K is free once these MMAs have read it
                tc_commit(bar_s_full(wg, buf));
                if (i == n_iter - 1) tc_commit(bar_q_empty);  // and so is Q after the last S of the item
                if (wg) ++rr1; else ++rr0;
                pre = __all_sync(0xffffffffu, nk && np);
            }
        }
      } else if (warp == 10) {
        // ================================================================== O += P V issuer
        const uint32_t idesc_pv = instr_desc(bf16, kQRows, kD, 1);
        unsigned gb = 0, wk = 0, rr0 = 0, rr1 = 0;
        bool ok = true;
        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), qb = (int)(w % groups);
            const int n_act = clamp_cnt(P, bh, qb) << P.lg_units;
            const int n_iter = max(2, n_act);
            // the epilogue of the previous item has read both O accumulators
            ok = mbar_wait_warp(bar_o_free, (wk & 1) ^ 1, ctl, 36, wk);
            bool pre = false;
            for (int i = 0; i < n_iter && ok; ++i, ++gb) {
                const int wg = i & 1;
                const unsigned rr = wg ? rr1 : rr0;
                const int slot = gb % kVSlots, buf = rr & 1;
                if (!pre) {
                    ok = mbar_wait_warp(bar_v_full(slot), (gb / kVSlots) & 1, ctl, 60, gb);
                    if (ok) ok = mbar_wait_warp(bar_p_full(wg, buf), (rr >> 1) & 1, ctl, 50 + wg, rr);
                    if (!ok) break;
                }
                bool nv = false, np = false;  // look ahead to the item's next unit
                if (i + 1 < n_iter) {
                    const int wg2 = wg ^ 1;
                    const unsigned rr2 = wg2 ? rr1 : rr0;
                    nv = mbar_test(bar_v_full((gb + 1) % kVSlots), ((gb + 1) / kVSlots) & 1);
                    np = mbar_test(bar_p_full(wg2, rr2 & 1), (rr2 >> 1) & 1);
                }
                tc_fence_after();
                // A: P in TMEM (first 32 columns of the S buffer), 8 columns per 16-key step.
                // B: V tile, MN-major: 64-column halves 8 KiB apart (LBO), 8-key groups 1 KiB apart (SBO).
                if (i < n_act) {
                    const uint32_t pa = tmem + kTmWg * wg + kTmS + 64u * buf;
                    const uint64_t vd = smem_desc(sbase + kOffV + slot * kSlotBytes, kHalfBytes, 1024);
                    const uint32_t d = tmem + kTmWg * wg + kTmO;
#pragma unroll
                    for (int j = 0; j < kBlk / 16; ++j)
                        tc_mma_ts(d, pa + 8u * j, vd + (uint64_t)((j * 2048) >> 4), idesc_pv, (i > 1 || j > 0) ? 1u : 0u);
                }
                // the V slots of the item's last two units go to the epilogue, which stages O in them and frees them
                if (i < n_iter - 2) tc_commit(bar_v_empty(slot));
                tc_commit(bar_pv_done(wg, buf));
                if (wg) ++rr1; else ++rr0;
                pre = __all_sync(0xffffffffu, nv && np);
            }
        }
      } else {
        // ================================================================== output store warp
        // Waits for the staged rows of a work item, sends them off by TMA and hands the two V slots they were staged
        // in back to the producer, so that the warpgroups do not wait for the store.
        unsigned gb = 0, wk = 0;
        bool ok = true;
        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), qb = (int)(w % groups);
            const int b = bh / P.heads, h = bh % P.heads;
            gb += max(2, clamp_cnt(P, bh, qb) << P.lg_units);
            const int s0 = (int)((gb - 2) % kVSlots);  // gb is even and so is the ring: slots s0 and s0 + 1
            ok = mbar_wait_warp(bar_o_staged, wk & 1, ctl, 110, wk);
            if (ok && lane == 0) {
                Coord cc = block_coord(P.gq, qb, b, h, P.heads, P.merge_o, P.Tq);
                const CUtensorMap* tmo = &P.tm_o[0];
                if (P.o_frames > 0) {  // blocks never straddle ranks: o_frames is a multiple of the block's frames
                    const int dst = cc.c3 / P.o_frames;
                    cc.c3 -= dst * P.o_frames;
                    tmo = &P.tm_o[dst];
                }
                const uint32_t src = sbase + kOffV + s0 * kSlotBytes;
                tma_store_5d(tmo, src, 0, cc.c1, cc.c2, cc.c3, cc.c4);
                tma_store_5d(tmo, src + kQHalfBytes, 64, cc.c1, cc.c2, cc.c3, cc.c4);
                tma_store_commit();
                tma_store_wait_read();
                mbar_arrive(bar_v_empty(s0));
                mbar_arrive(bar_v_empty(s0 + 1));
            }
            __syncwarp();
        }
        if (lane == 0) tma_store_wait_all();
      }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
        // ================================================================== softmax warpgroups
        const int wg = warp >> 2;         // warpgroup: takes units wg, wg + 2, ... of every work item
        const int wq = warp & 3;          // TMEM quadrant of this warp
        const int row = wq * 32 + lane;   // row of the query block = TMEM lane
        const uint32_t t_lane = (uint32_t)(wq * 32) << 16;
        const uint32_t tm_s = tmem + kTmWg * wg + kTmS + t_lane;
        const uint32_t tm_o_mine = tmem + kTmWg * wg + kTmO + t_lane, tm_o_other = tmem + kTmWg * (wg ^ 1) + kTmO + t_lane;
        const int ml_idx = row;
        unsigned rr = 0, wk = 0, gb = 0;
        bool ok = true;

        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), qt = (int)(w % groups);
            const int n_act = clamp_cnt(P, bh, qt) << P.lg_units;
            const int n_iter = max(2, n_act);
            const int32_t* my_list = P.idx + ((long long)bh * P.nq + qt) * P.cap;

            float m_ref = -INFINITY, l_sum = 0.f;
            bool first = true;  // no block of this item seen yet by this warpgroup

            // ragged grids: the block index of a round is fetched a round ahead, so that the global load never sits
            // between S and the softmax (unit i belongs to list entry i >> lg_units)
            int blk_ahead = (kRagged && wg < n_act) ? my_list[0] : 0;
            for (int i = wg; i < n_iter && ok; i += 2, ++rr) {
                const bool active = i < n_act;
                const int blk_now = blk_ahead;
                if (kRagged && i + 2 < n_act) blk_ahead = my_list[(i + 2) >> P.lg_units];
                const int buf = rr & 1;
                const unsigned bph = (rr >> 1) & 1;
                ok = mbar_wait_warp(bar_s_full(wg, buf), bph, ctl, 80 + wg, rr);
                if (!ok) break;
                tc_fence_after();
                uint32_t sr[64];
                tc_ld64(tm_s + 64u * buf, sr);
                tc_wait_ld();
                float alpha = 1.f;
                bool need = false;
                uint4 pk[8];  // this row of P in the input dtype, 8 keys per 16-byte chunk
                if (active) {
                    if (kRagged) {  // keys of a partial block that lie outside the grid
                        const int blk = blk_now;
                        int bt, bhh, bw;
                        block_coords(P.gk, blk, bt, bhh, bw);
                        // tokens left along each axis from the first token of this unit
                        int vt = P.gk.T - bt * P.gk.ct, vh = P.gk.H - bhh * P.gk.ch, vw = P.gk.W - bw * P.gk.cw;
                        const int sub = i & ((1 << P.lg_units) - 1);
                        vt -= P.sub_t[sub];
                        vh -= P.sub_h[sub];
                        vw -= P.sub_w[sub];
                        if (vt < P.gu.ct || vh < P.gu.ch || vw < P.gu.cw) {
                            const uint64_t present = slot_mask64(P.gu.ct, P.gu.ch, P.gu.cw, vt, vh, vw);
                            const uint32_t p_lo = (uint32_t)present, p_hi = (uint32_t)(present >> 32);
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (!((p_lo >> j) & 1u)) sr[j] = 0xff800000u;  // -inf
                                if (!((p_hi >> j) & 1u)) sr[32 + j] = 0xff800000u;
                            }
                        }
                    }
                    // One pass: the probabilities are computed against the current reference maximum while
                    // the row maximum is tracked on the side; only if the maximum has moved by more than 2^8
                    // (or this is the warpgroup's first block) is the pass repeated with the new reference.
                    auto probs = [&](float mref, float& rsum) {
                        // two keys per instruction where the machine has packed fp32 forms (fma, add); the four partial
                        // sums take the keys j = 0, 1, 2, 3 (mod 4) in ascending order
                        const float2 sc2 = make_float2(P.scale2, P.scale2), nm2 = make_float2(-mref, -mref);
                        float2 r01 = make_float2(0.f, 0.f), r23 = make_float2(0.f, 0.f);
#pragma unroll
                        for (int cch = 0; cch < 8; ++cch) {
                            float2 e[4];
#pragma unroll
                            for (int jp = 0; jp < 4; ++jp) {
                                const float2 s2 = make_float2(__uint_as_float(sr[cch * 8 + 2 * jp]), __uint_as_float(sr[cch * 8 + 2 * jp + 1]));
                                const float2 x = __ffma2_rn(s2, sc2, nm2);
                                e[jp] = make_float2(ex2(x.x), ex2(x.y));
                            }
                            r01 = __fadd2_rn(r01, e[0]);
                            r23 = __fadd2_rn(r23, e[1]);
                            r01 = __fadd2_rn(r01, e[2]);
                            r23 = __fadd2_rn(r23, e[3]);
                            pk[cch].x = pack2(bf16, e[0].x, e[0].y);
                            pk[cch].y = pack2(bf16, e[1].x, e[1].y);
                            pk[cch].z = pack2(bf16, e[2].x, e[2].y);
                            pk[cch].w = pack2(bf16, e[3].x, e[3].y);
                        }
                        rsum = (r01.x + r01.y) + (r23.x + r23.y);
                    };
                    // the reference maximum this row would have after this block (in units of log2)
                    auto row_reference = [&]() {
                        float mx8[8];  // eight chains of eight values, three at a time
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            auto sv = [&](int i) { return __uint_as_float(sr[8 * i + k]); };
                            mx8[k] = fmaxf(max3(max3(max3(sv(0), sv(1), sv(2)), sv(3), sv(4)), sv(5), sv(6)), sv(7));
                        }
                        const float mx = fmaxf(max3(max3(mx8[0], mx8[1], mx8[2]), mx8[3], mx8[4]), max3(mx8[5], mx8[6], mx8[7]));
                        return first ? mx * P.scale2 : fmaxf(m_ref, mx * P.scale2);  // no reference yet: m_ref is a placeholder
                    };
                    float rs = 0.f;
                    float m_new = m_ref;
                    if (kRagged) {
                        // the instantiation with the masking code: a single copy of the pass in the instruction stream.
                        // The loop body runs once in the common case (pass, then the row maximum, which confirms the
                        // reference) and twice when the reference moves; for the warpgroup's first block the first
                        // pass is skipped.
                        bool run_pass = !first, decided = false;
#pragma unroll 1
                        for (int turn = 0; turn < 2; ++turn) {
                            if (run_pass) probs(m_ref, rs);
                            if (decided) break;
                            m_new = row_reference();
                            run_pass = first || m_new - m_ref > 8.f;
                            if (!run_pass) break;
                            if (!first) {
                                need = true;
                                alpha = ex2(m_ref - m_new);
                            }
                            m_ref = (m_new == -INFINITY) ? 0.f : m_new;
                            decided = true;
                        }
                    } else {
                        // whole grids: straight-line code, the second copy of the pass off the common path
                        if (!first) probs(m_ref, rs);
                        m_new = row_reference();
                        if (LCBSA_UNLIKELY(first || m_new - m_ref > 8.f)) {
                            if (!first) {
                                need = true;
                                alpha = ex2(m_ref - m_new);
                            }
                            m_ref = (m_new == -INFINITY) ? 0.f : m_new;
                            probs(m_ref, rs);
                        }
                    }
                    l_sum = l_sum * alpha + rs;  // alpha is 1 unless this row's reference maximum moved
                    // a unit that lies wholly outside a ragged grid leaves no reference behind: the next one is the first
                    first = first && m_new == -INFINITY;
                } else {
                    first = false;
                }
                const bool any_need = __any_sync(0xffffffffu, need);
                // O is rescaled only at rest: the warpgroup's PV of the round before has to be finished
                // (need implies that this is not the warpgroup's first round of the item, so rr > 0)
                if (LCBSA_UNLIKELY(any_need)) {
                    ok = mbar_wait_warp(bar_pv_done(wg, buf ^ 1), ((rr - 1) >> 1) & 1, ctl, 92 + wg, rr);
                    if (!ok) break;
                }
                {   // P overwrites the first half of the S buffer just read (don't-cares for a unit that does not exist)
                    uint32_t pr[32];
#pragma unroll
                    for (int cch = 0; cch < 8; ++cch) {
                        pr[4 * cch + 0] = pk[cch].x;
                        pr[4 * cch + 1] = pk[cch].y;
                        pr[4 * cch + 2] = pk[cch].z;
                        pr[4 * cch + 3] = pk[cch].w;
                    }
                    tc_st32(tm_s + 64u * buf, pr);
                }
                if (LCBSA_UNLIKELY(any_need)) tc_scale_row128(tm_o_mine, alpha);  // rare: only when a row maximum jumps
                tc_wait_st();
                tc_fence_before();
                mbar_arrive_elect(bar_p_full(wg, buf));
            }
            if (!ok) break;
            gb += n_iter;

            // ---- epilogue of this work item.  The warpgroup's PVs are finished once its last one is; it then
            // publishes (maximum, row sum) of its rows and waits for the other warpgroup to do the same.
            {   // n_iter is even and at least 2: every warpgroup has had a round
                const unsigned lr = rr - 1;
                ok = mbar_wait_warp(bar_pv_done(wg, lr & 1), (lr >> 1) & 1, ctl, 100 + wg, lr);
                if (!ok) break;
            }
            // the other warpgroup has read this warpgroup's entry of the previous item before it arrived on o_free
            if (wk > 0) {
                ok = mbar_wait_warp(bar_o_free, (wk - 1) & 1, ctl, 102 + wg, wk);
                if (!ok) break;
            }
            ml[wg * 128 + ml_idx] = make_float2(m_ref, l_sum);
            __syncwarp();
            mbar_arrive_elect(bar_ml_ready);
            ok = mbar_wait_warp(bar_ml_ready, wk & 1, ctl, 104 + wg, wk);
            if (!ok) break;
            tc_fence_after();
            const float2 oth = ml[(wg ^ 1) * 128 + ml_idx];
            // merged scale of both partial sums: everything relative to the larger reference maximum
            const float m_all = fmaxf(l_sum > 0.f ? m_ref : -INFINITY, oth.y > 0.f ? oth.x : -INFINITY);  // a side that saw no key has no maximum
            const float w_mine = l_sum > 0.f ? ex2(m_ref - m_all) : 0.f;
            const float w_oth = oth.y > 0.f ? ex2(oth.x - m_all) : 0.f;
            const float l_all = l_sum * w_mine + oth.y * w_oth;
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
            const float f_mine = w_mine * inv, f_oth = w_oth * inv;
            // This warpgroup merges and stages columns 64*wg .. 64*wg+63 of O (input dtype, one 128B-swizzled
            // half-tile row per thread) in the V slot that its own last PV has just released: the last two units of
            // the item sit in slots s0 (warpgroup 0) and s0 + 1 (warpgroup 1), s0 even.
            unsigned char* o_half = smem + kOffV + ((gb - 2) % kVSlots + wg) * kSlotBytes;
#pragma unroll
            for (int cch = 0; cch < 2; ++cch) {
                uint32_t oa[32], ob[32];
                // a warpgroup that saw no block has weight 0; its accumulator holds garbage and is not used
                const bool rd_mine = __any_sync(0xffffffffu, w_mine > 0.f), rd_oth = __any_sync(0xffffffffu, w_oth > 0.f);
                if (rd_mine) tc_ld32(tm_o_mine + 64 * wg + 32 * cch, oa);
                if (rd_oth) tc_ld32(tm_o_other + 64 * wg + 32 * cch, ob);
                tc_wait_ld();
                {
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        float v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float a = w_mine > 0.f ? __uint_as_float(oa[q8 * 8 + j]) * f_mine : 0.f;
                            const float bb = w_oth > 0.f ? __uint_as_float(ob[q8 * 8 + j]) * f_oth : 0.f;
                            v[j] = a + bb;
                        }
                        uint4 pk;
                        pk.x = pack2(bf16, v[0], v[1]);
                        pk.y = pack2(bf16, v[2], v[3]);
                        pk.z = pack2(bf16, v[4], v[5]);
                        pk.w = pack2(bf16, v[6], v[7]);
                        const int chunk = cch * 4 + q8;
                        *reinterpret_cast<uint4*>(o_half + row * 128 + ((chunk ^ (row & 7)) << 4)) = pk;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            mbar_arrive_elect(bar_o_free);  // both O accumulators may be overwritten by the next item's first PVs
            if (wg == 0 && P.lse != nullptr) {
                int lt, lh, lw, bt, bhh, bw;
                slot_coords(P.gq, row, lt, lh, lw);
                block_coords(P.gq, qt, bt, bhh, bw);
                const int tt = bt * P.gq.ct + lt, hh = bhh * P.gq.ch + lh, ww = bw * P.gq.cw + lw;
                if (tt < P.gq.T && hh < P.gq.H && ww < P.gq.W) {
                    const long long Sq = (long long)P.gq.T * P.gq.H * P.gq.W;
                    const long long tok = ((long long)tt * P.gq.H + hh) * P.gq.W + ww;
                    P.lse[(long long)bh * Sq + tok] = l_all > 0.f ? (m_all + log2f(l_all)) * 0.6931471805599453f : -INFINITY;
                }
            }
            fence_proxy_async();
            __syncwarp();
            mbar_arrive_elect(bar_o_staged);  // the store warp takes it from here
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

}  // namespace

// Cuts a key block of 64 * 2^k tokens into units of 64 keys: the outermost even axis is halved until 64 tokens are
// left, so that a unit is one TMA box and the units are as close to contiguous runs of the block's slot order as the
// shape allows.  (ut, uh, uw): the unit's extents; units are numbered t-major, then h, then w.
struct UnitSplit {
    int ut, uh, uw, lg_units;
};
static UnitSplit split_into_units(const Geom& g) {
    UnitSplit u{g.ct, g.ch, g.cw, 0};
    while (u.ut * u.uh * u.uw > kBlk) {
        if (u.ut % 2 == 0) u.ut /= 2;
        else if (u.uh % 2 == 0) u.uh /= 2;
        else u.uw /= 2;  // the token count is a power of two, so some axis is even
        ++u.lg_units;
    }
    return u;
}

bool attn_tc128_supported(const AttnArgs& a, const char** why) {
    if (a.dtype != LCBSA_BF16 && a.dtype != LCBSA_FP16) { *why = "needs bf16 or fp16"; return false; }
    if (a.D != kD) { *why = "needs head_dim 128"; return false; }
    if (a.gq.bs != kQRows || (a.gk.bs != 128 && a.gk.bs != 256 && a.gk.bs != 512)) {
        *why = "needs 128-token query blocks and key blocks of 128, 256 or 512 tokens";
        return false;
    }
    if (a.gq.ct > 256 || a.gq.ch > 256 || a.gq.cw > 256 || a.gk.ct > 256 || a.gk.ch > 256 || a.gk.cw > 256) {
        *why = "block axis above the TMA box limit";
        return false;
    }
    if (a.gk.T > 1023 || a.gk.H > 1023 || a.gk.W > 1023) {
        *why = "key grid axis above 1023 tokens (block coordinates are packed into 10-bit fields)";
        return false;
    }
    if (a.n_out_dst > 0) {
        if (a.n_out_dst > kMaxOutDst) { *why = "more than 8 output destinations"; return false; }
        if (a.B != 1) { *why = "scattered output needs batch 1"; return false; }
        if (a.gq.ragged || a.gq.T % a.n_out_dst != 0 || (a.gq.T / a.n_out_dst) % a.gq.ct != 0) {
            *why = "scattered output needs a query grid whose frames split evenly, on block boundaries, over the destinations";
            return false;
        }
    }
    const View* vs[4] = {&a.q, &a.k, &a.v, &a.o};
    const Geom* gs[4] = {&a.gq, &a.gk, &a.gk, &a.gq};
    for (int i = 0; i < (a.n_out_dst > 0 ? 3 : 4); ++i) {
        if (merge_mode(*vs[i], a.B, a.H, *gs[i]) < 0) { *why = "batch stride cannot be folded into a 5-D tensor map"; return false; }
        if (vs[i]->ss * 2 >= (1ll << 40) || vs[i]->sh * 2 >= (1ll << 40)) { *why = "stride too large for a tensor map"; return false; }
    }
    return true;
}

cudaError_t launch_attn_tc128(const AttnArgs& a, cudaStream_t st, const char** why) {
    if (a.gq.nblk == 0 || a.B * a.H == 0) return cudaSuccess;
    TcParams P;
    // geometry of one unit of 64 keys, and where every unit starts inside its block
    const UnitSplit us = split_into_units(a.gk);
    Geom gu = a.gk;
    gu.ct = us.ut; gu.ch = us.uh; gu.cw = us.uw;
    gu.bs = kBlk;
    P.lg_units = us.lg_units;
    {
        const int ph = a.gk.ch / us.uh, pw = a.gk.cw / us.uw;
        for (int u = 0; u < (1 << us.lg_units); ++u) {
            P.sub_w[u] = (u % pw) * us.uw;
            P.sub_h[u] = ((u / pw) % ph) * us.uh;
            P.sub_t[u] = (u / (pw * ph)) * us.ut;
        }
        for (int u = 1 << us.lg_units; u < kMaxUnits; ++u) P.sub_t[u] = P.sub_h[u] = P.sub_w[u] = 0;
    }
    P.gu = gu;
    const int mq = merge_mode(a.q, a.B, a.H, a.gq), mk = merge_mode(a.k, a.B, a.H, a.gk);
    const int mv = merge_mode(a.v, a.B, a.H, a.gk), mo = merge_mode(a.o, a.B, a.H, a.gq);
    if (!make_map(&P.tm_q, a.dtype, a.q, a.B, a.H, a.gq, mq) || !make_map(&P.tm_k, a.dtype, a.k, a.B, a.H, gu, mk) ||
        !make_map(&P.tm_v, a.dtype, a.v, a.B, a.H, gu, mv)) {
        *why = "cuTensorMapEncodeTiled rejected a tensor";
        return cudaErrorInvalidValue;
    }
    P.o_frames = 0;
    if (a.n_out_dst > 0) {
        // one map per destination over [D, W, H, T / n, heads]: the rank-major grid split along T
        Geom gl = a.gq;
        gl.T = a.gq.T / a.n_out_dst;
        P.o_frames = gl.T;
        for (int r = 0; r < a.n_out_dst; ++r) {
            View vo = a.o;
            vo.data = a.out_dst[r];
            if (!make_map(&P.tm_o[r], a.dtype, vo, 1, a.H, gl, 0)) {
                *why = "cuTensorMapEncodeTiled rejected a destination of the scattered output";
                return cudaErrorInvalidValue;
            }
        }
    } else if (!make_map(&P.tm_o[0], a.dtype, a.o, a.B, a.H, a.gq, mo)) {
        *why = "cuTensorMapEncodeTiled rejected a tensor";
        return cudaErrorInvalidValue;
    }
    P.idx = a.idx; P.cnt = a.cnt; P.lse = a.lse; P.status = a.status;
    P.cap = a.cap; P.nq = a.gq.nblk; P.bh_total = a.B * a.H; P.heads = a.H;
    P.merge_q = mq; P.merge_k = mk; P.merge_v = mv; P.merge_o = mo; P.Tq = a.gq.T; P.Tk = a.gk.T;
    P.gq = a.gq; P.gk = a.gk;
    P.scale2 = a.sm_scale * 1.4426950408889634f;
    P.is_bf16 = a.dtype == LCBSA_BF16;

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) { *why = "device ordinal above 63"; return cudaErrorInvalidValue; }
    DeviceState& ds = device_states()[dev];
    int sm_count = ds.sm_count.load(std::memory_order_relaxed);
    if (sm_count == 0) {
        e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return e;
        ds.sm_count.store(sm_count, std::memory_order_relaxed);
    }
    const bool ragged = a.gk.ragged;
    auto kern = P.is_bf16 ? (ragged ? attn_tc128_kernel<true, true> : attn_tc128_kernel<true, false>)
                          : (ragged ? attn_tc128_kernel<false, true> : attn_tc128_kernel<false, false>);
    const int bit = 16 << ((P.is_bf16 ? 0 : 1) + (ragged ? 2 : 0));  // bits 4-7 of attr_set
    if (!(ds.attr_set.load(std::memory_order_relaxed) & bit)) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return e;
        ds.attr_set.fetch_or(bit, std::memory_order_relaxed);
    }
    const long long work = (long long)a.gq.nblk * a.B * a.H;
    const int reserve = attn_sm_reserve();
    const int usable = sm_count - reserve > 0 ? sm_count - reserve : 1;
    const int grid = (int)(work < usable ? work : usable);
    kern<<<grid, kThreads, kSmemBytes, st>>>(P);
    return cudaGetLastError();
}

}  // namespace lcbsa
