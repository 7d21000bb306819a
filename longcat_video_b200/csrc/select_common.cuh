// Shared by the two forms of the block-select score/top-k stage (select.cu, select_gemm.cu): order-preserving
// score keys and the per-row selection.
#pragma once
#include "common.cuh"

namespace lcbsa {
namespace sel {

constexpr int kRegWords = 24;  // 32-bit words of a 16-bit key row that a lane may keep in registers (rows up to 1536 keys)

template <typename T> struct KeyOf { using type = uint16_t; };
template <> struct KeyOf<float> { using type = uint32_t; };

// Order-preserving key: a larger key is a larger score; -0 equals +0; NaN ranks above +inf.
__device__ __forceinline__ uint16_t make_key(__nv_bfloat16 v) {
    uint16_t u = __bfloat16_as_ushort(v);
    if ((u & 0x7fffu) > 0x7f80u) return 0xffffu;
    if (u == 0x8000u) u = 0;
    return (u & 0x8000u) ? (uint16_t)~u : (uint16_t)(u | 0x8000u);
}
__device__ __forceinline__ uint16_t make_key(__half v) {
    uint16_t u = __half_as_ushort(v);
    if ((u & 0x7fffu) > 0x7c00u) return 0xffffu;
    if (u == 0x8000u) u = 0;
    return (u & 0x8000u) ? (uint16_t)~u : (uint16_t)(u | 0x8000u);
}
__device__ __forceinline__ uint32_t make_key(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
    if (u == 0x80000000u) u = 0;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Number of keys of a row that are >= cand (gt == false) or > cand (gt == true).
__device__ __forceinline__ int count_row(const uint16_t* row, int nk_pad, uint32_t cand, bool gt, int lane) {
    const uint32_t* r32 = reinterpret_cast<const uint32_t*>(row);
    const uint32_t c = gt ? cand + 1u : cand;  // cand + 1 may be 0x10000: no 16-bit key reaches it
    int n = 0;
    for (int p = lane; p < nk_pad / 2; p += 32) {
        const uint32_t kk = r32[p];
        n += ((kk & 0xffffu) >= c) + ((kk >> 16) >= c);
    }
    return warp_sum(n);
}
__device__ __forceinline__ int count_row(const uint32_t* row, int nk_pad, uint32_t cand, bool gt, int lane) {
    int n = 0;
    for (int p = lane; p < nk_pad; p += 32) {
        const uint32_t kk = row[p];
        n += gt ? (kk > cand) : (kk >= cand);
    }
    return warp_sum(n);
}

// Which key blocks a row may select from.  Blocks are numbered frame-major (t, then h, then w); a block belongs to the
// "first part" when (its frame-block index % period) < split -- period = all frame blocks and split = the conditioning
// frame blocks for a single grid, period = the frame blocks of one rank for the rank-major grid of a context-parallel
// group.  period == 0: every block is allowed.
struct KeyMask {
    int hw, period, split;
    __device__ __forceinline__ bool operator()(int j) const { return period == 0 || ((j / hw) % period) < split; }
};

// The nsel largest keys of one row (ties at the threshold broken towards the lower block index), emitted as
// ascending block indices by one warp; the cap - nsel trailing entries are set to -1.  `row` may be shared or
// global memory; nk_pad (a multiple of 64) entries are readable and those past Nk hold key 0.
template <typename Key>
__device__ __forceinline__ void select_row(const Key* row, int Nk, int nk_pad, int nsel, int cap, int32_t* out, int32_t* cnt_out,
                                           int lane, const KeyMask mask = KeyMask{1, 0, 0}) {
    constexpr int kKeyBits = sizeof(Key) * 8;
    if (lane == 0) *cnt_out = nsel;
    if (nsel > 0) {
        uint32_t thr = 0;
        int above;
        if (sizeof(Key) == 2 && nk_pad <= 2 * 32 * kRegWords) {
            // 16-bit keys of a row that fits: every lane keeps its share of the row (two keys per word) in registers,
            // so the 17 counting passes of the bisection read the row once
            const uint32_t* r32 = reinterpret_cast<const uint32_t*>(row);
            const int nwords = nk_pad / 2;
            uint32_t w[kRegWords];
#pragma unroll
            for (int i = 0; i < kRegWords; ++i) w[i] = (lane + 32 * i < nwords) ? r32[lane + 32 * i] : 0u;  // key 0 is never counted
            if (mask.period != 0) {  // keys of blocks this row may not select become key 0
#pragma unroll
                for (int i = 0; i < kRegWords; ++i) {
                    const int j = 2 * (lane + 32 * i);
                    if (!mask(j)) w[i] &= 0xffff0000u;
                    if (!mask(j + 1)) w[i] &= 0x0000ffffu;
                }
            }
            auto count = [&](uint32_t c) {  // keys >= c, c >= 1
                int n = 0;
#pragma unroll
                for (int i = 0; i < kRegWords; ++i) n += ((w[i] & 0xffffu) >= c) + ((w[i] >> 16) >= c);
                return warp_sum(n);
            };
            for (int bit = kKeyBits - 1; bit >= 0; --bit) {
                const uint32_t cand = thr | (1u << bit);
                if (count(cand) >= nsel) thr = cand;
            }
            above = count(thr + 1u);
        } else if (mask.period != 0) {
            // a masked row is only handled where it fits in registers (the host checks this before the launch):
            // select nothing rather than something wrong
            if (lane == 0) *cnt_out = 0;
            for (int j = lane; j < cap; j += 32) out[j] = -1;
            return;
        } else {
            for (int bit = kKeyBits - 1; bit >= 0; --bit) {
                const uint32_t cand = thr | (1u << bit);
                if (count_row(row, nk_pad, cand, false, lane) >= nsel) thr = cand;
            }
            above = count_row(row, nk_pad, thr, true, lane);
        }
        const int take_eq = nsel - above;  // ties at the threshold to keep, lowest block index first
        int n_out = 0, n_eq = 0;
        const unsigned lt_mask = (1u << lane) - 1u;
        for (int j0 = 0; j0 < Nk; j0 += 32) {
            const int j = j0 + lane;
            const bool ok = (j < Nk) && mask(j);
            const uint32_t key = ok ? (uint32_t)row[j] : 0u;
            const bool gt = key > thr;
            const bool eq = (key == thr) && ok;
            const unsigned eq_mask = __ballot_sync(0xffffffffu, eq);
            const bool take = gt || (eq && (n_eq + __popc(eq_mask & lt_mask) < take_eq));
            const unsigned take_mask = __ballot_sync(0xffffffffu, take);
            if (take) out[n_out + __popc(take_mask & lt_mask)] = j;
            n_out += __popc(take_mask);
            n_eq += __popc(eq_mask);
        }
    }
    for (int j = nsel + lane; j < cap; j += 32) out[j] = -1;
}

}  // namespace sel
}  // namespace lcbsa
