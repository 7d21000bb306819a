// Block-select stage, cdf_threshold selectors: per row of block scores, softmax weights, the whole row sorted by
// descending weight, the running sum of the sorted weights, and the number of entries whose running sum stays at or
// below the threshold.
//
// Replaces get_select_indices_cdf_from_score and get_select_indices_cdf_topk_from_score
// (longcat_video/block_sparse_attention/bsa_interface.py:234-244, 253-266): torch.softmax, torch.sort, torch.cumsum and
// torch.searchsorted over [B, H, Nq, Nk] tensors, five passes over HBM and an int64 index tensor.  Here a row never
// leaves the SM: one CTA per row reads the 16-bit score keys that score_gemm_kernel wrote (2 bytes per score) and
// writes the int32 index row (4 bytes per entry) and one count.
//
// Arithmetic, in the order the CPU oracle fixes where the reference leaves it to the library:
//   x = T(score * sm_scale);  e = exp(x - max x) with the machine-independent exp below;  the denominator as 256
//   partial sums (thread t adds its E consecutive entries t E .. t E + E - 1 in ascending order, E = 8 up to 2048
//   entries and 16 above), a butterfly over each warp and over the 8 warp sums;  w = T(e / sum);  sort by (w descending, index ascending): all keys are distinct, so the result does
//   not depend on the sorting network;  cdf = T(fp32 running sum), count = #(cdf <= threshold), at least nsel_min.
#include "select_common.cuh"

namespace lcbsa {

namespace {

constexpr int kCdfThreads = 256;

// exp(t), t <= 0, from fmaf / rintf / one scaling by a power of two: the same bits as the oracle's lco_exp.
__device__ __forceinline__ float exp_portable(float t) {
    if (!(t >= -87.0f)) return 0.0f;
    const float n = rintf(__fmul_rn(t, 1.44269504f));
    float r = fmaf(-n, 0.693145751953125f, t);
    r = fmaf(-n, 1.42860677e-6f, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    return __fmul_rn(p, __uint_as_float((uint32_t)((int)n + 127) << 23));
}

template <typename T>
__device__ __forceinline__ T from_bits(uint16_t u);
template <>
__device__ __forceinline__ __nv_bfloat16 from_bits<__nv_bfloat16>(uint16_t u) { return __ushort_as_bfloat16(u); }
template <>
__device__ __forceinline__ __half from_bits<__half>(uint16_t u) { return __ushort_as_half(u); }
__device__ __forceinline__ uint16_t to_bits(__nv_bfloat16 v) { return __bfloat16_as_ushort(v); }
__device__ __forceinline__ uint16_t to_bits(__half v) { return __half_as_ushort(v); }

// The running sum of the sorted weights is sequential by definition (fp32, every partial result rounded to T for the
// comparison).  One warp: lane l holds entry 32 c + l of chunk c, the weights go round by shuffle and every lane adds
// them in order, keeping the sum as it stood after its own entry.  Stops at the first chunk that passes the threshold.
template <typename T>
__device__ __forceinline__ void count_row_cdf(const uint32_t* row, int Nk, float threshold, int nsel_min, int32_t* cnt, int lane) {
    float acc = 0.0f;
    int n = 0;
    for (int c = 0; c < Nk; c += 32) {
        const bool have = c + lane < Nk;
        const float w = have ? DType<T>::to_f32(from_bits<T>((uint16_t)(row[c + lane] >> 16))) : 0.0f;
        float mine = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            acc = __fadd_rn(acc, __shfl_sync(0xffffffffu, w, i));  // absent entries add +0: no change
            mine = lane == i ? acc : mine;
        }
        const bool ok = have && DType<T>::to_f32(DType<T>::from_f32(mine)) <= threshold;
        const uint32_t pass = __ballot_sync(0xffffffffu, ok);
        const int lead = __ffs(~pass) - 1;  // entries before the first that fails (the sums do not decrease)
        if (lead >= 0) {
            n += lead;
            break;
        }
        n += 32;
    }
    if (lane == 0) *cnt = max(min(n, Nk), nsel_min);
}

// Rows of up to 2048 entries: thread t keeps entries 8 t .. 8 t + 7 in registers from the load to the sorted row.
// Of the 66 compare-exchange stages of the 2048-wide bitonic network, the 30 with a distance below 8 stay inside a
// thread, the 30 with a distance of 8 .. 128 entries go through warp shuffles, and only the 6 with a distance of
// 256 .. 1024 entries cross warps through shared memory.
constexpr int kFastE = 8;
constexpr int kFastP = kFastE * kCdfThreads;

template <typename T>
__global__ void __launch_bounds__(kCdfThreads) cdf_rows_fast_kernel(const uint16_t* __restrict__ keys, int Nk, int nk_pad, float sm_scale,
                                                                   float threshold, int nsel_min, int32_t* __restrict__ idx,
                                                                   int32_t* __restrict__ cnt) {
    __shared__ __align__(16) uint32_t row[kFastP];
    __shared__ float red[kCdfThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long r = blockIdx.x;
    const int base = tid * kFastE;

    // x = T(score * sm_scale) and its maximum
    float x[kFastE];
    float m = -INFINITY;
    {
        uint4 raw4 = make_uint4(0u, 0u, 0u, 0u);
        if (base < nk_pad) raw4 = __ldg(reinterpret_cast<const uint4*>(keys + r * nk_pad + base));
        const uint16_t* kk = reinterpret_cast<const uint16_t*>(&raw4);
#pragma unroll
        for (int e = 0; e < kFastE; ++e) {
            const uint16_t raw = (kk[e] & 0x8000u) ? (uint16_t)(kk[e] & 0x7fffu) : (uint16_t)~kk[e];  // inverse of make_key
            x[e] = DType<T>::to_f32(DType<T>::from_f32(__fmul_rn(DType<T>::to_f32(from_bits<T>(raw)), sm_scale)));
            if (base + e < Nk) m = fmaxf(m, x[e]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < kCdfThreads / 32; ++w) m = fmaxf(m, red[w]);
    __syncthreads();

    // e = exp(x - m) and the denominator
    float part = 0.0f;
#pragma unroll
    for (int e = 0; e < kFastE; ++e) {
        if (base + e < Nk) {
            x[e] = exp_portable(__fsub_rn(x[e], m));
            part = __fadd_rn(part, x[e]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
    if (lane == 0) red[warp] = part;
    __syncthreads();
    float grp[kCdfThreads / 32];
#pragma unroll
    for (int w = 0; w < kCdfThreads / 32; ++w) grp[w] = red[w];
#pragma unroll
    for (int o = kCdfThreads / 64; o > 0; o >>= 1) {
        float nxt[kCdfThreads / 32];
#pragma unroll
        for (int w = 0; w < kCdfThreads / 32; ++w) nxt[w] = __fadd_rn(grp[w], grp[w ^ o]);
#pragma unroll
        for (int w = 0; w < kCdfThreads / 32; ++w) grp[w] = nxt[w];
    }
    const float sum = grp[0];

    // sort keys: weight bits above, reversed index below; padding sorts last
    uint32_t v[kFastE];
#pragma unroll
    for (int e = 0; e < kFastE; ++e) {
        v[e] = 0u;
        if (base + e < Nk) v[e] = ((uint32_t)to_bits(DType<T>::from_f32(__fdiv_rn(x[e], sum))) << 16) | (uint32_t)(0xffff - (base + e));
    }

    // bitonic network, descending: entry i and entry i ^ j; the lower index keeps the larger key where (i & k) == 0
#pragma unroll
    for (int k = 2; k <= kFastP; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j < kFastE) {
#pragma unroll
                for (int e = 0; e < kFastE; ++e) {
                    if ((e & j) == 0) {
                        const bool desc = ((base + e) & k) == 0;
                        const uint32_t a = v[e], b = v[e | j];
                        const uint32_t hi = max(a, b), lo = min(a, b);
                        v[e] = desc ? hi : lo;
                        v[e | j] = desc ? lo : hi;
                    }
                }
            } else {
                const bool keep_max = ((base & j) == 0) == ((base & k) == 0);
                uint32_t other[kFastE];
                if (j < kFastE * 32) {
#pragma unroll
                    for (int e = 0; e < kFastE; ++e) other[e] = __shfl_xor_sync(0xffffffffu, v[e], j / kFastE);
                } else {
                    __syncthreads();  // the previous exchange has been read
                    uint4* mine = reinterpret_cast<uint4*>(row + base);
                    mine[0] = make_uint4(v[0], v[1], v[2], v[3]);
                    mine[1] = make_uint4(v[4], v[5], v[6], v[7]);
                    __syncthreads();
                    const uint4* theirs = reinterpret_cast<const uint4*>(row + (base ^ j));
                    const uint4 t0 = theirs[0], t1 = theirs[1];
                    other[0] = t0.x; other[1] = t0.y; other[2] = t0.z; other[3] = t0.w;
                    other[4] = t1.x; other[5] = t1.y; other[6] = t1.z; other[7] = t1.w;
                }
#pragma unroll
                for (int e = 0; e < kFastE; ++e) v[e] = keep_max ? max(v[e], other[e]) : min(v[e], other[e]);
            }
        }
    }

    __syncthreads();
    {
        uint4* mine = reinterpret_cast<uint4*>(row + base);
        mine[0] = make_uint4(v[0], v[1], v[2], v[3]);
        mine[1] = make_uint4(v[4], v[5], v[6], v[7]);
    }
    __syncthreads();
    int32_t* out = idx + r * Nk;
    for (int j = tid; j < Nk; j += kCdfThreads) out[j] = (int32_t)(0xffffu - (row[j] & 0xffffu));
    if (warp == 0) count_row_cdf<T>(row, Nk, threshold, nsel_min, cnt + r, lane);
}

// keys: [rows, nk_pad] order-preserving 16-bit keys of the scores; idx: [rows, Nk]; cnt: [rows].  P: power of two >= Nk.
template <typename T>
__global__ void __launch_bounds__(kCdfThreads) cdf_rows_kernel(const uint16_t* __restrict__ keys, int Nk, int nk_pad, int P, float sm_scale,
                                                              float threshold, int nsel_min, int32_t* __restrict__ idx,
                                                              int32_t* __restrict__ cnt) {
    extern __shared__ uint32_t row[];  // P words: x, then e, then the sort keys
    __shared__ float red[kCdfThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long r = blockIdx.x;
    const uint16_t* src = keys + r * nk_pad;

    // x = T(score * sm_scale) and its maximum
    float m = -INFINITY;
    for (int j = tid; j < Nk; j += kCdfThreads) {
        const uint16_t kk = src[j];
        const uint16_t raw = (kk & 0x8000u) ? (uint16_t)(kk & 0x7fffu) : (uint16_t)~kk;  // inverse of make_key
        const float x = DType<T>::to_f32(DType<T>::from_f32(__fmul_rn(DType<T>::to_f32(from_bits<T>(raw)), sm_scale)));
        row[j] = __float_as_uint(x);
        m = fmaxf(m, x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < kCdfThreads / 32; ++w) m = fmaxf(m, red[w]);
    __syncthreads();

    // e = exp(x - m) and the denominator: thread t sums its E consecutive entries
    float part = 0.0f;
    const int E = Nk <= 2048 ? 8 : 16;
    for (int j = tid * E; j < min(Nk, tid * E + E); ++j) {
        const float e = exp_portable(__fsub_rn(__uint_as_float(row[j]), m));
        row[j] = __float_as_uint(e);
        part = __fadd_rn(part, e);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
    if (lane == 0) red[warp] = part;
    __syncthreads();
    float grp[kCdfThreads / 32];
#pragma unroll
    for (int w = 0; w < kCdfThreads / 32; ++w) grp[w] = red[w];
#pragma unroll
    for (int o = kCdfThreads / 64; o > 0; o >>= 1) {
        float nxt[kCdfThreads / 32];
#pragma unroll
        for (int w = 0; w < kCdfThreads / 32; ++w) nxt[w] = __fadd_rn(grp[w], grp[w ^ o]);
#pragma unroll
        for (int w = 0; w < kCdfThreads / 32; ++w) grp[w] = nxt[w];
    }
    const float sum = grp[0];
    __syncthreads();  // every e is in place before other threads read it

    // sort keys: weight bits above, reversed index below; padding sorts last
    for (int j = tid; j < P; j += kCdfThreads) {
        uint32_t key = 0u;
        if (j < Nk) {
            const uint32_t wb = to_bits(DType<T>::from_f32(__fdiv_rn(__uint_as_float(row[j]), sum)));
            key = (wb << 16) | (uint32_t)(0xffff - j);
        }
        row[j] = key;
    }
    __syncthreads();

    // bitonic network, descending
    for (int k = 2; k <= P; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = tid; t < P / 2; t += kCdfThreads) {
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1));
                const int p = i | j;
                const uint32_t a = row[i], b = row[p];
                const bool desc = (i & k) == 0;
                if (desc ? (a < b) : (a > b)) {
                    row[i] = b;
                    row[p] = a;
                }
            }
            __syncthreads();
        }
    }

    int32_t* out = idx + r * Nk;
    for (int j = tid; j < Nk; j += kCdfThreads) out[j] = (int32_t)(0xffffu - (row[j] & 0xffffu));

    if (warp == 0) count_row_cdf<T>(row, Nk, threshold, nsel_min, cnt + r, lane);
}

}  // namespace

cudaError_t launch_cdf_rows(int dtype, const void* keys, long long rows, int Nk, float sm_scale, float threshold, int nsel_min,
                            int32_t* idx, int32_t* cnt, cudaStream_t st, const char** why) {
    if (rows == 0) return cudaSuccess;
    if (dtype == LCBSA_FP32 || Nk < 1 || Nk > 4096) {
        *why = "the cdf selectors take bf16 or fp16 scores and at most 4096 key blocks";
        return cudaErrorInvalidValue;
    }
    if (rows > 0x7fffffffLL) {
        *why = "the cdf selectors take at most 2^31 - 1 rows";
        return cudaErrorInvalidValue;
    }
    const int nk_pad = (Nk + 63) / 64 * 64;
    const uint16_t* kp0 = static_cast<const uint16_t*>(keys);
    if (Nk <= kFastP) {
        if (dtype == LCBSA_BF16)
            cdf_rows_fast_kernel<__nv_bfloat16><<<(unsigned)rows, kCdfThreads, 0, st>>>(kp0, Nk, nk_pad, sm_scale, threshold, nsel_min, idx, cnt);
        else
            cdf_rows_fast_kernel<__half><<<(unsigned)rows, kCdfThreads, 0, st>>>(kp0, Nk, nk_pad, sm_scale, threshold, nsel_min, idx, cnt);
        return cudaGetLastError();
    }
    int P = 2;
    while (P < Nk) P <<= 1;
    const size_t smem = (size_t)P * sizeof(uint32_t);
    const uint16_t* kp = static_cast<const uint16_t*>(keys);
    if (dtype == LCBSA_BF16)
        cdf_rows_kernel<__nv_bfloat16><<<(unsigned)rows, kCdfThreads, smem, st>>>(kp, Nk, nk_pad, P, sm_scale, threshold, nsel_min, idx, cnt);
    else
        cdf_rows_kernel<__half><<<(unsigned)rows, kCdfThreads, smem, st>>>(kp, Nk, nk_pad, P, sm_scale, threshold, nsel_min, idx, cnt);
    return cudaGetLastError();
}

}  // namespace lcbsa
