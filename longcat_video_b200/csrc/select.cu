// Block-select stage, parts 2 and 3: block scores and per-row top-k, fused so that the score
// matrix never reaches HBM.
//
// Replaces cal_score + get_select_indices_topk_from_score
// (longcat_video/block_sparse_attention/bsa_interface.py:180-184, 212-224).
//
// One CTA owns a strip of RQ pooled-Q rows of one (batch, head) and streams the pooled K rows
// (L2 resident: Nk*D elements per head) through shared memory in chunks of 64 rows.
//   score(i,j) = fp32 FMA chain over d = 0..D-1 (ascending), rounded to the input dtype,
//                i.e. the value a GEMM with fp32 accumulation and a 16-bit result would store.
// The rounded scores are kept in shared memory as order-preserving integer keys.  Each warp then
// selects, for its rows, the nsel largest keys: the threshold key is found by bisection over the key
// bits, ties at the threshold are broken towards the lower block index, and the selected block
// indices are emitted in ascending order with warp ballots.  No atomics: the result is deterministic.
#include "select_common.cuh"

namespace lcbsa {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kChunk = 64;  // pooled K rows per shared-memory chunk

using namespace sel;

template <typename T, int D, int QPW>
__global__ void __launch_bounds__(kThreads) score_topk_kernel(const T* __restrict__ qc, const T* __restrict__ kc,
                                                             int Nq, int Nk, int nk_pad, int nsel, int cap,
                                                             int32_t* __restrict__ idx, int32_t* __restrict__ cnt) {
    using Key = typename KeyOf<T>::type;
    constexpr int RQ = kWarps * QPW;
    constexpr int DP = D + 4;  // padded fp32 row pitch: 16-byte aligned, conflict-free float4 reads
    constexpr int VEC = 16 / sizeof(T);
    constexpr int KV = kChunk * D / VEC / kThreads;  // 16-byte vectors of a K chunk per thread
    static_assert(kChunk * D / VEC % kThreads == 0, "chunk must split evenly over the CTA");

    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* qs = reinterpret_cast<float*>(smem_raw);                     // [RQ][DP]
    float* ks = qs + RQ * DP;                                            // [2][kChunk][DP]
    Key* keys = reinterpret_cast<Key*>(ks + 2 * kChunk * DP);            // [RQ][nk_pad]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int bh = blockIdx.y;
    const int q0 = blockIdx.x * RQ;
    const T* qbase = qc + (long long)bh * Nq * D;
    const T* kbase = kc + (long long)bh * Nk * D;

    // pooled Q strip -> fp32 shared memory (rows past Nq are zero)
    for (int v = tid; v < RQ * D / VEC; v += kThreads) {
        const int row = v / (D / VEC), c = v % (D / VEC);
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (q0 + row < Nq) raw = __ldg(reinterpret_cast<const uint4*>(qbase + (long long)(q0 + row) * D + c * VEC));
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < VEC; ++i) qs[row * DP + c * VEC + i] = DType<T>::to_f32(e[i]);
    }

    const int nchunks = nk_pad / kChunk;
    uint4 pre[KV];
    auto fetch = [&](int chunk) {
#pragma unroll
        for (int i = 0; i < KV; ++i) {
            const int v = tid + i * kThreads;
            const int row = v / (D / VEC), c = v % (D / VEC);
            const int j = chunk * kChunk + row;
            pre[i] = make_uint4(0u, 0u, 0u, 0u);
            if (j < Nk) pre[i] = __ldg(reinterpret_cast<const uint4*>(kbase + (long long)j * D + c * VEC));
        }
    };
    auto stash = [&](int buf) {
        float* dst = ks + buf * kChunk * DP;
#pragma unroll
        for (int i = 0; i < KV; ++i) {
            const int v = tid + i * kThreads;
            const int row = v / (D / VEC), c = v % (D / VEC);
            const T* e = reinterpret_cast<const T*>(&pre[i]);
#pragma unroll
            for (int u = 0; u < VEC; ++u) dst[row * DP + c * VEC + u] = DType<T>::to_f32(e[u]);
        }
    };

    fetch(0);
    stash(0);
    __syncthreads();

    for (int chunk = 0; chunk < nchunks; ++chunk) {
        const int buf = chunk & 1;
        if (chunk + 1 < nchunks) fetch(chunk + 1);

        float acc[QPW][2];
#pragma unroll
        for (int i = 0; i < QPW; ++i) acc[i][0] = acc[i][1] = 0.f;
        const float* k0 = ks + buf * kChunk * DP + lane * DP;
        const float* k1 = k0 + 32 * DP;
        const float* qw = qs + warp * QPW * DP;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
            const float4 a = *reinterpret_cast<const float4*>(k0 + d);
            const float4 b = *reinterpret_cast<const float4*>(k1 + d);
#pragma unroll
            for (int i = 0; i < QPW; ++i) {
                const float4 qv = *reinterpret_cast<const float4*>(qw + i * DP + d);
                acc[i][0] = fmaf(qv.x, a.x, acc[i][0]);
                acc[i][0] = fmaf(qv.y, a.y, acc[i][0]);
                acc[i][0] = fmaf(qv.z, a.z, acc[i][0]);
                acc[i][0] = fmaf(qv.w, a.w, acc[i][0]);
                acc[i][1] = fmaf(qv.x, b.x, acc[i][1]);
                acc[i][1] = fmaf(qv.y, b.y, acc[i][1]);
                acc[i][1] = fmaf(qv.z, b.z, acc[i][1]);
                acc[i][1] = fmaf(qv.w, b.w, acc[i][1]);
            }
        }
#pragma unroll
        for (int i = 0; i < QPW; ++i) {
            Key* row = keys + (long long)(warp * QPW + i) * nk_pad + chunk * kChunk;
            const int j0 = chunk * kChunk + lane, j1 = j0 + 32;
            row[lane] = (j0 < Nk) ? make_key(DType<T>::from_f32(acc[i][0])) : (Key)0;
            row[lane + 32] = (j1 < Nk) ? make_key(DType<T>::from_f32(acc[i][1])) : (Key)0;
        }
        if (chunk + 1 < nchunks) stash(buf ^ 1);
        __syncthreads();
    }

    // ---- per-row selection: each warp owns its QPW rows
    for (int i = 0; i < QPW; ++i) {
        const int qrow = q0 + warp * QPW + i;
        if (qrow >= Nq) break;
        select_row<Key>(keys + (long long)(warp * QPW + i) * nk_pad, Nk, nk_pad, nsel, cap, idx + ((long long)bh * Nq + qrow) * cap,
                        cnt + (long long)bh * Nq + qrow, lane);
    }
}

template <typename T, int D, int QPW>
cudaError_t launch(const void* qc, const void* kc, int BH, int Nq, int Nk, int nk_pad, int nsel, int cap, int32_t* idx,
                   int32_t* cnt, size_t smem, cudaStream_t st) {
    auto kern = score_topk_kernel<T, D, QPW>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    constexpr int RQ = kWarps * QPW;
    dim3 grid((Nq + RQ - 1) / RQ, BH);
    kern<<<grid, kThreads, smem, st>>>(reinterpret_cast<const T*>(qc), reinterpret_cast<const T*>(kc), Nq, Nk, nk_pad,
                                       nsel, cap, idx, cnt);
    return cudaGetLastError();
}

template <typename T, int D>
cudaError_t pick_qpw(const void* qc, const void* kc, int BH, int Nq, int Nk, int nsel, int cap, int32_t* idx,
                     int32_t* cnt, cudaStream_t st, const char** why) {
    using Key = typename KeyOf<T>::type;
    const int nk_pad = (Nk + kChunk - 1) / kChunk * kChunk;
    const size_t limit = 227 * 1024;
    auto need = [&](int qpw) {
        const size_t rq = (size_t)kWarps * qpw;
        return (rq * (D + 4) + 2 * (size_t)kChunk * (D + 4)) * sizeof(float) + rq * nk_pad * sizeof(Key);
    };
    if (need(4) <= limit) return launch<T, D, 4>(qc, kc, BH, Nq, Nk, nk_pad, nsel, cap, idx, cnt, need(4), st);
    if (need(2) <= limit) return launch<T, D, 2>(qc, kc, BH, Nq, Nk, nk_pad, nsel, cap, idx, cnt, need(2), st);
    if (need(1) <= limit) return launch<T, D, 1>(qc, kc, BH, Nq, Nk, nk_pad, nsel, cap, idx, cnt, need(1), st);
    *why = "too many K blocks for the shared-memory score strip";
    return cudaErrorInvalidValue;
}

template <typename T>
cudaError_t pick_d(const void* qc, const void* kc, int BH, int Nq, int Nk, int D, int nsel, int cap, int32_t* idx,
                   int32_t* cnt, cudaStream_t st, const char** why) {
    switch (D) {
        case 64: return pick_qpw<T, 64>(qc, kc, BH, Nq, Nk, nsel, cap, idx, cnt, st, why);
        case 128: return pick_qpw<T, 128>(qc, kc, BH, Nq, Nk, nsel, cap, idx, cnt, st, why);
        default: *why = "head_dim must be 64 or 128"; return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_score_topk(int dtype, const void* qc, const void* kc, int BH, int Nq, int Nk, int D, int nsel,
                              int cap, int32_t* idx, int32_t* cnt, cudaStream_t st, const char** why) {
    if (BH == 0 || Nq == 0) return cudaSuccess;
    switch (dtype) {
        case LCBSA_BF16: return pick_d<__nv_bfloat16>(qc, kc, BH, Nq, Nk, D, nsel, cap, idx, cnt, st, why);
        case LCBSA_FP16: return pick_d<__half>(qc, kc, BH, Nq, Nk, D, nsel, cap, idx, cnt, st, why);
        default: return pick_d<float>(qc, kc, BH, Nq, Nk, D, nsel, cap, idx, cnt, st, why);
    }
}

}  // namespace lcbsa
