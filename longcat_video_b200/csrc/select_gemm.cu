// Block-select stage, parts 2 and 3, two-kernel form: block scores as a register-tiled fp32 GEMM, then per-row top-k.
//
// Replaces cal_score + get_select_indices_topk_from_score
// (longcat_video/block_sparse_attention/bsa_interface.py:180-184, 212-224) like select.cu does, with the same
// arithmetic:  score(i,j) = fp32 FMA chain over d = 0..D-1 (ascending), rounded to the input dtype.  The FMA pipe
// can only be kept busy if every operand word read from shared memory feeds several FMAs (shared memory hands a
// warp 32 words per cycle, the FMA pipes take 128 lanes per cycle), and that needs a two-dimensional register
// tile: here 8 x 8 scores per thread, 128 x 128 per CTA, 16 FMAs per 128-bit operand read.  A tile of that shape
// cannot keep whole rows of scores on chip, so the rounded scores go to a workspace as order-preserving 16-bit keys
// (2 bytes per score, written once and read once: 0.27 GB of traffic at 720p with 32 heads) and a second kernel
// selects per row, one warp per row with the row in registers.  Used by lcbsa_block_select when the caller's
// workspace has room for the keys; otherwise the fused kernel of select.cu runs.
#include "select_common.cuh"

namespace lcbsa {

namespace {

using namespace sel;

constexpr int kTile = 128;          // scores per CTA: kTile x kTile
constexpr int kBK = 16;             // head-dimension elements per shared-memory slab
constexpr int kPitch = kTile + 4;   // slab row pitch in floats
constexpr int kGemmThreads = 256;   // 16 x 16 threads, 8 x 8 scores each

// q: [BH, Nq, D], k: [BH, Nk, D] pooled rows in the input dtype; keys: [BH, Nq, nk_pad]
template <typename T, int D>
__global__ void __launch_bounds__(kGemmThreads, 2) score_gemm_kernel(const T* __restrict__ qc, const T* __restrict__ kc, int Nq, int Nk,
                                                                    int nk_pad, uint16_t* __restrict__ keys) {
    static_assert(sizeof(T) == 2 && D % kBK == 0, "16-bit inputs, head_dim a multiple of 16");
    __shared__ __align__(16) float qs[2][kBK][kPitch];  // [slab][d][row]: transposed, so that a thread's rows are contiguous
    __shared__ __align__(16) float ks[2][kBK][kPitch];

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int bh = blockIdx.z;
    const int i0 = blockIdx.y * kTile, j0 = blockIdx.x * kTile;
    const T* qbase = qc + (long long)bh * Nq * D;
    const T* kbase = kc + (long long)bh * Nk * D;

    // global -> registers: thread t brings 8 consecutive d of row t / 2 of the Q tile and of the K tile
    const int lrow = tid >> 1, ldh = (tid & 1) * 8;
    const bool q_ok = i0 + lrow < Nq, k_ok = j0 + lrow < Nk;
    const T* qsrc = qbase + (long long)(q_ok ? i0 + lrow : 0) * D + ldh;
    const T* ksrc = kbase + (long long)(k_ok ? j0 + lrow : 0) * D + ldh;
    uint4 qpre, kpre;
    auto fetch = [&](int slab) {
        qpre = q_ok ? __ldg(reinterpret_cast<const uint4*>(qsrc + slab * kBK)) : make_uint4(0u, 0u, 0u, 0u);
        kpre = k_ok ? __ldg(reinterpret_cast<const uint4*>(ksrc + slab * kBK)) : make_uint4(0u, 0u, 0u, 0u);
    };
    auto stash = [&](int buf) {
        const T* qe = reinterpret_cast<const T*>(&qpre);
        const T* ke = reinterpret_cast<const T*>(&kpre);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            qs[buf][ldh + i][lrow] = DType<T>::to_f32(qe[i]);
            ks[buf][ldh + i][lrow] = DType<T>::to_f32(ke[i]);
        }
    };

    // this thread's scores: rows {4 ty .. 4 ty + 3, 64 + 4 ty ..}, columns {4 tx .. 4 tx + 3, 64 + 4 tx ..}
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    fetch(0);
    stash(0);
    __syncthreads();
    constexpr int kSlabs = D / kBK;
#pragma unroll 1
    for (int slab = 0; slab < kSlabs; ++slab) {
        const int buf = slab & 1;
        if (slab + 1 < kSlabs) fetch(slab + 1);
#pragma unroll
        for (int d = 0; d < kBK; ++d) {  // ascending d: every score is one chain acc = fmaf(q[d], k[d], acc)
            const float4 qa = *reinterpret_cast<const float4*>(&qs[buf][d][4 * ty]);
            const float4 qb = *reinterpret_cast<const float4*>(&qs[buf][d][64 + 4 * ty]);
            const float4 ka = *reinterpret_cast<const float4*>(&ks[buf][d][4 * tx]);
            const float4 kb = *reinterpret_cast<const float4*>(&ks[buf][d][64 + 4 * tx]);
            const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            const float kv[8] = {ka.x, ka.y, ka.z, ka.w, kb.x, kb.y, kb.z, kb.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
        }
        if (slab + 1 < kSlabs) stash(buf ^ 1);
        __syncthreads();
    }

    // rounded scores -> keys; columns past Nk get the smallest key, columns past nk_pad do not exist
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = i0 + (i < 4 ? 4 * ty + i : 64 + 4 * ty + (i - 4));
        if (row >= Nq) continue;
        uint16_t* out = keys + ((long long)bh * Nq + row) * nk_pad;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int col = j0 + 64 * h + 4 * tx;
            if (col >= nk_pad) continue;  // nk_pad is a multiple of 64, so a group of four columns is all in or all out
            uint16_t kk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) kk[j] = (col + j < Nk) ? make_key(DType<T>::from_f32(acc[i][4 * h + j])) : (uint16_t)0;
            uint2 pk;
            pk.x = (uint32_t)kk[0] | ((uint32_t)kk[1] << 16);
            pk.y = (uint32_t)kk[2] | ((uint32_t)kk[3] << 16);
            *reinterpret_cast<uint2*>(out + col) = pk;
        }
    }
}

// one warp per row of keys
__global__ void __launch_bounds__(256) topk_rows_kernel(const uint16_t* __restrict__ keys, long long rows, int Nk, int nk_pad, int nsel,
                                                       int cap, int32_t* __restrict__ idx, int32_t* __restrict__ cnt) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    select_row<uint16_t>(keys + row * nk_pad, Nk, nk_pad, nsel, cap, idx + row * cap, cnt + row, lane);
}

// The same for a grid with a "first part" (the conditioning frames of video continuation): query blocks of the first
// part take nsel_first blocks among the key blocks of the first part, all other query blocks nsel blocks among all.
__global__ void __launch_bounds__(256) topk_rows_split_kernel(const uint16_t* __restrict__ keys, long long rows, int Nq, int Nk, int nk_pad,
                                                             SelectSplit sp, int nsel, int cap, int32_t* __restrict__ idx,
                                                             int32_t* __restrict__ cnt) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int qblk = (int)(row % Nq);
    const bool first = ((qblk / sp.hw_q) % sp.period_q) < sp.split_q;
    const KeyMask mask{sp.hw_k, first ? sp.period_k : 0, sp.split_k};
    select_row<uint16_t>(keys + row * nk_pad, Nk, nk_pad, first ? sp.nsel_first : nsel, cap, idx + row * cap, cnt + row, lane, mask);
}

template <typename T, int D>
cudaError_t launch_gemm(const void* qc, const void* kc, int BH, int Nq, int Nk, int nk_pad, uint16_t* keys, cudaStream_t st) {
    dim3 grid((nk_pad + kTile - 1) / kTile, (Nq + kTile - 1) / kTile, BH);
    score_gemm_kernel<T, D><<<grid, kGemmThreads, 0, st>>>(reinterpret_cast<const T*>(qc), reinterpret_cast<const T*>(kc), Nq, Nk, nk_pad, keys);
    return cudaGetLastError();
}

}  // namespace

size_t score_keys_bytes(int dtype, int BH, int Nq, int Nk, int D) {
    if (dtype == LCBSA_FP32 || (D != 64 && D != 128) || BH > 65535) return 0;  // this form does not apply
    const size_t nk_pad = ((size_t)Nk + 63) / 64 * 64;
    return (size_t)BH * Nq * nk_pad * sizeof(uint16_t);
}

// scores only: the 16-bit keys of all [BH, Nq, Nk] scores into keys_ws (score_keys_bytes(...) bytes)
cudaError_t launch_score_keys(int dtype, const void* qc, const void* kc, int BH, int Nq, int Nk, int D, void* keys_ws, cudaStream_t st,
                              const char** why) {
    if (BH == 0 || Nq == 0) return cudaSuccess;
    if (score_keys_bytes(dtype, BH, Nq, Nk, D) == 0) {
        *why = "the score kernel takes bf16 or fp16 with head_dim 64 or 128";
        return cudaErrorInvalidValue;
    }
    const int nk_pad = (Nk + 63) / 64 * 64;
    uint16_t* keys = static_cast<uint16_t*>(keys_ws);
    if (dtype == LCBSA_BF16)
        return D == 128 ? launch_gemm<__nv_bfloat16, 128>(qc, kc, BH, Nq, Nk, nk_pad, keys, st)
                        : launch_gemm<__nv_bfloat16, 64>(qc, kc, BH, Nq, Nk, nk_pad, keys, st);
    return D == 128 ? launch_gemm<__half, 128>(qc, kc, BH, Nq, Nk, nk_pad, keys, st) : launch_gemm<__half, 64>(qc, kc, BH, Nq, Nk, nk_pad, keys, st);
}

cudaError_t launch_score_gemm_topk(int dtype, const void* qc, const void* kc, int BH, int Nq, int Nk, int D, int nsel, int cap,
                                   int32_t* idx, int32_t* cnt, void* keys_ws, cudaStream_t st, const char** why, const SelectSplit* split) {
    if (BH == 0 || Nq == 0) return cudaSuccess;
    if (score_keys_bytes(dtype, BH, Nq, Nk, D) == 0) {
        *why = "the two-kernel form takes bf16 or fp16 with head_dim 64 or 128";
        return cudaErrorInvalidValue;
    }
    const int nk_pad = (Nk + 63) / 64 * 64;
    uint16_t* keys = static_cast<uint16_t*>(keys_ws);
    cudaError_t e;
    if (dtype == LCBSA_BF16)
        e = D == 128 ? launch_gemm<__nv_bfloat16, 128>(qc, kc, BH, Nq, Nk, nk_pad, keys, st)
                     : launch_gemm<__nv_bfloat16, 64>(qc, kc, BH, Nq, Nk, nk_pad, keys, st);
    else
        e = D == 128 ? launch_gemm<__half, 128>(qc, kc, BH, Nq, Nk, nk_pad, keys, st) : launch_gemm<__half, 64>(qc, kc, BH, Nq, Nk, nk_pad, keys, st);
    if (e != cudaSuccess) return e;
    const long long rows = (long long)BH * Nq;
    if (split != nullptr) {
        if (nk_pad > 2 * 32 * kRegWords) {
            *why = "the split selection handles up to 1536 key blocks";
            return cudaErrorInvalidValue;
        }
        topk_rows_split_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(keys, rows, Nq, Nk, nk_pad, *split, nsel, cap, idx, cnt);
    } else {
        topk_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(keys, rows, Nk, nk_pad, nsel, cap, idx, cnt);
    }
    return cudaGetLastError();
}

}  // namespace lcbsa
