// The step immediately before the BSA path: RMSNorm (fp32) of q and k over the head dimension, times the learned
// weight, then the 3-D rotary embedding, written straight into the [B, H, S, D] layout the attention (or the Ulysses
// exchange) reads.
//
// Replaces, for q and k each (longcat_video/modules/attention.py:113-121):
//   RMSNorm_FP32.forward   (longcat_video/modules/blocks.py:42-53)
//   RotaryPositionalEmbedding.forward   (longcat_video/modules/rope_3d.py:99-120)
// which in the reference are six elementwise passes over q and k with fp32 temporaries.  Here it is one pass:
// every input element is read once from the strided view of the fused qkv projection and every output element
// written once.  HBM-bound: 2 bytes in + 2 bytes out per element.
//
// Eight lanes per token: a lane owns D/8 consecutive elements (whole rotation pairs, two 16-byte loads at
// head_dim 128), a warp works on four neighbouring tokens and walks over a group of heads, so that the position
// arithmetic, the angles and the weights are set up once and stay in registers, and every warp instruction of the
// row arithmetic serves four rows (the kernel is bound by instruction issue as much as by HBM: at the HBM rate an
// SM has about 90 issue slots per 256-byte row).
// Arithmetic, in the order the CPU oracle fixes it: per-lane sum of squares with fmaf in ascending order, butterfly
// over the 8 lanes (xor 4, 2, 1), mean = sum / D, 1 / sqrtf(mean + eps) correctly rounded, y = T(x * r),
// z = T(y * w) (one packed multiply in the storage type: the product of two 8- or 11-bit significands is exact in
// fp32, so rounding it once is the same thing), out = T(z * cos + rot(z) * sin) with the two products rounded
// separately.
//
// The rotary angles depend on t for the first D - 4*(D/6) elements of the head dimension, on h for the next
// 2*(D/6) and on w for the last 2*(D/6) (rope_3d.py:62-84), so the [S, D] cos/sin tables of the reference factor
// into three small ones, [T, dt], [H, dh], [W, dw]; both elements of a pair have the same angle (rope_3d.py:113-115).
#include "common.cuh"

namespace lcbsa {

namespace {

constexpr int kWarps = 8;         // warps per CTA, four tokens each
constexpr int kTokens = 4;        // tokens per warp: eight lanes each
constexpr int kHeadsPerCta = 16;  // heads one warp walks over

// Two values of the storage type in one 32-bit word: rounding two floats costs one packed conversion.
template <typename T>
struct Pair;
template <>
struct Pair<__nv_bfloat16> {
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&t);
    }
    __device__ static __forceinline__ void unpack(uint32_t u, float& lo, float& hi) {
        lo = __uint_as_float(u << 16);
        hi = __uint_as_float(u & 0xffff0000u);
    }
    __device__ static __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {  // round(a * b) per half, one rounding
        const __nv_bfloat162 t = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
        return *reinterpret_cast<const uint32_t*>(&t);
    }
};
template <>
struct Pair<__half> {
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        const __half2 t = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&t);
    }
    __device__ static __forceinline__ void unpack(uint32_t u, float& lo, float& hi) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
        lo = f.x;
        hi = f.y;
    }
    __device__ static __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
        const __half2 t = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&t);
    }
};

// NORM: RMSNorm times weight (off: the input is already normalised, e.g. cached keys); ROPE: the rotary embedding
// (off: normalised q / k as they are cached before the embedding, attention.py:118-119).  The token at grid position
// (t, h, w) takes the angles of frame t + t_off; tab_t is the number of frames the table holds (>= T + t_off).
template <typename T, int D, bool NORM, bool ROPE>
__global__ void __launch_bounds__(kWarps * 32) norm_rope_kernel(View x, int H, int S, int tab_t, int t_off, int Hg, int Wg,
                                                               const T* __restrict__ weight, const float* __restrict__ tab, float eps, T* out,
                                                               long long osb, long long osh, long long oss) {
    constexpr int PER = D / 8;   // elements per lane: 16 or 8
    constexpr int NV = PER / 8;  // 16-byte vectors per lane
    constexpr int NP = PER / 2;  // rotation pairs per lane
    static_assert(PER == 8 || PER == 16, "a lane owns one or two 16-byte vectors");
    constexpr int DH = 2 * (D / 6), DW = DH, DT = D - DH - DW;
    const int lane = threadIdx.x & 31, sub = lane & 7, tok = lane >> 3;
    const long long first = ((long long)blockIdx.x * kWarps + (threadIdx.x >> 5)) * kTokens;  // the warp's first token
    if (first >= S) return;
    const bool live = first + tok < S;  // the last warp may have fewer than four tokens
    const int s = live ? (int)(first + tok) : S - 1;
    const int b = blockIdx.z;
    const int h0 = blockIdx.y * kHeadsPerCta, h1 = min(H, h0 + kHeadsPerCta);
    const int w_pos = s % Wg, h_pos = (s / Wg) % Hg, t_pos = s / (Wg * Hg) + t_off;

    // table layout: cos_t [T, DT] sin_t [T, DT] cos_h [H, DH] sin_h [H, DH] cos_w [W, DW] sin_w [W, DW]
    const float* cos_t = tab;
    const float* sin_t = cos_t + (long long)tab_t * DT;
    const float* cos_h = sin_t + (long long)tab_t * DT;
    const float* sin_h = cos_h + (long long)Hg * DH;
    const float* cos_w = sin_h + (long long)Hg * DH;
    const float* sin_w = cos_w + (long long)Wg * DW;
    float cs[NP], sn[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) {
        const int d = sub * PER + 2 * p;  // even: d and d + 1 are one rotation pair and lie in the same part
        const float *c, *n;
        if (d < DT) {
            c = cos_t + t_pos * DT + d; n = sin_t + t_pos * DT + d;
        } else if (d < DT + DH) {
            c = cos_h + h_pos * DH + (d - DT); n = sin_h + h_pos * DH + (d - DT);
        } else {
            c = cos_w + w_pos * DW + (d - DT - DH); n = sin_w + w_pos * DW + (d - DT - DH);
        }
        cs[p] = ROPE ? __ldg(c) : 1.0f;
        sn[p] = ROPE ? __ldg(n) : 0.0f;
    }
    uint4 wv[NV];  // the lane's weights, packed as they are stored
#pragma unroll
    for (int j = 0; j < NV; ++j) wv[j] = NORM ? __ldg(reinterpret_cast<const uint4*>(weight + sub * PER) + j) : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t* wp = reinterpret_cast<const uint32_t*>(wv);

    const T* sp = reinterpret_cast<const T*>(x.data) + (long long)b * x.sb + (long long)s * x.ss + (long long)h0 * x.sh + sub * PER;
    T* dp = out + (long long)b * osb + (long long)s * oss + (long long)h0 * osh + sub * PER;
    uint4 cur[NV], nxt[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) cur[j] = reinterpret_cast<const uint4*>(sp)[j];
#pragma unroll 1
    for (int h = h0; h < h1; ++h) {
        sp += x.sh;
        if (h + 1 < h1) {  // the next head's row is in flight during the arithmetic
#pragma unroll
            for (int j = 0; j < NV; ++j) nxt[j] = reinterpret_cast<const uint4*>(sp)[j];
        }
        const uint32_t* cw = reinterpret_cast<const uint32_t*>(cur);
        float rinv = 1.0f;
        if (NORM) {
            float v[PER];
#pragma unroll
            for (int p = 0; p < NP; ++p) Pair<T>::unpack(cw[p], v[2 * p], v[2 * p + 1]);
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < PER; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
            const float mean = __fmul_rn(ss, 1.0f / (float)D);
            rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
        }
        uint4 res[NV];
        uint32_t* rw = reinterpret_cast<uint32_t*>(res);
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            uint32_t z = cw[p];
            if (NORM) {
                float v0, v1;
                Pair<T>::unpack(cw[p], v0, v1);
                z = Pair<T>::mul(Pair<T>::pack(__fmul_rn(v0, rinv), __fmul_rn(v1, rinv)), wp[p]);
            }
            if (ROPE) {
                float z0, z1;
                Pair<T>::unpack(z, z0, z1);
                z = Pair<T>::pack(__fadd_rn(__fmul_rn(z0, cs[p]), __fmul_rn(-z1, sn[p])),
                                  __fadd_rn(__fmul_rn(z1, cs[p]), __fmul_rn(z0, sn[p])));
            }
            rw[p] = z;
        }
        if (live) {
#pragma unroll
            for (int j = 0; j < NV; ++j) reinterpret_cast<uint4*>(dp)[j] = res[j];
        }
        dp += osh;
#pragma unroll
        for (int j = 0; j < NV; ++j) cur[j] = nxt[j];
    }
}

template <typename T, int D, bool NORM, bool ROPE>
cudaError_t run(const View& x, int B, int H, int S, int tab_t, int t_off, int Hg, int Wg, const void* weight, const float* tab, float eps,
                void* out, long long osb, long long osh, long long oss, cudaStream_t st) {
    if ((long long)B * H * S == 0) return cudaSuccess;
    dim3 grid((unsigned)((S + kTokens * kWarps - 1) / (kTokens * kWarps)), (unsigned)((H + kHeadsPerCta - 1) / kHeadsPerCta), (unsigned)B);
    norm_rope_kernel<T, D, NORM, ROPE><<<grid, kWarps * 32, 0, st>>>(x, H, S, tab_t, t_off, Hg, Wg, reinterpret_cast<const T*>(weight), tab,
                                                                    eps, reinterpret_cast<T*>(out), osb, osh, oss);
    return cudaGetLastError();
}

template <typename T, int D>
cudaError_t pick(bool norm, bool rope, const View& x, int B, int H, int S, int tab_t, int t_off, int Hg, int Wg, const void* weight,
                 const float* tab, float eps, void* out, long long osb, long long osh, long long oss, cudaStream_t st) {
    if (norm && rope) return run<T, D, true, true>(x, B, H, S, tab_t, t_off, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st);
    if (norm) return run<T, D, true, false>(x, B, H, S, tab_t, t_off, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st);
    return run<T, D, false, true>(x, B, H, S, tab_t, t_off, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st);
}

}  // namespace

size_t rope_table_floats(int Tg, int Hg, int Wg, int D) {
    const int dh = 2 * (D / 6), dt = D - 2 * dh;
    return 2 * ((size_t)Tg * dt + (size_t)Hg * dh + (size_t)Wg * dh);
}

// weight == nullptr: no normalisation; tab == nullptr: no rotary embedding (not both)
cudaError_t launch_norm_rope(int dtype, const View& x, int B, int H, int S, int D, int tab_t, int t_off, int Hg, int Wg, const void* weight,
                             const float* tab, float eps, void* out, long long osb, long long osh, long long oss, cudaStream_t st,
                             const char** why) {
    if (dtype == LCBSA_FP32 || (D != 64 && D != 128)) {
        *why = "norm_rope takes bf16 or fp16 with head_dim 64 or 128";
        return cudaErrorInvalidValue;
    }
    if (B > 65535) {
        *why = "norm_rope: batch above 65535";
        return cudaErrorInvalidValue;
    }
    const bool norm = weight != nullptr, rope = tab != nullptr;
    if (!norm && !rope) {
        *why = "norm_rope: neither a weight nor a rope table";
        return cudaErrorInvalidValue;
    }
    if (dtype == LCBSA_BF16)
        return D == 128 ? pick<__nv_bfloat16, 128>(norm, rope, x, B, H, S, tab_t, t_off, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st)
                        : pick<__nv_bfloat16, 64>(norm, rope, x, B, H, S, tab_t, t_off, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st);
    return D == 128 ? pick<__half, 128>(norm, rope, x, B, H, S, tab_t, t_off, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st)
                    : pick<__half, 64>(norm, rope, x, B, H, S, tab_t, t_off, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st);
}

}  // namespace lcbsa
