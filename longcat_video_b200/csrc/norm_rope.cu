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
// One warp per (batch, head, token) row; a lane owns D/32 consecutive elements, i.e. whole rotation pairs.
// Arithmetic, in the order the CPU oracle fixes it: per-lane sum of squares with fmaf in ascending order, butterfly
// over the lanes (xor 16, 8, 4, 2, 1), mean = sum / D, 1 / sqrtf(mean + eps) correctly rounded, y = T(x * r),
// z = T(y * w), out = T(z * cos + rot(z) * sin) with the two products rounded separately.
//
// The rotary angles depend on t for the first D - 4*(D/6) elements of the head dimension, on h for the next
// 2*(D/6) and on w for the last 2*(D/6) (rope_3d.py:62-84), so the [S, D] cos/sin tables of the reference factor
// into three small ones, [T, dt], [H, dh], [W, dw], that stay in L1.
#include "common.cuh"

namespace lcbsa {

namespace {

constexpr int kRowsPerCta = 8;  // one warp per row

template <typename T, int D>
__global__ void __launch_bounds__(kRowsPerCta * 32) norm_rope_kernel(View x, int H, int S, int Tg, int Hg, int Wg, const T* __restrict__ weight,
                                                                    const float* __restrict__ tab, float eps, T* __restrict__ out,
                                                                    long long osb, long long osh, long long oss, long long rows) {
    constexpr int PER = D / 32;
    static_assert(PER >= 2 && PER % 2 == 0, "a lane owns whole rotation pairs");
    constexpr int DH = 2 * (D / 6), DW = DH, DT = D - DH - DW;
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * kRowsPerCta + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int s = (int)(row % S);
    const long long bh = row / S;
    const int h = (int)(bh % H), b = (int)(bh / H);
    const int w_pos = s % Wg, h_pos = (s / Wg) % Hg, t_pos = s / (Wg * Hg);

    const T* src = reinterpret_cast<const T*>(x.data) + (long long)b * x.sb + (long long)h * x.sh + (long long)s * x.ss + lane * PER;
    float v[PER];
    if (PER == 4) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < PER; ++i) v[i] = DType<T>::to_f32(e[i]);
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) v[i] = DType<T>::to_f32(src[i]);
    }
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    const float mean = __fmul_rn(ss, 1.0f / (float)D);
    const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));

    // table layout: cos_t [T, DT] sin_t [T, DT] cos_h [H, DH] sin_h [H, DH] cos_w [W, DW] sin_w [W, DW]
    const float* cos_t = tab;
    const float* sin_t = cos_t + (long long)Tg * DT;
    const float* cos_h = sin_t + (long long)Tg * DT;
    const float* sin_h = cos_h + (long long)Hg * DH;
    const float* cos_w = sin_h + (long long)Hg * DH;
    const float* sin_w = cos_w + (long long)Wg * DW;

    T res[PER];
#pragma unroll
    for (int i = 0; i < PER; i += 2) {
        const int d = lane * PER + i;  // even: d and d + 1 are one rotation pair and lie in the same part
        float c0, c1, s0, s1;
        if (d < DT) {
            c0 = cos_t[t_pos * DT + d]; c1 = cos_t[t_pos * DT + d + 1];
            s0 = sin_t[t_pos * DT + d]; s1 = sin_t[t_pos * DT + d + 1];
        } else if (d < DT + DH) {
            c0 = cos_h[h_pos * DH + d - DT]; c1 = cos_h[h_pos * DH + d - DT + 1];
            s0 = sin_h[h_pos * DH + d - DT]; s1 = sin_h[h_pos * DH + d - DT + 1];
        } else {
            c0 = cos_w[w_pos * DW + d - DT - DH]; c1 = cos_w[w_pos * DW + d - DT - DH + 1];
            s0 = sin_w[w_pos * DW + d - DT - DH]; s1 = sin_w[w_pos * DW + d - DT - DH + 1];
        }
        const float y0 = DType<T>::to_f32(DType<T>::from_f32(__fmul_rn(v[i], rinv)));
        const float y1 = DType<T>::to_f32(DType<T>::from_f32(__fmul_rn(v[i + 1], rinv)));
        const float z0 = DType<T>::to_f32(DType<T>::from_f32(__fmul_rn(y0, DType<T>::to_f32(weight[d]))));
        const float z1 = DType<T>::to_f32(DType<T>::from_f32(__fmul_rn(y1, DType<T>::to_f32(weight[d + 1]))));
        res[i] = DType<T>::from_f32(__fadd_rn(__fmul_rn(z0, c0), __fmul_rn(-z1, s0)));
        res[i + 1] = DType<T>::from_f32(__fadd_rn(__fmul_rn(z1, c1), __fmul_rn(z0, s1)));
    }
    T* dst = out + (long long)b * osb + (long long)h * osh + (long long)s * oss + lane * PER;
    if (PER == 4) {
        *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(res);
    } else {
#pragma unroll
        for (int i = 0; i < PER; ++i) dst[i] = res[i];
    }
}

template <typename T, int D>
cudaError_t run(const View& x, int B, int H, int S, int Tg, int Hg, int Wg, const void* weight, const float* tab, float eps, void* out,
                long long osb, long long osh, long long oss, cudaStream_t st) {
    const long long rows = (long long)B * H * S;
    if (rows == 0) return cudaSuccess;
    const long long grid = (rows + kRowsPerCta - 1) / kRowsPerCta;
    norm_rope_kernel<T, D><<<(unsigned)grid, kRowsPerCta * 32, 0, st>>>(x, H, S, Tg, Hg, Wg, reinterpret_cast<const T*>(weight), tab, eps,
                                                                       reinterpret_cast<T*>(out), osb, osh, oss, rows);
    return cudaGetLastError();
}

}  // namespace

size_t rope_table_floats(int Tg, int Hg, int Wg, int D) {
    const int dh = 2 * (D / 6), dt = D - 2 * dh;
    return 2 * ((size_t)Tg * dt + (size_t)Hg * dh + (size_t)Wg * dh);
}

cudaError_t launch_norm_rope(int dtype, const View& x, int B, int H, int S, int D, int Tg, int Hg, int Wg, const void* weight,
                             const float* tab, float eps, void* out, long long osb, long long osh, long long oss, cudaStream_t st,
                             const char** why) {
    if (dtype == LCBSA_FP32 || (D != 64 && D != 128)) {
        *why = "norm_rope takes bf16 or fp16 with head_dim 64 or 128";
        return cudaErrorInvalidValue;
    }
    if (dtype == LCBSA_BF16)
        return D == 128 ? run<__nv_bfloat16, 128>(x, B, H, S, Tg, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st)
                        : run<__nv_bfloat16, 64>(x, B, H, S, Tg, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st);
    return D == 128 ? run<__half, 128>(x, B, H, S, Tg, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st)
                    : run<__half, 64>(x, B, H, S, Tg, Hg, Wg, weight, tab, eps, out, osb, osh, oss, st);
}

}  // namespace lcbsa
