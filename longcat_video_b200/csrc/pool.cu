// Block-select stage, part 1: mean-pool Q or K over every 3-D token block.
//
// Replaces rearrange_THW_to_3d_block + mean_pooling_compression
// (longcat_video/block_sparse_attention/bsa_interface.py:600-604, 168-178): the block's tokens are
// addressed in place through the tensor's strides, so no rearranged copy is made.
//
// HBM-bound: every input byte is read exactly once with 128-bit loads.  A group of D*sizeof(T)/16
// lanes owns one block; each lane keeps a 16-byte column slice and walks the block's tokens in
// (t,h,w) order, so the fp32 running sum has a fixed, documented order:
//   sum over present tokens in slot order -> * fp32(1/block_size) -> round-to-nearest-even to T.
#include "common.cuh"

namespace lcbsa {

namespace {

constexpr int kBatch = 8;  // independent 16-byte loads in flight per lane (64 registers: four CTAs per SM; measured 5.1 TB/s against 4.5 with 16)

template <typename T, int VEC>
__global__ void __launch_bounds__(256, 4) pool_kernel(View x, int H, int D, Geom g, T* __restrict__ out, int lpr,
                                                    long long total_groups) {
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long group = gtid / lpr;
    const int lane = (int)(gtid % lpr);
    if (group >= total_groups) return;
    const int blk = (int)(group % g.nblk);
    const long long bh = group / g.nblk;
    const int b = (int)(bh / H), h = (int)(bh % H);

    int bt, bhh, bw;
    block_coords(g, blk, bt, bhh, bw);
    const int t0 = bt * g.ct, h0 = bhh * g.ch, w0 = bw * g.cw;
    const T* base = reinterpret_cast<const T*>(x.data) + (long long)b * x.sb + (long long)h * x.sh + lane * VEC;

    float acc[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[e] = 0.f;

    int lt = 0, lh = 0, lw = 0;  // coordinates of slot r inside the block
    for (int r0 = 0; r0 < g.bs; r0 += kBatch) {
        uint4 buf[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            buf[u] = make_uint4(0u, 0u, 0u, 0u);
            if (r0 + u < g.bs) {
                const int t = t0 + lt, hh = h0 + lh, w = w0 + lw;
                if (t < g.T && hh < g.H && w < g.W) {
                    const long long tok = ((long long)t * g.H + hh) * g.W + w;
                    buf[u] = __ldg(reinterpret_cast<const uint4*>(base + tok * x.ss));
                }
                if (++lw == g.cw) {
                    lw = 0;
                    if (++lh == g.ch) {
                        lh = 0;
                        ++lt;
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const T* e8 = reinterpret_cast<const T*>(&buf[u]);
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = acc[e] + DType<T>::to_f32(e8[e]);
        }
    }

    const float inv = 1.0f / (float)g.bs;
    uint4 o;
    T* o8 = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int e = 0; e < VEC; ++e) o8[e] = DType<T>::from_f32(acc[e] * inv);
    *reinterpret_cast<uint4*>(out + ((long long)bh * g.nblk + blk) * D + lane * VEC) = o;
}

template <typename T>
cudaError_t run(const View& x, int B, int H, int D, const Geom& g, void* out, cudaStream_t st) {
    constexpr int VEC = 16 / sizeof(T);
    const int lpr = D / VEC;
    const long long groups = (long long)B * H * g.nblk;
    const long long threads = groups * lpr;
    const int block = 256;
    const long long grid = (threads + block - 1) / block;
    if (grid == 0) return cudaSuccess;
    pool_kernel<T, VEC><<<(unsigned)grid, block, 0, st>>>(x, H, D, g, reinterpret_cast<T*>(out), lpr, groups);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_pool(int dtype, const View& x, int B, int H, int D, const Geom& g, void* out, cudaStream_t st) {
    switch (dtype) {
        case LCBSA_BF16: return run<__nv_bfloat16>(x, B, H, D, g, out, st);
        case LCBSA_FP16: return run<__half>(x, B, H, D, g, out, st);
        default: return run<float>(x, B, H, D, g, out, st);
    }
}

}  // namespace lcbsa
