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

// One tensor to pool and where its rows go.
//   plain   (n_dst == 0): dense [B*H, nblk, D] at dst[0].
//   scatter (n_dst  > 0): head h belongs to rank h / heads_per_dst; its rows go to that rank's buffer dst[h / heads_per_dst]
//                         (this GPU's own memory or a peer's, mapped into this process) laid out
//                         [heads_per_dst][n_dst source ranks][nblk][D], this rank filling source slot src_rank --
//                         which is the dense [heads_per_dst, n_dst * nblk, D] pooled tensor of the gathered,
//                         rank-major sequence on the receiving side.  B must be 1.
struct PoolJob {
    View x;
    Geom g;
    long long groups;  // B * H * nblk
    void* dst[kPoolMaxDst];
    int n_dst, heads_per_dst, src_rank;
};

template <typename T, int VEC>
__global__ void __launch_bounds__(256, 4) pool_kernel(const __grid_constant__ PoolJob j0, const __grid_constant__ PoolJob j1, int H, int D, int lpr) {
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long group = gtid / lpr;
    const int lane = (int)(gtid % lpr);
    const bool second = group >= j0.groups;
    if (second) group -= j0.groups;
    const PoolJob& job = second ? j1 : j0;
    if (group >= job.groups) return;
    const View& x = job.x;
    const Geom& g = job.g;
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
    T* out;
    long long row;
    if (job.n_dst == 0) {
        out = reinterpret_cast<T*>(job.dst[0]);
        row = bh * g.nblk + blk;
    } else {
        const int owner = h / job.heads_per_dst, hl = h % job.heads_per_dst;
        out = reinterpret_cast<T*>(job.dst[owner]);
        row = ((long long)hl * job.n_dst + job.src_rank) * g.nblk + blk;
    }
    *reinterpret_cast<uint4*>(out + row * D + lane * VEC) = o;
}

template <typename T>
cudaError_t run(const PoolJob& j0, const PoolJob& j1, int H, int D, cudaStream_t st) {
    constexpr int VEC = 16 / sizeof(T);
    const int lpr = D / VEC;
    const long long threads = (j0.groups + j1.groups) * lpr;
    const int block = 256;
    const long long grid = (threads + block - 1) / block;
    if (grid == 0) return cudaSuccess;
    pool_kernel<T, VEC><<<(unsigned)grid, block, 0, st>>>(j0, j1, H, D, lpr);
    return cudaGetLastError();
}

PoolJob make_job(const View& x, int B, int H, const Geom& g, const PoolDst& d) {
    PoolJob j;
    j.x = x;
    j.g = g;
    j.groups = (long long)B * H * g.nblk;
    for (int i = 0; i < kPoolMaxDst; ++i) j.dst[i] = d.dst[i];
    j.n_dst = d.n_dst;
    j.heads_per_dst = d.heads_per_dst;
    j.src_rank = d.src_rank;
    return j;
}

}  // namespace

cudaError_t launch_pool2(int dtype, const View& x0, const Geom& g0, const PoolDst& d0, const View* x1, const Geom* g1, const PoolDst* d1,
                         int B, int H, int D, cudaStream_t st) {
    const PoolJob j0 = make_job(x0, B, H, g0, d0);
    PoolJob j1 = j0;
    j1.groups = 0;
    if (x1 != nullptr) j1 = make_job(*x1, B, H, *g1, *d1);
    switch (dtype) {
        case LCBSA_BF16: return run<__nv_bfloat16>(j0, j1, H, D, st);
        case LCBSA_FP16: return run<__half>(j0, j1, H, D, st);
        default: return run<float>(j0, j1, H, D, st);
    }
}

cudaError_t launch_pool(int dtype, const View& x, int B, int H, int D, const Geom& g, void* out, cudaStream_t st) {
    PoolDst d{};
    d.dst[0] = out;
    return launch_pool2(dtype, x, g, d, nullptr, nullptr, nullptr, B, H, D, st);
}

}  // namespace lcbsa
