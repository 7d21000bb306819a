// Shared by the kernels that run on warp-level MMA (attn_mma.cu: the generic forward; attn_bwd.cu: the backward):
// cp.async / ldmatrix / mma.sync wrappers, the gather of a 3-D block's slots into a swizzled shared-memory tile.
#pragma once
#include "common.cuh"

namespace lcbsa {
namespace mm {

struct SlotEntry {
    int off;     // token offset of the slot relative to the block's first token
    int packed;  // lt | lh << 10 | lw << 20
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
    const int n = pred ? 16 : 0;  // src-size 0 -> the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <typename T> __device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(__nv_bfloat16, float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t pack2(__half, float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ bool slot_present(const Geom& g, int packed, int t0, int h0, int w0) {
    return (t0 + (packed & 1023) < g.T) && (h0 + ((packed >> 10) & 1023) < g.H) && (w0 + (packed >> 20) < g.W);
}

// Gather ROWS block slots (starting at slot0) of block `blk` into a swizzled [ROWS][D] tile.
template <typename T, int D, int ROWS, int NTHREADS>
__device__ __forceinline__ void load_tile(unsigned char* tile, const T* head_base, long long ss, const Geom& g,
                                          const SlotEntry* tab, int blk, int slot0, int tid) {
    constexpr int CPR = D * 2 / 16;  // 16-byte chunks per row
    int bt, bh, bw;
    // a block number outside the grid (a caller's list may hold anything) is never turned into an address:
    // the whole tile is zero-filled and the caller of load_tile masks the block out of the softmax
    const bool blk_ok = (unsigned)blk < (unsigned)g.nblk;
    block_coords(g, blk_ok ? blk : 0, bt, bh, bw);
    const int t0 = bt * g.ct, h0 = bh * g.ch, w0 = bw * g.cw;
    const long long origin = ((long long)t0 * g.H + h0) * g.W + w0;
    const uint32_t sbase = smem_u32(tile);
#pragma unroll
    for (int v = tid; v < ROWS * CPR; v += NTHREADS) {
        const int row = v / CPR, c = v % CPR;
        const SlotEntry e = tab[slot0 + row];
        const bool present = blk_ok && (!g.ragged || slot_present(g, e.packed, t0, h0, w0));
        const T* src = head_base + (present ? (origin + e.off) * ss : 0) + c * 8;
        cp_async16(sbase + row * (D * 2) + ((c ^ (row & 7)) << 4), src, present);
    }
}

}  // namespace mm
}  // namespace lcbsa
