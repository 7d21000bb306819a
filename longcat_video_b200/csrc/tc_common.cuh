// Internal header of the tcgen05 attention kernels (attn_tc.cu: 64-token blocks in pairs; attn_tc128.cu: 128-token
// blocks): the PTX wrappers (mbarrier, TMA, tcgen05), the bounded waits, the shared-memory and instruction descriptors,
// and on the host the tensor-map encoder with its per-thread cache and the per-device launch state.
#pragma once
#include <cuda.h>

#include <atomic>

#include "common.cuh"

namespace lcbsa {
namespace tc {

constexpr int kMaxOutDst = 8;
constexpr unsigned kSpinsBeforeClock = 1u << 12;     // failed try_waits before the clock is consulted
constexpr long long kWaitLimitCycles = 4000000000ll;  // about 2 s

// ------------------------------------------------------------------------------------------ PTX

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// called by all lanes of a converged warp: one elected lane arrives (no divergent branch around it)
__device__ __forceinline__ void mbar_arrive_elect(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}"
        ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// non-blocking probe of a phase (used to look ahead while other work is being issued)
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Branches that are rarely taken and whose code should not sit in the instruction stream of a hot loop.
#define LCBSA_UNLIKELY(x) __builtin_expect(!!(x), 0)

struct Ctl {
    volatile int* abort;    // shared flag
    unsigned int* status;   // global status words
};

// Reached only after many failed tries: bound the wait by the cycle counter and flag a timeout.
__device__ __forceinline__ bool mbar_wait_timeout(uint32_t bar, uint32_t parity, const Ctl& c, unsigned code, unsigned it) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int k = 0; k < 64; ++k)
            if (mbar_try(bar, parity)) return true;
        if (*c.abort) return false;
        if (clock64() - t0 > kWaitLimitCycles) {
            *c.abort = 1;
            if (atomicCAS(c.status, 0u, code) == 0u) {
                c.status[1] = blockIdx.x;
                c.status[2] = threadIdx.x;
                c.status[3] = it;
            }
            __threadfence();
            return false;
        }
    }
}
// Bounded wait of one thread. Returns false when the CTA is aborting (this wait or another one ran out).
// try_wait itself blocks for a hardware-defined interval, so the loop turns over rarely.
__device__ __forceinline__ bool mbar_wait_thread(uint32_t bar, uint32_t parity, const Ctl& c, unsigned code, unsigned it) {
    unsigned spins = 0;
    while (!mbar_try(bar, parity)) {
        if (LCBSA_UNLIKELY(*c.abort)) return false;
        if (LCBSA_UNLIKELY(++spins >= kSpinsBeforeClock)) return mbar_wait_timeout(bar, parity, c, code, it);
    }
    return true;
}
// The same for all 32 lanes of a warp; the verdict is made warp-uniform so that the warp-collective
// tcgen05 instructions that follow are never reached by only some of the lanes.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const Ctl& c, unsigned code, unsigned it) {
    return __all_sync(0xffffffffu, mbar_wait_thread(bar, parity, c, code, it));
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2,
                                            int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* tm, uint32_t src, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(tm),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// The three issuing wrappers below are called by ALL lanes of a converged warp; one elected lane issues.
// Measured on B200: issued this way a tcgen05.mma costs its warp about 23 cycles, against about 50 (and up to
// 125 next to busy arithmetic warps) when a single lane issues it from inside a divergent branch.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
        : "memory");
}

// A operand from TMEM (M x K, two 16-bit elements per column), B from shared memory
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "elect.sync _|q, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accum)
        : "memory");
}

// 32 lanes x 32 columns of fp32: thread i of the warp gets lane (base + i), columns c .. c+31
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 64 columns of fp32 in one instruction
__device__ __forceinline__ void tc_ld64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// 32 lanes x 16 columns
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// max of three (one instruction on sm_100; NaN operands are ignored like fmaxf does)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack2(bool bf16, float lo, float hi) {
    if (bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Rare path of the online softmax, as a rolled loop so that it takes little room in the instruction stream of the loop:
// multiply this thread's row of a 128-column fp32 accumulator in TMEM by alpha.  Warp-collective.
__device__ __forceinline__ void tc_scale_row128(uint32_t taddr, float alpha) {
    tc_fence_after();
#pragma unroll 1
    for (int cch = 0; cch < 4; ++cch) {
        uint32_t orr[32];
        tc_ld32(taddr + 32 * cch, orr);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * alpha);
        tc_st32(taddr + 32 * cch, orr);
    }
}

// ------------------------------------------------------------------------------------------ descriptors

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
//   bits [0,14)  start address >> 4          bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4     bits [46,48) version = 1      bits [61,64) layout = 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A/B both bf16 (1) or fp16 (0).
//   [4,6) c format = 1 (f32)  [7,10) a format  [10,13) b format  [15] a major  [16] b major (1 = MN-major)
//   [17,23) N >> 3            [24,29) M >> 4
__device__ __forceinline__ uint32_t instr_desc(bool bf16, int M, int N, int b_mn_major) {
    const uint32_t f = bf16 ? 1u : 0u;
    return (1u << 4) | (f << 7) | (f << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) |
           ((uint32_t)(M >> 4) << 24);
}

// Which of the 64 slots of a block (w fastest, then h, then t) lie inside the first vt x vh x vw tokens of it: bit j
// for slot j.  The extents are powers of two whose product is 64 (any 3-D factorisation of 64 is), so a row of cw
// slots and a plane of cw * ch slots tile the 64 bits exactly.  Limits below 1 give an empty mask.
__device__ __forceinline__ uint64_t slot_mask64(int ct, int ch, int cw, int vt, int vh, int vw) {
    auto low = [](int n) { return n >= 64 ? ~0ull : ((1ull << n) - 1ull); };
    vt = max(0, min(vt, ct));
    vh = max(0, min(vh, ch));
    vw = max(0, min(vw, cw));
    const int plane = cw * ch;
    uint64_t mw = low(vw);
    for (int s = cw; s < 64; s <<= 1) mw |= mw << s;
    uint64_t mh = low(vh * cw);
    for (int s = plane; s < 64; s <<= 1) mh |= mh << s;
    return mw & mh & low(vt * plane);
}

struct Coord {
    int c1, c2, c3, c4;
};
// TMA coordinates (w, h, t, head) of block `blk` for (batch b, head h).
__device__ __forceinline__ Coord block_coord(const Geom& g, int blk, int b, int h, int heads, int merge, int T) {
    int bt, bhh, bw;
    block_coords(g, blk, bt, bhh, bw);
    Coord c;
    c.c1 = bw * g.cw;
    c.c2 = bhh * g.ch;
    c.c3 = bt * g.ct + (merge ? b * T : 0);
    c.c4 = merge ? h : b * heads + h;
    return c;
}

// ------------------------------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// How the batch axis is folded into the 5-D map: 0 = with heads, 1 = with frames, -1 = impossible.
inline int merge_mode(const View& v, int B, int H, const Geom& g) {
    if (B == 1) return 0;
    if (v.sb == (long long)H * v.sh) return 0;
    const long long frame = (long long)g.H * g.W * v.ss;
    if (v.sb == (long long)g.T * frame && g.T % g.ct == 0) return 1;
    return -1;
}

inline bool encode_map(CUtensorMap* tm, int dtype, const View& v, int B, int H, const Geom& g, int merge) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t es = 2;
    cuuint64_t dims[5] = {(cuuint64_t)128, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)(merge ? (long long)g.T * B : g.T),
                          (cuuint64_t)(merge ? H : (long long)B * H)};
    cuuint64_t strides[4] = {(cuuint64_t)v.ss * es, (cuuint64_t)v.ss * g.W * es, (cuuint64_t)v.ss * g.W * g.H * es,
                             (cuuint64_t)v.sh * es};
    cuuint32_t box[5] = {64u, (cuuint32_t)g.cw, (cuuint32_t)g.ch, (cuuint32_t)g.ct, 1u};
    cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
    const CUtensorMapDataType dt = dtype == LCBSA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = fn(tm, dt, 5, const_cast<void*>(v.data), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Tensor maps are a pure function of (pointer, dtype, strides, batch, heads, grid, block, fold mode); a DiT calls the
// op with the same few buffers layer after layer, so the last encodings are kept per host thread and reused.
struct MapKey {
    const void* data;
    long long sb, sh, ss;
    int dtype, B, H, T, Hh, W, ct, ch, cw, merge;
    bool operator==(const MapKey& o) const {
        return data == o.data && sb == o.sb && sh == o.sh && ss == o.ss && dtype == o.dtype && B == o.B && H == o.H && T == o.T &&
               Hh == o.Hh && W == o.W && ct == o.ct && ch == o.ch && cw == o.cw && merge == o.merge;
    }
};
constexpr int kMapCache = 32;
struct MapCache {
    MapKey key[kMapCache];
    CUtensorMap map[kMapCache];
    int used = 0, next = 0;
};

inline bool make_map(CUtensorMap* tm, int dtype, const View& v, int B, int H, const Geom& g, int merge) {
    static thread_local MapCache cache;
    const MapKey k{v.data, v.sb, v.sh, v.ss, dtype, B, H, g.T, g.H, g.W, g.ct, g.ch, g.cw, merge};
    for (int i = 0; i < cache.used; ++i)
        if (cache.key[i] == k) {
            *tm = cache.map[i];
            return true;
        }
    if (!encode_map(tm, dtype, v, B, H, g, merge)) return false;
    const int slot = cache.next;
    cache.key[slot] = k;
    cache.map[slot] = *tm;
    cache.next = (slot + 1) % kMapCache;
    if (cache.used < kMapCache) ++cache.used;
    return true;
}

// Per-device launch state: SM count, and whether the kernels' shared-memory limit has been raised on that device.
constexpr int kMaxDevices = 64;
struct DeviceState {
    std::atomic<int> sm_count{0};
    std::atomic<int> attr_set{0};  // one bit per kernel instantiation: bits 0-3 64-token blocks (dtype, ragged), bits 4-7 128-token blocks
};
DeviceState* device_states();  // defined once, in attn_tc.cu
int attn_sm_reserve();           // SMs the persistent attention kernels leave idle (lcbsa_set_attn_sm_reserve)

}  // namespace tc
}  // namespace lcbsa
