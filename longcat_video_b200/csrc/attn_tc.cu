// Block-sparse flash-attention forward for sm_100a: TMA + tcgen05 + TMEM.
//
// Stands in for the Triton kernel _attn_fwd_bsa_varlen_align
// (longcat_video/block_sparse_attention/flash_attn_bsa_varlen_mask.py:172-285) together with the
// three rearrange copies before it and the one after it (bsa_interface.py:650-659): the 3-D token
// blocks are fetched and the output is written by 5-D TMA boxes straight from/to T,H,W order.
//
// Shape handled: head_dim 128, query and key blocks of 64 tokens, bf16 or fp16.
//
// One persistent CTA per SM.  A work item is four consecutive query blocks of one head, handled as
// two pairs.  Each query block is a 64-row tile, i.e. an M=64 tcgen05 MMA whose accumulator
// occupies 16 lanes of every 32-lane TMEM quadrant; the two tiles of a pair sit in the lower and the
// upper 16 lanes of the same columns, so that one softmax warpgroup (128 threads, one TMEM lane each)
// serves both with every lane busy.
//
//   warps 0-3 : softmax warpgroup of pair 0      warp 8 : TMA producer (Q tiles, K/V tile ring)
//   warps 4-7 : softmax warpgroup of pair 1      warp 9 : MMA issuer (one elected lane)
//
// Per selected K/V block and tile:  S = Q K^T  (M64 N64 K128, fp32 in TMEM)  ->  softmax warpgroup
// reads S with tcgen05.ld, exp2 online softmax in registers, P (input dtype) into swizzled shared
// memory  ->  O += P V  (M64 N128 K64, fp32 in TMEM).  The running maximum baked into O is only
// refreshed when the row maximum grows by more than 2^8 (the accumulated values stay finite and the
// result is unchanged after the final division), so O is rarely rescaled in TMEM.
// The MMA warp interleaves the two pairs (PV of one pair, then the next S of the same pair, then
// the other pair) so the tensor pipe has work while a warpgroup does its softmax.
//
// Every wait on an mbarrier is bounded: when a wait runs out the CTA records where, raises an abort
// flag that all roles poll, drains its outstanding bulk copies, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"

namespace lcbsa {

namespace {

constexpr int kD = 128;
constexpr int kBlk = 64;                 // tokens per query / key block
constexpr int kTileBytes = kBlk * kD * 2;  // 16 KiB: one Q, K, V or O tile
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column half: 64 rows x 128 B, 128B-swizzled
constexpr int kPBytes = kBlk * kBlk * 2;    // 8 KiB: one P tile
constexpr int kStages = 8;                  // K/V tile ring
constexpr int kTilesPerWork = 4;
constexpr int kThreads = 320;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

// shared memory map (offsets from a 1024-byte aligned base)
constexpr int kOffQ = 0;                                   // 4 tiles (reused to stage O)
constexpr int kOffKV = kOffQ + kTilesPerWork * kTileBytes;  // ring
constexpr int kOffP = kOffKV + kStages * kTileBytes;        // 4 P tiles
constexpr int kOffBar = kOffP + kTilesPerWork * kPBytes;
constexpr int kNumBars = 2 * kStages + 2 /*q_full*/ + 2 /*q_empty*/ + 2 /*s_full*/ + 2 /*p_full*/ + 2 /*pv_done*/ + 2 /*o_staged*/;
constexpr int kOffMisc = kOffBar + kNumBars * 8;
constexpr int kSmemBytes = kOffMisc + 64 + 1024;  // + slack for the 1024-byte alignment

struct TcParams {
    CUtensorMap tm_q, tm_k, tm_v, tm_o;
    const int32_t* idx;
    const int32_t* cnt;
    float* lse;
    unsigned int* status;
    int cap;
    int nq;         // query blocks per head
    int bh_total;   // B*H
    int heads;      // H
    int merge_q, merge_k, merge_v, merge_o;  // 0: batch folded into the head axis of the map, 1: into the T axis
    int Tq, Tk;     // frames (for merge == 1 coordinates)
    Geom gq, gk;
    float scale2;   // sm_scale * log2(e)
    int is_bf16;
#ifdef LCBSA_TC_DEBUG
    float* dbg;     // [4 tiles][64 rows][64] raw S of the first work item's first iteration, then [4][64][128] raw O
#endif
};

// ------------------------------------------------------------------------------------------ PTX

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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

struct Ctl {
    volatile int* abort;    // shared flag
    unsigned int* status;   // global status words
};

// Bounded wait. Returns false when the CTA is aborting (this wait or another one ran out).
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const Ctl& c, unsigned code, unsigned it) {
    const unsigned long long t0 = globaltimer();
    for (;;) {
#pragma unroll 1
        for (int k = 0; k < 32; ++k)
            if (mbar_try(bar, parity)) return true;
        if (*c.abort) return false;
        if (globaltimer() - t0 > kWaitLimitNs) {
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
// Called by all 32 lanes of a warp; the verdict is made warp-uniform so that the warp-collective
// tcgen05 instructions that follow are never reached by only some of the lanes.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const Ctl& c, unsigned code, unsigned it) {
    bool ok = mbar_try(bar, parity);
    if (!ok) ok = mbar_wait_slow(bar, parity, c, code, it);
    return __all_sync(0xffffffffu, ok);
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

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
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

// ------------------------------------------------------------------------------------------ schedule

// The order in which K and V tiles enter the ring is the order in which the MMA warp first uses them.
// For a work item with per-pair iteration counts n0, n1 the events are
//   S(0,0) S(1,0) | PV(0,0) S(0,1) PV(1,0) S(1,1) | PV(0,1) S(0,2) ...
// Event e of this list: e < 2 -> S(e, 0); otherwise k = e-2: pair = (k>>1)&1, i = k>>2, PV if (k&1)==0 else S(i+1).
struct Event {
    int pair, iter, is_pv, valid;
};
__device__ __forceinline__ Event event_at(int e, int n0, int n1) {
    Event ev;
    if (e < 2) {
        ev.pair = e; ev.iter = 0; ev.is_pv = 0;
    } else {
        const int k = e - 2;
        ev.pair = (k >> 1) & 1;
        ev.is_pv = (k & 1) == 0;
        ev.iter = (k >> 2) + (ev.is_pv ? 0 : 1);
    }
    ev.valid = ev.iter < (ev.pair ? n1 : n0);
    return ev;
}
__device__ __forceinline__ int num_events(int n0, int n1) { return 2 + 4 * max(n0, n1); }

__device__ __forceinline__ int sel4(int a0, int a1, int a2, int a3, int i) {
    return i == 0 ? a0 : i == 1 ? a1 : i == 2 ? a2 : a3;
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

// ------------------------------------------------------------------------------------------ kernel

__global__ void __launch_bounds__(kThreads, 1) attn_tc_kernel(const __grid_constant__ TcParams P) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + kOffBar;
    auto bar_kv_full = [&](int s) { return bar0 + 8u * s; };
    auto bar_kv_empty = [&](int s) { return bar0 + 8u * (kStages + s); };
    auto bar_q_full = [&](int p) { return bar0 + 8u * (2 * kStages + p); };
    auto bar_q_empty = [&](int p) { return bar0 + 8u * (2 * kStages + 2 + p); };
    auto bar_s_full = [&](int p) { return bar0 + 8u * (2 * kStages + 4 + p); };
    auto bar_p_full = [&](int p) { return bar0 + 8u * (2 * kStages + 6 + p); };
    auto bar_pv_done = [&](int p) { return bar0 + 8u * (2 * kStages + 8 + p); };
    auto bar_o_staged = [&](int p) { return bar0 + 8u * (2 * kStages + 10 + p); };
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffMisc);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kOffMisc + 8);
    const Ctl ctl{abort_flag, P.status};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_kv_full(s), 1);
            mbar_init(bar_kv_empty(s), 1);
        }
        for (int p = 0; p < 2; ++p) {
            mbar_init(bar_q_full(p), 1);
            mbar_init(bar_q_empty(p), 1);
            mbar_init(bar_s_full(p), 1);
            mbar_init(bar_p_full(p), 128);
            mbar_init(bar_pv_done(p), 1);
            mbar_init(bar_o_staged(p), 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {  // TMEM: all 512 columns, allocated and freed by the MMA warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int groups = (P.nq + kTilesPerWork - 1) / kTilesPerWork;
    const long long total_work = (long long)P.bh_total * groups;
    const bool bf16 = P.is_bf16 != 0;

    if (warp == 8) {
        // ================================================================== TMA producer
        unsigned ring = 0;  // tiles pushed so far
        unsigned wk = 0;
        bool ok = true;
        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), g = (int)(w % groups);
            const int b = bh / P.heads, h = bh % P.heads;
            int c[kTilesPerWork];
#pragma unroll
            for (int t = 0; t < kTilesPerWork; ++t) {
                const int qt = g * kTilesPerWork + t;
                c[t] = qt < P.nq ? min(max(P.cnt[(long long)bh * P.nq + qt], 0), P.cap) : 0;
            }
            // Q tiles of both pairs
            for (int p = 0; p < 2 && ok; ++p) {
                ok = mbar_wait(bar_q_empty(p), (wk & 1) ^ 1, ctl, 10 + p, wk);
                if (!ok) break;
                if (lane == 0) {
                    int ntile = 0;
                    for (int hf = 0; hf < 2; ++hf) ntile += (g * kTilesPerWork + 2 * p + hf) < P.nq;
                    mbar_arrive_tx(bar_q_full(p), ntile * kTileBytes);
                    for (int hf = 0; hf < 2; ++hf) {
                        const int t = 2 * p + hf, qt = g * kTilesPerWork + t;
                        if (qt >= P.nq) continue;
                        const Coord cc = block_coord(P.gq, qt, b, h, P.heads, P.merge_q, P.Tq);
                        const uint32_t dst = sbase + kOffQ + t * kTileBytes;
                        tma_load_5d(dst, &P.tm_q, bar_q_full(p), 0, cc.c1, cc.c2, cc.c3, cc.c4);
                        tma_load_5d(dst + kHalfBytes, &P.tm_q, bar_q_full(p), 64, cc.c1, cc.c2, cc.c3, cc.c4);
                    }
                }
            }
            const int n0 = max(c[0], c[1]), n1 = max(c[2], c[3]);
            const int nev = num_events(n0, n1);
            // Block indices are prefetched by the whole warp: lane L holds the entry of tile (L & 3) for
            // iteration win + (L >> 2); a second register holds the next window of eight iterations.
            const int my_t = lane & 3, my_s = lane >> 2;
            const int my_c = sel4(c[0], c[1], c[2], c[3], my_t);
            const int32_t* my_l = P.idx + ((long long)bh * P.nq + min(g * kTilesPerWork + my_t, P.nq - 1)) * P.cap;
            int win = 0;
            int cur = (my_s < my_c) ? my_l[my_s] : 0;
            int nxt = (8 + my_s < my_c) ? my_l[8 + my_s] : 0;
            int pend0 = 0, pend1 = 0, pend2 = 0, pend3 = 0;  // block of each tile's iteration in flight (K queued, V not yet)
            for (int e = 0; e < nev && ok; ++e) {
                const Event ev = event_at(e, n0, n1);
                if (!ev.valid) continue;
                for (int hf = 0; hf < 2 && ok; ++hf) {
                    const int t = 2 * ev.pair + hf;
                    if (ev.iter >= sel4(c[0], c[1], c[2], c[3], t)) continue;
                    if (!ev.is_pv) {
                        while (ev.iter >= win + 8) {
                            win += 8;
                            cur = nxt;
                            nxt = (win + 8 + my_s < my_c) ? my_l[win + 8 + my_s] : 0;
                        }
                        const int v = __shfl_sync(0xffffffffu, cur, ((ev.iter - win) << 2) | t);
                        if (t == 0) pend0 = v; else if (t == 1) pend1 = v; else if (t == 2) pend2 = v; else pend3 = v;
                    }
                    const int stage = ring % kStages;
                    ok = mbar_wait(bar_kv_empty(stage), ((ring / kStages) & 1) ^ 1, ctl, 20, ring);
                    if (!ok) break;
                    if (lane == 0) {
                        const Coord cc = block_coord(P.gk, sel4(pend0, pend1, pend2, pend3, t), b, h, P.heads, ev.is_pv ? P.merge_v : P.merge_k, P.Tk);
                        const CUtensorMap* tm = ev.is_pv ? &P.tm_v : &P.tm_k;
                        const uint32_t dst = sbase + kOffKV + stage * kTileBytes;
                        mbar_arrive_tx(bar_kv_full(stage), kTileBytes);
                        tma_load_5d(dst, tm, bar_kv_full(stage), 0, cc.c1, cc.c2, cc.c3, cc.c4);
                        tma_load_5d(dst + kHalfBytes, tm, bar_kv_full(stage), 64, cc.c1, cc.c2, cc.c3, cc.c4);
                    }
                    ++ring;
                }
            }
        }
        if (!ok && lane == 0) {
            // drain: give the copies this warp issued a bounded time to land before the CTA exits
            const unsigned long long t0 = globaltimer();
            for (unsigned r = ring > kStages ? ring - kStages : 0; r < ring; ++r)
                while (!mbar_try(bar_kv_full(r % kStages), (r / kStages) & 1) && globaltimer() - t0 < 20000000ull) {
                }
        }
    } else if (warp == 9) {
        // ================================================================== MMA issuer
        const uint32_t idesc_s = instr_desc(bf16, 64, 64, 0);
        const uint32_t idesc_pv = instr_desc(bf16, 64, 128, 1);
        unsigned ring = 0, wk = 0;
        unsigned n_p0 = 0, n_p1 = 0;  // completed (pair, iteration) events: phase counters of p_full
        bool ok = true;
        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), g = (int)(w % groups);
            int c[kTilesPerWork];
#pragma unroll
            for (int t = 0; t < kTilesPerWork; ++t) {
                const int qt = g * kTilesPerWork + t;
                c[t] = qt < P.nq ? min(max(P.cnt[(long long)bh * P.nq + qt], 0), P.cap) : 0;
            }
            const int n0 = max(c[0], c[1]), n1 = max(c[2], c[3]);
            const int nev = num_events(n0, n1);
            for (int e = 0; e < nev && ok; ++e) {
                const Event ev = event_at(e, n0, n1);
                if (!ev.valid) continue;
                const int p = ev.pair;
                if (!ev.is_pv) {
                    // ---- S(p, iter) = Q K^T for the active halves
                    if (ev.iter == 0) ok = mbar_wait(bar_q_full(p), wk & 1, ctl, 30 + p, wk);
                    // S(p, iter) overwrites S(p, iter-1): the warpgroup has read it once P(iter-1) is posted,
                    // and that was already waited for before PV(p, iter-1).
                    for (int hf = 0; hf < 2 && ok; ++hf) {
                        const int t = 2 * p + hf;
                        if (ev.iter >= sel4(c[0], c[1], c[2], c[3], t)) continue;
                        const int stage = ring % kStages;
                        ok = mbar_wait(bar_kv_full(stage), (ring / kStages) & 1, ctl, 40, ring);
                        if (!ok) break;
                        tc_fence_after();
                        if (lane == 0) {
                            const uint32_t qa = sbase + kOffQ + t * kTileBytes;
                            const uint32_t kb = sbase + kOffKV + stage * kTileBytes;
                            const uint32_t d = tmem + 64u * p + ((16u * hf) << 16);
#pragma unroll
                            for (int j = 0; j < kD / 16; ++j) {
                                const uint32_t off = (j >> 2) * kHalfBytes + (j & 3) * 32;
                                tc_mma(d, smem_desc(qa + off, 16, 1024), smem_desc(kb + off, 16, 1024), idesc_s, j > 0);
                            }
                            tc_commit(bar_kv_empty(stage));  // K tile free once these MMAs have read it
                        }
                        __syncwarp();
                        ++ring;
                    }
                    if (ok && lane == 0) tc_commit(bar_s_full(p));
                    __syncwarp();
                } else {
                    // ---- O(p) += P V for the active halves (ring order is event order: this event's V tiles are next)
                    const unsigned np_cur = p ? n_p1 : n_p0;
                    ok = mbar_wait(bar_p_full(p), np_cur & 1, ctl, 50 + p, np_cur);
                    if (!ok) break;
                    if (p) ++n_p1; else ++n_p0;
                    for (int hf = 0; hf < 2 && ok; ++hf) {
                        const int t = 2 * p + hf;
                        if (ev.iter >= sel4(c[0], c[1], c[2], c[3], t)) continue;
                        const int stage = ring % kStages;
                        ok = mbar_wait(bar_kv_full(stage), (ring / kStages) & 1, ctl, 60, ring);
                        if (!ok) break;
                        tc_fence_after();
                        if (lane == 0) {
                            const uint32_t pa = sbase + kOffP + t * kPBytes;
                            const uint32_t vb = sbase + kOffKV + stage * kTileBytes;
                            const uint32_t d = tmem + 128u + 128u * p + ((16u * hf) << 16);
#pragma unroll
                            for (int j = 0; j < kBlk / 16; ++j) {
                                // A: P tile, K-major, 32 bytes per 16-key step.
                                // B: V tile, MN-major: 64-column halves 8 KiB apart (LBO), 8-key groups 1 KiB apart (SBO).
                                tc_mma(d, smem_desc(pa + j * 32, 16, 1024), smem_desc(vb + j * 2048, kHalfBytes, 1024),
                                       idesc_pv, (ev.iter > 0 || j > 0) ? 1u : 0u);
                            }
                            tc_commit(bar_kv_empty(stage));
                        }
                        __syncwarp();
                        ++ring;
                    }
                    if (ok && lane == 0) tc_commit(bar_pv_done(p));
                    __syncwarp();
                }
            }
        }
    } else {
        // ================================================================== softmax warpgroups
        const int p = warp >> 2;          // pair
        const int wq = warp & 3;          // TMEM quadrant of this warp
        const int hf = lane >> 4;         // tile of the pair this lane serves
        const int row = wq * 16 + (lane & 15);  // row of that tile
        const int t = 2 * p + hf;
        const uint32_t t_lane = (uint32_t)(wq * 32) << 16;
        const uint32_t tm_s = tmem + 64u * p + t_lane;
        const uint32_t tm_o = tmem + 128u + 128u * p + t_lane;
        unsigned char* p_tile = smem + kOffP + t * kPBytes;
        unsigned char* o_tile = smem + kOffQ + t * kTileBytes;
        unsigned n_s = 0, n_pv = 0, wk = 0;
        bool ok = true;

        for (long long w = blockIdx.x; w < total_work && ok; w += gridDim.x, ++wk) {
            const int bh = (int)(w / groups), g = (int)(w % groups);
            const int b = bh / P.heads, h = bh % P.heads;
            const int qt = g * kTilesPerWork + t;
            const int qt_other = g * kTilesPerWork + (t ^ 1);
            const bool tile_valid = qt < P.nq;
            const int my_cnt = tile_valid ? min(max(P.cnt[(long long)bh * P.nq + qt], 0), P.cap) : 0;
            const int other_cnt = qt_other < P.nq ? min(max(P.cnt[(long long)bh * P.nq + qt_other], 0), P.cap) : 0;
            const int n_iter = max(my_cnt, other_cnt);
            const int32_t* my_list = P.idx + ((long long)bh * P.nq + (tile_valid ? qt : 0)) * P.cap;

            float m_ref = -INFINITY, l_sum = 0.f;

            ok = mbar_wait(bar_q_full(p), wk & 1, ctl, 70 + p, wk);
            if (!ok) break;

            for (int i = 0; i < n_iter && ok; ++i) {
                const bool active = i < my_cnt;
                ok = mbar_wait(bar_s_full(p), n_s & 1, ctl, 80 + p, n_s);
                if (!ok) break;
                ++n_s;
                tc_fence_after();
                uint32_t sr[64];
                tc_ld64(tm_s, sr);
                tc_wait_ld();
#ifdef LCBSA_TC_DEBUG
                if (P.dbg && w == 0 && i == 0)
                    for (int j = 0; j < 64; ++j) P.dbg[(t * 64 + row) * 64 + j] = __uint_as_float(sr[j]);
#endif
                float alpha = 1.f;
                bool need = false;
                if (active) {
                    if (P.gk.ragged) {  // keys of a partial block that lie outside the grid
                        const int blk = my_list[i];
                        int bt, bhh, bw;
                        block_coords(P.gk, blk, bt, bhh, bw);
                        const int vt = P.gk.T - bt * P.gk.ct, vh = P.gk.H - bhh * P.gk.ch, vw = P.gk.W - bw * P.gk.cw;
                        if (vt < P.gk.ct || vh < P.gk.ch || vw < P.gk.cw) {
#pragma unroll
                            for (int j = 0; j < 64; ++j) {
                                int lt, lh, lw;
                                slot_coords(P.gk, j, lt, lh, lw);
                                if (lt >= vt || lh >= vh || lw >= vw) sr[j] = 0xff800000u;  // -inf
                            }
                        }
                    }
                    float mx = -INFINITY;
#pragma unroll
                    for (int j = 0; j < 64; ++j) mx = fmaxf(mx, __uint_as_float(sr[j]));
                    const float m_new = fmaxf(m_ref, mx * P.scale2);
                    if (i == 0) {
                        m_ref = (m_new == -INFINITY) ? 0.f : m_new;
                    } else if (m_new - m_ref > 8.f) {
                        need = true;
                        alpha = ex2(m_ref - m_new);
                        m_ref = m_new;
                    }
                }
                // P(i-1) is still being read by PV(i-1), and O must be at rest before it is rescaled
                if (i > 0) {
                    ok = mbar_wait(bar_pv_done(p), n_pv & 1, ctl, 90 + p, n_pv);
                    if (!ok) break;
                    ++n_pv;
                }
                l_sum *= alpha;  // alpha is 1 unless this row's reference maximum moved
                if (active) {
                    float rs = 0.f;
#pragma unroll
                    for (int cch = 0; cch < 8; ++cch) {
                        float pv[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            pv[j] = ex2(fmaf(__uint_as_float(sr[cch * 8 + j]), P.scale2, -m_ref));
                            rs += pv[j];
                        }
                        uint4 pk;
                        pk.x = pack2(bf16, pv[0], pv[1]);
                        pk.y = pack2(bf16, pv[2], pv[3]);
                        pk.z = pack2(bf16, pv[4], pv[5]);
                        pk.w = pack2(bf16, pv[6], pv[7]);
                        *reinterpret_cast<uint4*>(p_tile + row * 128 + ((cch ^ (row & 7)) << 4)) = pk;
                    }
                    l_sum += rs;
                }
                // O is rescaled after P is out of the registers (both only need PV(i-1) to have finished)
                if (__any_sync(0xffffffffu, need)) {
                    tc_fence_after();
#pragma unroll
                    for (int cch = 0; cch < 4; ++cch) {
                        uint32_t orr[32];
                        tc_ld32(tm_o + 32 * cch, orr);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) orr[j] = __float_as_uint(__uint_as_float(orr[j]) * alpha);
                        tc_st32(tm_o + 32 * cch, orr);
                    }
                    tc_wait_st();
                }
                fence_proxy_async();
                tc_fence_before();
                mbar_arrive(bar_p_full(p));
            }
            if (!ok) break;

            // ---- epilogue of this work item
            if (n_iter > 0) {
                ok = mbar_wait(bar_pv_done(p), n_pv & 1, ctl, 100 + p, n_pv);
                if (!ok) break;
                ++n_pv;
                tc_fence_after();
            }
            const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
#pragma unroll
            for (int cch = 0; cch < 4; ++cch) {
                uint32_t orr[32];
                if (n_iter > 0) {
                    tc_ld32(tm_o + 32 * cch, orr);
                    tc_wait_ld();
                }
#ifdef LCBSA_TC_DEBUG
                if (P.dbg && w == 0 && n_iter > 0)
                    for (int j = 0; j < 32; ++j) P.dbg[4 * 64 * 64 + (t * 64 + row) * 128 + cch * 32 + j] = __uint_as_float(orr[j]);
#endif
                if (tile_valid) {
                    unsigned char* half = o_tile + (cch >> 1) * kHalfBytes;
#pragma unroll
                    for (int q8 = 0; q8 < 4; ++q8) {
                        uint4 pk;
                        if (my_cnt > 0) {
                            const uint32_t* s8 = orr + q8 * 8;
                            pk.x = pack2(bf16, __uint_as_float(s8[0]) * inv, __uint_as_float(s8[1]) * inv);
                            pk.y = pack2(bf16, __uint_as_float(s8[2]) * inv, __uint_as_float(s8[3]) * inv);
                            pk.z = pack2(bf16, __uint_as_float(s8[4]) * inv, __uint_as_float(s8[5]) * inv);
                            pk.w = pack2(bf16, __uint_as_float(s8[6]) * inv, __uint_as_float(s8[7]) * inv);
                        } else {
                            pk = make_uint4(0u, 0u, 0u, 0u);
                        }
                        const int chunk = (cch & 1) * 4 + q8;
                        *reinterpret_cast<uint4*>(half + row * 128 + ((chunk ^ (row & 7)) << 4)) = pk;
                    }
                }
            }
            tc_fence_before();
            if (P.lse != nullptr && tile_valid) {
                int lt, lh, lw, bt, bhh, bw;
                slot_coords(P.gq, row, lt, lh, lw);
                block_coords(P.gq, qt, bt, bhh, bw);
                const int tt = bt * P.gq.ct + lt, hh = bhh * P.gq.ch + lh, ww = bw * P.gq.cw + lw;
                if (tt < P.gq.T && hh < P.gq.H && ww < P.gq.W) {
                    const long long Sq = (long long)P.gq.T * P.gq.H * P.gq.W;
                    const long long tok = ((long long)tt * P.gq.H + hh) * P.gq.W + ww;
                    P.lse[(long long)bh * Sq + tok] = l_sum > 0.f ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
                }
            }
            fence_proxy_async();
            mbar_arrive(bar_o_staged(p));
            if (warp == 4 * p) {  // first warp of the warpgroup: wait for all 128 rows, then one lane stores
                ok = mbar_wait(bar_o_staged(p), wk & 1, ctl, 110 + p, wk);
                if (ok && lane == 0) {
                    for (int hh2 = 0; hh2 < 2; ++hh2) {
                        const int tt2 = 2 * p + hh2, qq = g * kTilesPerWork + tt2;
                        if (qq >= P.nq) continue;
                        const Coord cc = block_coord(P.gq, qq, b, h, P.heads, P.merge_o, P.Tq);
                        const uint32_t src = sbase + kOffQ + tt2 * kTileBytes;
                        tma_store_5d(&P.tm_o, src, 0, cc.c1, cc.c2, cc.c3, cc.c4);
                        tma_store_5d(&P.tm_o, src + kHalfBytes, 64, cc.c1, cc.c2, cc.c3, cc.c4);
                    }
                    tma_store_commit();
                    tma_store_wait_read();
                    mbar_arrive(bar_q_empty(p));
                }
                __syncwarp();
            }
        }
        if ((tid & 127) == 0) tma_store_wait_all();
    }

    // ---- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}

// ------------------------------------------------------------------------------------------ host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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
int merge_mode(const View& v, int B, int H, const Geom& g) {
    if (B == 1) return 0;
    if (v.sb == (long long)H * v.sh) return 0;
    const long long frame = (long long)g.H * g.W * v.ss;
    if (v.sb == (long long)g.T * frame && g.T % g.ct == 0) return 1;
    return -1;
}

bool make_map(CUtensorMap* tm, int dtype, const View& v, int B, int H, const Geom& g, int merge) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t es = 2;
    cuuint64_t dims[5] = {(cuuint64_t)kD, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)(merge ? (long long)g.T * B : g.T),
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

#ifdef LCBSA_TC_DEBUG
float* g_tc_debug = nullptr;
#endif

}  // namespace

#ifdef LCBSA_TC_DEBUG
extern "C" void lcbsa_debug_set_buffer(float* p) { g_tc_debug = p; }
#endif

bool attn_tc_supported(const AttnArgs& a, const char** why) {
    if (a.dtype != LCBSA_BF16 && a.dtype != LCBSA_FP16) { *why = "needs bf16 or fp16"; return false; }
    if (a.D != kD) { *why = "needs head_dim 128"; return false; }
    if (a.gq.bs != kBlk || a.gk.bs != kBlk) { *why = "needs 64-token query and key blocks"; return false; }
    if (a.gq.ct > 256 || a.gq.ch > 256 || a.gq.cw > 256 || a.gk.ct > 256 || a.gk.ch > 256 || a.gk.cw > 256) {
        *why = "block axis above the TMA box limit";
        return false;
    }
    const View* vs[4] = {&a.q, &a.k, &a.v, &a.o};
    const Geom* gs[4] = {&a.gq, &a.gk, &a.gk, &a.gq};
    for (int i = 0; i < 4; ++i) {
        if (merge_mode(*vs[i], a.B, a.H, *gs[i]) < 0) { *why = "batch stride cannot be folded into a 5-D tensor map"; return false; }
        if (vs[i]->ss * 2 >= (1ll << 40) || vs[i]->sh * 2 >= (1ll << 40)) { *why = "stride too large for a tensor map"; return false; }
    }
    return true;
}

cudaError_t launch_attn_tc(const AttnArgs& a, cudaStream_t st, const char** why) {
    if (a.gq.nblk == 0 || a.B * a.H == 0) return cudaSuccess;
    static thread_local TcParams P;
    const int mq = merge_mode(a.q, a.B, a.H, a.gq), mk = merge_mode(a.k, a.B, a.H, a.gk);
    const int mv = merge_mode(a.v, a.B, a.H, a.gk), mo = merge_mode(a.o, a.B, a.H, a.gq);
    if (!make_map(&P.tm_q, a.dtype, a.q, a.B, a.H, a.gq, mq) || !make_map(&P.tm_k, a.dtype, a.k, a.B, a.H, a.gk, mk) ||
        !make_map(&P.tm_v, a.dtype, a.v, a.B, a.H, a.gk, mv) || !make_map(&P.tm_o, a.dtype, a.o, a.B, a.H, a.gq, mo)) {
        *why = "cuTensorMapEncodeTiled rejected a tensor";
        return cudaErrorInvalidValue;
    }
    P.idx = a.idx; P.cnt = a.cnt; P.lse = a.lse; P.status = a.status;
    P.cap = a.cap; P.nq = a.gq.nblk; P.bh_total = a.B * a.H; P.heads = a.H;
    P.merge_q = mq; P.merge_k = mk; P.merge_v = mv; P.merge_o = mo; P.Tq = a.gq.T; P.Tk = a.gk.T;
    P.gq = a.gq; P.gk = a.gk;
    P.scale2 = a.sm_scale * 1.4426950408889634f;
    P.is_bf16 = a.dtype == LCBSA_BF16;
#ifdef LCBSA_TC_DEBUG
    P.dbg = g_tc_debug;
#endif

    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    }
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    const long long groups = (a.gq.nblk + kTilesPerWork - 1) / kTilesPerWork;
    const long long work = groups * a.B * a.H;
    const int grid = (int)(work < sm_count ? work : sm_count);
    attn_tc_kernel<<<grid, kThreads, kSmemBytes, st>>>(P);
    return cudaGetLastError();
}

}  // namespace lcbsa
