// Generic block-sparse flash-attention forward on warp-level MMA (mma.sync m16n8k16).
//
// Covers the shapes the tcgen05 kernel does not: head_dim 64, 128-token blocks, and serves as the
// on-device comparator for it.  Same contract as the Triton kernels it stands in for
// (longcat_video/block_sparse_attention/flash_attn_bsa_varlen_mask.py:172-285 and :35-153):
// one CTA keeps a query block resident and walks that block's list of selected K/V blocks with an
// exp2-based online softmax (row sum from the unrounded probabilities, probabilities rounded to the
// input dtype for the PV product, fp32 accumulation).  Unlike the reference, q/k/v are read and the
// output is written directly in T,H,W token order: the 3-D block gather is done by the loads.
#include "mma_common.cuh"

namespace lcbsa {

namespace {

constexpr int kKT = 64;  // keys per inner tile

using namespace mm;

template <typename T, int D, int BQ>
__global__ void __launch_bounds__(BQ * 2) attn_mma_kernel(AttnArgs a) {
    constexpr int NT = BQ * 2;  // threads: one warp per 16 query rows
    constexpr int CPR = D * 2 / 16;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                      // [BQ][D]   (reused to stage the output)
    unsigned char* k_s = q_s + BQ * D * 2;          // [2][64][D]
    unsigned char* v_s = k_s + 2 * kKT * D * 2;     // [2][64][D]
    SlotEntry* qtab = reinterpret_cast<SlotEntry*>(v_s + 2 * kKT * D * 2);  // [bsq]
    SlotEntry* ktab = qtab + a.gq.bs;                                       // [bsk]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int qb = blockIdx.x;
    const int bh = blockIdx.y;
    const int b = bh / a.H, h = bh % a.H;
    const Geom& gq = a.gq;
    const Geom& gk = a.gk;

    for (int r = tid; r < gq.bs; r += NT) {
        int lt, lh, lw;
        slot_coords(gq, r, lt, lh, lw);
        qtab[r] = SlotEntry{(lt * gq.H + lh) * gq.W + lw, lt | (lh << 10) | (lw << 20)};
    }
    for (int r = tid; r < gk.bs; r += NT) {
        int lt, lh, lw;
        slot_coords(gk, r, lt, lh, lw);
        ktab[r] = SlotEntry{(lt * gk.H + lh) * gk.W + lw, lt | (lh << 10) | (lw << 20)};
    }
    __syncthreads();

    const T* qh = reinterpret_cast<const T*>(a.q.data) + (long long)b * a.q.sb + (long long)h * a.q.sh;
    const T* kh = reinterpret_cast<const T*>(a.k.data) + (long long)b * a.k.sb + (long long)h * a.k.sh;
    const T* vh = reinterpret_cast<const T*>(a.v.data) + (long long)b * a.v.sb + (long long)h * a.v.sh;
    T* oh = reinterpret_cast<T*>(const_cast<void*>(a.o.data)) + (long long)b * a.o.sb + (long long)h * a.o.sh;

    const int32_t* list = a.idx + ((long long)bh * gq.nblk + qb) * a.cap;
    int n = a.cnt[(long long)bh * gq.nblk + qb];
    n = min(max(n, 0), a.cap);
    const int nsub = gk.bs / kKT;
    const int ntiles = n * nsub;

    load_tile<T, D, BQ, NT>(q_s, qh, a.q.ss, gq, qtab, qb, 0, tid);
    cp_async_commit();
    if (ntiles > 0) {
        const int blk0 = list[0];
        load_tile<T, D, kKT, NT>(k_s, kh, a.k.ss, gk, ktab, blk0, 0, tid);
        load_tile<T, D, kKT, NT>(v_s, vh, a.v.ss, gk, ktab, blk0, 0, tid);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    uint32_t qf[D / 16][4];
    {
        const int row = warp * 16 + (lane & 15);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            const int c = 2 * ks + (lane >> 4);
            ldsm_x4(qf[ks], smem_u32(q_s) + row * (D * 2) + ((c ^ (row & 7)) << 4));
        }
    }

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float scale2 = a.sm_scale * 1.4426950408889634f;

    for (int it = 0; it < ntiles; ++it) {
        const int buf = it & 1;
        const int blk = list[it / nsub];
        const int sub = it % nsub;
        if (it + 1 < ntiles) {
            const int nblk = list[(it + 1) / nsub], nsubi = (it + 1) % nsub;
            load_tile<T, D, kKT, NT>(k_s + (buf ^ 1) * kKT * D * 2, kh, a.k.ss, gk, ktab, nblk, nsubi * kKT, tid);
            load_tile<T, D, kKT, NT>(v_s + (buf ^ 1) * kKT * D * 2, vh, a.v.ss, gk, ktab, nblk, nsubi * kKT, tid);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();

        const uint32_t kt = smem_u32(k_s) + buf * kKT * D * 2;
        const uint32_t vt = smem_u32(v_s) + buf * kKT * D * 2;

        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const int mid = lane >> 3;
                const int row = np * 16 + (lane & 7) + (mid >> 1) * 8;
                const int c = 2 * ks + (mid & 1);
                uint32_t kb[4];
                ldsm_x4(kb, kt + row * (D * 2) + ((c ^ (row & 7)) << 4));
                mma16816<T>(s[2 * np], qf[ks], kb[0], kb[1]);
                mma16816<T>(s[2 * np + 1], qf[ks], kb[2], kb[3]);
            }
        }

        if ((unsigned)blk >= (unsigned)gk.nblk) {
            // list entry outside [0, Nk): the block is skipped and the call is flagged (lcbsa_check_device_status)
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = -INFINITY;
            if (tid == 0 && sub == 0 && atomicCAS(a.status, 0u, kStatusBadBlockIndex) == 0u) {
                a.status[1] = bh;
                a.status[2] = qb;
                a.status[3] = (unsigned)(it / nsub);
            }
        } else if (gk.ragged) {  // absent keys of a partial block do not take part in the softmax
            int bt, bhh, bw;
            block_coords(gk, blk, bt, bhh, bw);
            const int t0 = bt * gk.ct, h0 = bhh * gk.ch, w0 = bw * gk.cw;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int col = nt * 8 + 2 * (lane & 3) + e;
                    if (!slot_present(gk, ktab[sub * kKT + col].packed, t0, h0, w0)) {
                        s[nt][e] = -INFINITY;
                        s[nt][2 + e] = -INFINITY;
                    }
                }
            }
        }

        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0 * scale2), mn1 = fmaxf(m1, mx1 * scale2);
        const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
        const float al0 = ex2(m0 - ms0), al1 = ex2(m1 - ms1);
        m0 = mn0;
        m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s[nt][0] = ex2(fmaf(s[nt][0], scale2, -ms0));
            s[nt][1] = ex2(fmaf(s[nt][1], scale2, -ms0));
            s[nt][2] = ex2(fmaf(s[nt][2], scale2, -ms1));
            s[nt][3] = ex2(fmaf(s[nt][3], scale2, -ms1));
            rs0 += s[nt][0] + s[nt][1];
            rs1 += s[nt][2] + s[nt][3];
        }
        l0 = l0 * al0 + rs0;
        l1 = l1 * al1 + rs1;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            o[i][0] *= al0;
            o[i][1] *= al0;
            o[i][2] *= al1;
            o[i][3] *= al1;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa[4];
            pa[0] = pack2(T(), s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack2(T(), s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack2(T(), s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack2(T(), s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                const int mid = lane >> 3;
                const int row = kk * 16 + (lane & 7) + (mid & 1) * 8;
                const int c = 2 * dp + (mid >> 1);
                uint32_t vb[4];
                ldsm_x4_t(vb, vt + row * (D * 2) + ((c ^ (row & 7)) << 4));
                mma16816<T>(o[2 * dp], pa, vb[0], vb[1]);
                mma16816<T>(o[2 * dp + 1], pa, vb[2], vb[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

    // ---- epilogue: normalise, stage through shared memory, write rows back in T,H,W order
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    __syncthreads();  // every warp is done reading q_s fragments (they live in registers) and K/V tiles
    {
        const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const int col = i * 8 + 2 * (lane & 3);  // element column; chunk = col / 8
            const int c = col >> 3, within = (col & 7) * 2;
            *reinterpret_cast<uint32_t*>(q_s + r0 * (D * 2) + ((c ^ (r0 & 7)) << 4) + within) =
                pack2(T(), o[i][0] * inv0, o[i][1] * inv0);
            *reinterpret_cast<uint32_t*>(q_s + r1 * (D * 2) + ((c ^ (r1 & 7)) << 4) + within) =
                pack2(T(), o[i][2] * inv1, o[i][3] * inv1);
        }
    }
    int bt, bhh, bw;
    block_coords(gq, qb, bt, bhh, bw);
    const int t0 = bt * gq.ct, h0 = bhh * gq.ch, w0 = bw * gq.cw;
    const long long origin = ((long long)t0 * gq.H + h0) * gq.W + w0;
    if (a.lse != nullptr && (lane & 3) == 0) {
        const long long Sq = (long long)gq.T * gq.H * gq.W;
        const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
        const SlotEntry e0 = qtab[r0], e1 = qtab[r1];
        if (!gq.ragged || slot_present(gq, e0.packed, t0, h0, w0))
            a.lse[(long long)bh * Sq + origin + e0.off] = l0 > 0.f ? (m0 + log2f(l0)) * 0.6931471805599453f : -INFINITY;
        if (!gq.ragged || slot_present(gq, e1.packed, t0, h0, w0))
            a.lse[(long long)bh * Sq + origin + e1.off] = l1 > 0.f ? (m1 + log2f(l1)) * 0.6931471805599453f : -INFINITY;
    }
    __syncthreads();
    for (int v = tid; v < BQ * CPR; v += NT) {
        const int row = v / CPR, c = v % CPR;
        const SlotEntry e = qtab[row];
        if (gq.ragged && !slot_present(gq, e.packed, t0, h0, w0)) continue;
        const uint4 val = *reinterpret_cast<const uint4*>(q_s + row * (D * 2) + ((c ^ (row & 7)) << 4));
        *reinterpret_cast<uint4*>(oh + (origin + e.off) * a.o.ss + c * 8) = val;
    }
}

template <typename T, int D, int BQ>
cudaError_t launch(const AttnArgs& a, cudaStream_t st) {
    auto kern = attn_mma_kernel<T, D, BQ>;
    const size_t smem = (size_t)BQ * D * 2 + 4 * (size_t)kKT * D * 2 + sizeof(SlotEntry) * (size_t)(a.gq.bs + a.gk.bs);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid(a.gq.nblk, a.B * a.H);
    kern<<<grid, BQ * 2, smem, st>>>(a);
    return cudaGetLastError();
}

template <typename T>
cudaError_t pick(const AttnArgs& a, cudaStream_t st, const char** why) {
    if (a.D == 128 && a.gq.bs == 64) return launch<T, 128, 64>(a, st);
    if (a.D == 128 && a.gq.bs == 128) return launch<T, 128, 128>(a, st);
    if (a.D == 64 && a.gq.bs == 64) return launch<T, 64, 64>(a, st);
    if (a.D == 64 && a.gq.bs == 128) return launch<T, 64, 128>(a, st);
    *why = "generic attention kernel needs head_dim in {64,128} and a query block of 64 or 128 tokens";
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_attn_mma(const AttnArgs& a, cudaStream_t st, const char** why) {
    if (a.gk.bs % kKT != 0) {
        *why = "generic attention kernel needs a key block that is a multiple of 64 tokens";
        return cudaErrorInvalidValue;
    }
    if (a.gq.nblk == 0 || a.B * a.H == 0) return cudaSuccess;
    switch (a.dtype) {
        case LCBSA_BF16: return pick<__nv_bfloat16>(a, st, why);
        case LCBSA_FP16: return pick<__half>(a, st, why);
        default: *why = "attention kernels take bf16 or fp16"; return cudaErrorInvalidValue;
    }
}

}  // namespace lcbsa
