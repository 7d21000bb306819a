// C ABI of liblcbsa.so: argument validation and dispatch (see include/lcbsa.h).
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "common.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// Status words written by kernels whose bounded waits ran out: [0] = flag, [1..3] = where.
__device__ unsigned int g_device_status[4];

unsigned int* device_status_ptr() {
    // one lookup per device; the symbol's address differs per device
    static thread_local int cached_dev = -1;
    static thread_local unsigned int* cached = nullptr;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (dev != cached_dev) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) != cudaSuccess) return nullptr;
        cached = static_cast<unsigned int*>(p);
        cached_dev = dev;
    }
    return cached;
}

size_t elem_size(int dtype) { return dtype == LCBSA_FP32 ? 4 : 2; }

bool grid_ok(const LcbsaGrid* g) {
    return g && g->T > 0 && g->H > 0 && g->W > 0 && g->ct > 0 && g->ch > 0 && g->cw > 0 && g->ct < 1024 &&
           g->ch < 1024 && g->cw < 1024;
}

// Checks a [B,H,S,D] operand against its grid and the 16-byte rules of the vector / TMA loads.
int check_tensor(const char* name, const LcbsaTensor* t, const LcbsaGrid* g) {
    if (!t || !t->data) return fail(LCBSA_EINVAL, "%s: null tensor", name);
    if (t->dtype != LCBSA_BF16 && t->dtype != LCBSA_FP16 && t->dtype != LCBSA_FP32)
        return fail(LCBSA_EINVAL, "%s: unknown dtype %d", name, t->dtype);
    for (int i = 0; i < 4; ++i)
        if (t->size[i] < 0) return fail(LCBSA_EINVAL, "%s: negative size", name);
    const long long S = (long long)g->T * g->H * g->W;
    if (t->size[2] != S)
        return fail(LCBSA_EINVAL, "%s: sequence length %lld does not match the latent grid %dx%dx%d", name,
                    (long long)t->size[2], g->T, g->H, g->W);
    if (t->stride[3] != 1) return fail(LCBSA_EINVAL, "%s: the head_dim axis must be contiguous", name);
    const size_t es = elem_size(t->dtype);
    if (reinterpret_cast<uintptr_t>(t->data) % 16 != 0) return fail(LCBSA_EINVAL, "%s: data pointer not 16-byte aligned", name);
    for (int i = 0; i < 3; ++i)
        if ((t->stride[i] * (long long)es) % 16 != 0 || t->stride[i] < 0)
            return fail(LCBSA_EINVAL, "%s: stride[%d] must be a non-negative multiple of 16 bytes", name, i);
    if ((t->size[3] * (long long)es) % 16 != 0) return fail(LCBSA_EINVAL, "%s: head_dim row must be a multiple of 16 bytes", name);
    return LCBSA_OK;
}

lcbsa::View view_of(const LcbsaTensor* t) { return lcbsa::View{t->data, t->stride[0], t->stride[1], t->stride[2]}; }

int cuda_fail(cudaError_t e, const char* what, const char* why) {
    if (why && *why) return fail(e == cudaErrorInvalidValue ? LCBSA_EUNSUPPORTED : LCBSA_ECUDA, "%s: %s", what, why);
    return fail(LCBSA_ECUDA, "%s: %s", what, cudaGetErrorString(e));
}

}  // namespace

namespace lcbsa {
void set_last_error(const char* msg) { snprintf(g_err, sizeof(g_err), "%s", msg); }
}  // namespace lcbsa

extern "C" {

int lcbsa_version(void) { return LCBSA_VERSION; }

const char* lcbsa_last_error(void) { return g_err; }

int lcbsa_num_blocks(const LcbsaGrid* g) {
    if (!grid_ok(g)) return fail(LCBSA_EINVAL, "bad grid");
    return lcbsa::make_geom(*g).nblk;
}

int lcbsa_num_selected(double sparsity, int n_k_blocks) { return (int)((1.0 - sparsity) * (double)n_k_blocks); }

int lcbsa_pool(const LcbsaTensor* x, const LcbsaGrid* g, void* out, void* stream) {
    if (!grid_ok(g)) return fail(LCBSA_EINVAL, "pool: bad grid");
    if (int rc = check_tensor("pool input", x, g)) return rc;
    if (!out) return fail(LCBSA_EINVAL, "pool: null output");
    if (reinterpret_cast<uintptr_t>(out) % 16 != 0) return fail(LCBSA_EINVAL, "pool: output not 16-byte aligned");
    const int D = (int)x->size[3];
    const int lpr = (int)(D * elem_size(x->dtype) / 16);
    if (lpr < 1 || lpr > 32 || (lpr & (lpr - 1)) != 0)
        return fail(LCBSA_EUNSUPPORTED, "pool: head_dim row of %d bytes is not 16..512 bytes and a power of two", (int)(D * elem_size(x->dtype)));
    cudaError_t e = lcbsa::launch_pool(x->dtype, view_of(x), (int)x->size[0], (int)x->size[1], D, lcbsa::make_geom(*g), out,
                                       static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "pool", nullptr);
    return LCBSA_OK;
}

int lcbsa_pool_scatter(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk, void* const* dst_q,
                       void* const* dst_k, int n_ranks, int rank, void* stream) {
    if (!grid_ok(gq) || !grid_ok(gk)) return fail(LCBSA_EINVAL, "pool_scatter: bad grid");
    if (int rc = check_tensor("q", q, gq)) return rc;
    if (int rc = check_tensor("k", k, gk)) return rc;
    if (q->dtype != k->dtype) return fail(LCBSA_EINVAL, "pool_scatter: q and k dtypes differ");
    if (q->size[0] != 1 || k->size[0] != 1) return fail(LCBSA_EUNSUPPORTED, "pool_scatter: batch must be 1");
    if (q->size[1] != k->size[1] || q->size[3] != k->size[3]) return fail(LCBSA_EINVAL, "pool_scatter: q and k disagree on heads or head_dim");
    if (n_ranks < 1 || n_ranks > lcbsa::kPoolMaxDst) return fail(LCBSA_EUNSUPPORTED, "pool_scatter: 1..%d ranks", lcbsa::kPoolMaxDst);
    if (rank < 0 || rank >= n_ranks) return fail(LCBSA_EINVAL, "pool_scatter: rank %d outside 0..%d", rank, n_ranks - 1);
    if (q->size[1] % n_ranks != 0) return fail(LCBSA_EINVAL, "pool_scatter: %lld heads do not split over %d ranks", (long long)q->size[1], n_ranks);
    if (!dst_q || !dst_k) return fail(LCBSA_EINVAL, "pool_scatter: null destination table");
    const size_t es = elem_size(q->dtype);
    const int lpr = (int)(q->size[3] * es / 16);
    if (lpr < 1 || lpr > 32 || (lpr & (lpr - 1)) != 0)
        return fail(LCBSA_EUNSUPPORTED, "pool_scatter: head_dim row of %d bytes is not 16..512 bytes and a power of two", (int)(q->size[3] * es));
    lcbsa::PoolDst dq{}, dk{};
    for (int r = 0; r < n_ranks; ++r) {
        if (!dst_q[r] || !dst_k[r] || reinterpret_cast<uintptr_t>(dst_q[r]) % 16 || reinterpret_cast<uintptr_t>(dst_k[r]) % 16)
            return fail(LCBSA_EINVAL, "pool_scatter: destination %d is null or not 16-byte aligned", r);
        dq.dst[r] = dst_q[r];
        dk.dst[r] = dst_k[r];
    }
    dq.n_dst = dk.n_dst = n_ranks;
    dq.heads_per_dst = dk.heads_per_dst = (int)(q->size[1] / n_ranks);
    dq.src_rank = dk.src_rank = rank;
    const lcbsa::Geom ggq = lcbsa::make_geom(*gq), ggk = lcbsa::make_geom(*gk);
    const lcbsa::View vq = view_of(q), vk = view_of(k);
    cudaError_t e = lcbsa::launch_pool2(q->dtype, vq, ggq, dq, &vk, &ggk, &dk, 1, (int)q->size[1], (int)q->size[3], static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "pool_scatter", nullptr);
    return LCBSA_OK;
}

int lcbsa_score_topk(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D, int nsel, int cap,
                     int32_t* idx, int32_t* cnt, void* stream) {
    if (!q_cmp || !k_cmp || !idx || !cnt) return fail(LCBSA_EINVAL, "score_topk: null pointer");
    if (dtype != LCBSA_BF16 && dtype != LCBSA_FP16 && dtype != LCBSA_FP32) return fail(LCBSA_EINVAL, "score_topk: unknown dtype");
    if (BH < 0 || Nq < 0 || Nk <= 0) return fail(LCBSA_EINVAL, "score_topk: bad sizes");
    if (BH > 65535) return fail(LCBSA_EUNSUPPORTED, "score_topk: batch*heads above 65535");
    if (nsel < 0 || nsel > Nk) return fail(LCBSA_EINVAL, "score_topk: nsel %d outside [0, %d]", nsel, Nk);
    if (cap < nsel || cap < 1) return fail(LCBSA_EINVAL, "score_topk: list capacity %d below nsel %d", cap, nsel);
    if (reinterpret_cast<uintptr_t>(q_cmp) % 16 || reinterpret_cast<uintptr_t>(k_cmp) % 16)
        return fail(LCBSA_EINVAL, "score_topk: pooled tensors must be 16-byte aligned");
    const char* why = "";
    cudaError_t e = lcbsa::launch_score_topk(dtype, q_cmp, k_cmp, BH, Nq, Nk, D, nsel, cap, idx, cnt,
                                             static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess) return cuda_fail(e, "score_topk", why);
    return LCBSA_OK;
}

size_t lcbsa_score_keys_bytes(int dtype, int BH, int Nq, int Nk, int D) { return lcbsa::score_keys_bytes(dtype, BH, Nq, Nk, D); }

int lcbsa_score_topk_ws(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D, int nsel, int cap,
                        int32_t* idx, int32_t* cnt, void* keys_ws, size_t keys_bytes, void* stream) {
    const size_t need = lcbsa::score_keys_bytes(dtype, BH, Nq, Nk, D);
    if (need == 0 || !keys_ws || keys_bytes < need)  // the two-kernel form does not apply or has no room: fused form
        return lcbsa_score_topk(q_cmp, k_cmp, dtype, BH, Nq, Nk, D, nsel, cap, idx, cnt, stream);
    if (!q_cmp || !k_cmp || !idx || !cnt) return fail(LCBSA_EINVAL, "score_topk: null pointer");
    if (BH < 0 || Nq < 0 || Nk <= 0) return fail(LCBSA_EINVAL, "score_topk: bad sizes");
    if (nsel < 0 || nsel > Nk) return fail(LCBSA_EINVAL, "score_topk: nsel %d outside [0, %d]", nsel, Nk);
    if (cap < nsel || cap < 1) return fail(LCBSA_EINVAL, "score_topk: list capacity %d below nsel %d", cap, nsel);
    if (reinterpret_cast<uintptr_t>(q_cmp) % 16 || reinterpret_cast<uintptr_t>(k_cmp) % 16 || reinterpret_cast<uintptr_t>(keys_ws) % 16)
        return fail(LCBSA_EINVAL, "score_topk: pooled tensors and workspace must be 16-byte aligned");
    const char* why = "";
    cudaError_t e = lcbsa::launch_score_gemm_topk(dtype, q_cmp, k_cmp, BH, Nq, Nk, D, nsel, cap, idx, cnt, keys_ws,
                                                  static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess) return cuda_fail(e, "score_gemm_topk", why);
    return LCBSA_OK;
}

static int check_split(const char* who, const LcbsaSplit* sp, int Nq, int Nk, int nsel, int cap) {
    if (!sp) return fail(LCBSA_EINVAL, "%s: null split description", who);
    if (sp->hw_q < 1 || sp->hw_k < 1 || sp->period_q < 1 || sp->period_k < 1 || sp->split_q < 0 || sp->split_k < 0 ||
        sp->split_q > sp->period_q || sp->split_k > sp->period_k)
        return fail(LCBSA_EINVAL, "%s: bad split description", who);
    if (Nq % sp->hw_q != 0 || Nk % sp->hw_k != 0 || (Nq / sp->hw_q) % sp->period_q != 0 || (Nk / sp->hw_k) % sp->period_k != 0)
        return fail(LCBSA_EINVAL, "%s: block counts %d / %d are not whole periods of the split", who, Nq, Nk);
    const long long first_k = (long long)(Nk / sp->hw_k / sp->period_k) * sp->split_k * sp->hw_k;  // key blocks of the first part
    if (sp->nsel_first < 0 || sp->nsel_first > first_k || sp->nsel_first > cap || nsel > cap)
        return fail(LCBSA_EINVAL, "%s: nsel_first %d outside [0, min(%lld, cap %d)]", who, sp->nsel_first, first_k, cap);
    return LCBSA_OK;
}

int lcbsa_score_topk_split(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D, const LcbsaSplit* sp, int nsel,
                           int cap, int32_t* idx, int32_t* cnt, void* keys_ws, size_t keys_bytes, void* stream) {
    if (!q_cmp || !k_cmp || !idx || !cnt) return fail(LCBSA_EINVAL, "score_topk_split: null pointer");
    if (BH < 0 || Nq < 0 || Nk <= 0) return fail(LCBSA_EINVAL, "score_topk_split: bad sizes");
    if (nsel < 0 || nsel > Nk) return fail(LCBSA_EINVAL, "score_topk_split: nsel %d outside [0, %d]", nsel, Nk);
    if (cap < nsel || cap < 1) return fail(LCBSA_EINVAL, "score_topk_split: list capacity %d below nsel %d", cap, nsel);
    if (int rc = check_split("score_topk_split", sp, Nq, Nk, nsel, cap)) return rc;
    const size_t need = lcbsa::score_keys_bytes(dtype, BH, Nq, Nk, D);
    if (need == 0) return fail(LCBSA_EUNSUPPORTED, "score_topk_split: bf16 or fp16, head_dim 64 or 128, batch*heads up to 65535");
    if (!keys_ws || keys_bytes < need) return fail(LCBSA_EWORKSPACE, "score_topk_split: workspace of %zu bytes, %zu needed", keys_bytes, need);
    if (reinterpret_cast<uintptr_t>(q_cmp) % 16 || reinterpret_cast<uintptr_t>(k_cmp) % 16 || reinterpret_cast<uintptr_t>(keys_ws) % 16)
        return fail(LCBSA_EINVAL, "score_topk_split: pooled tensors and workspace must be 16-byte aligned");
    const lcbsa::SelectSplit s2{sp->hw_q, sp->period_q, sp->split_q, sp->hw_k, sp->period_k, sp->split_k, sp->nsel_first};
    const char* why = "";
    cudaError_t e = lcbsa::launch_score_gemm_topk(dtype, q_cmp, k_cmp, BH, Nq, Nk, D, nsel, cap, idx, cnt, keys_ws,
                                                  static_cast<cudaStream_t>(stream), &why, &s2);
    if (e != cudaSuccess) return cuda_fail(e, "score_topk_split", why);
    return LCBSA_OK;
}

size_t lcbsa_select_workspace_bytes(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk) {
    if (!q || !k || !grid_ok(gq) || !grid_ok(gk)) return 0;
    const size_t es = elem_size(q->dtype);
    const size_t nq = (size_t)lcbsa::make_geom(*gq).nblk, nk = (size_t)lcbsa::make_geom(*gk).nblk;
    const size_t bhd = (size_t)q->size[0] * (size_t)q->size[1] * (size_t)q->size[3] * es;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    return up(bhd * nq) + up(bhd * nk);
}

size_t lcbsa_select_workspace_bytes_fast(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk) {
    const size_t base = lcbsa_select_workspace_bytes(q, k, gq, gk);
    if (base == 0) return 0;
    const size_t keys = lcbsa::score_keys_bytes(q->dtype, (int)(q->size[0] * q->size[1]), lcbsa::make_geom(*gq).nblk,
                                                lcbsa::make_geom(*gk).nblk, (int)q->size[3]);
    return base + (keys + 255) / 256 * 256;
}

static int block_select_impl(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk, int nsel, int cap,
                             int32_t* idx, int32_t* cnt, void* workspace, size_t workspace_bytes, void* stream, const LcbsaSplit* sp);

int lcbsa_block_select(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk, int nsel,
                       int cap, int32_t* idx, int32_t* cnt, void* workspace, size_t workspace_bytes, void* stream) {
    return block_select_impl(q, k, gq, gk, nsel, cap, idx, cnt, workspace, workspace_bytes, stream, nullptr);
}

int lcbsa_block_select_split(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk, int period_tq,
                             int split_tq, int period_tk, int split_tk, int nsel_first, int nsel, int cap, int32_t* idx, int32_t* cnt,
                             void* workspace, size_t workspace_bytes, void* stream) {
    if (!grid_ok(gq) || !grid_ok(gk)) return fail(LCBSA_EINVAL, "block_select_split: bad grid");
    const lcbsa::Geom a = lcbsa::make_geom(*gq), b = lcbsa::make_geom(*gk);
    const LcbsaSplit sp{a.Nh * a.Nw, period_tq, split_tq, b.Nh * b.Nw, period_tk, split_tk, nsel_first};
    return block_select_impl(q, k, gq, gk, nsel, cap, idx, cnt, workspace, workspace_bytes, stream, &sp);
}

static int block_select_impl(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaGrid* gq, const LcbsaGrid* gk, int nsel, int cap,
                             int32_t* idx, int32_t* cnt, void* workspace, size_t workspace_bytes, void* stream, const LcbsaSplit* sp) {
    if (!grid_ok(gq) || !grid_ok(gk)) return fail(LCBSA_EINVAL, "block_select: bad grid");
    if (int rc = check_tensor("q", q, gq)) return rc;
    if (int rc = check_tensor("k", k, gk)) return rc;
    if (q->dtype != k->dtype) return fail(LCBSA_EINVAL, "block_select: q and k dtypes differ");
    if (q->size[0] != k->size[0] || q->size[1] != k->size[1] || q->size[3] != k->size[3])
        return fail(LCBSA_EINVAL, "block_select: q and k disagree on batch, heads or head_dim");
    const size_t need = lcbsa_select_workspace_bytes(q, k, gq, gk);
    if (!workspace || workspace_bytes < need)
        return fail(LCBSA_EWORKSPACE, "block_select: workspace of %zu bytes, need %zu", workspace_bytes, need);
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(LCBSA_EINVAL, "block_select: workspace not 256-byte aligned");
    const lcbsa::Geom ggq = lcbsa::make_geom(*gq), ggk = lcbsa::make_geom(*gk);
    const size_t es = elem_size(q->dtype);
    const size_t bhd = (size_t)q->size[0] * (size_t)q->size[1] * (size_t)q->size[3] * es;
    unsigned char* qc = static_cast<unsigned char*>(workspace);
    unsigned char* kc = qc + (bhd * ggq.nblk + 255) / 256 * 256;
    {   // pooled Q and pooled K in one launch
        const int lpr = (int)(q->size[3] * es / 16);
        if (lpr < 1 || lpr > 32 || (lpr & (lpr - 1)) != 0)
            return fail(LCBSA_EUNSUPPORTED, "pool: head_dim row of %d bytes is not 16..512 bytes and a power of two", (int)(q->size[3] * es));
        lcbsa::PoolDst dq{}, dk{};
        dq.dst[0] = qc;
        dk.dst[0] = kc;
        const lcbsa::View vq = view_of(q), vk = view_of(k);
        cudaError_t e = lcbsa::launch_pool2(q->dtype, vq, ggq, dq, &vk, &ggk, &dk, (int)q->size[0], (int)q->size[1], (int)q->size[3],
                                            static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) return cuda_fail(e, "pool", nullptr);
    }
    // With room for the score keys the scores are computed by the register-tiled GEMM kernel and selected by a second
    // kernel; otherwise by the fused kernel that keeps them in shared memory.
    const size_t fast = lcbsa_select_workspace_bytes_fast(q, k, gq, gk);
    if (fast > need && workspace_bytes >= fast) {
        if (nsel < 0 || cap < 1 || nsel > cap || nsel > ggk.nblk || !idx || !cnt)
            return fail(LCBSA_EINVAL, "block_select: bad nsel/cap (%d/%d for %d key blocks) or null outputs", nsel, cap, ggk.nblk);
        lcbsa::SelectSplit s2{};
        if (sp) {
            if (int rc = check_split("block_select_split", sp, ggq.nblk, ggk.nblk, nsel, cap)) return rc;
            s2 = lcbsa::SelectSplit{sp->hw_q, sp->period_q, sp->split_q, sp->hw_k, sp->period_k, sp->split_k, sp->nsel_first};
        }
        const char* why = "";
        cudaError_t e = lcbsa::launch_score_gemm_topk(q->dtype, qc, kc, (int)(q->size[0] * q->size[1]), ggq.nblk, ggk.nblk,
                                                      (int)q->size[3], nsel, cap, idx, cnt,
                                                      static_cast<unsigned char*>(workspace) + need, static_cast<cudaStream_t>(stream), &why,
                                                      sp ? &s2 : nullptr);
        if (e != cudaSuccess) return cuda_fail(e, "score_gemm_topk", why);
        return LCBSA_OK;
    }
    if (sp) return fail(LCBSA_EWORKSPACE, "block_select_split: needs the workspace of lcbsa_select_workspace_bytes_fast (%zu bytes) and bf16/fp16 with head_dim 64 or 128", fast);
    return lcbsa_score_topk(qc, kc, q->dtype, (int)(q->size[0] * q->size[1]), ggq.nblk, ggk.nblk, (int)q->size[3], nsel, cap,
                            idx, cnt, stream);
}

int lcbsa_attn_fwd(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaTensor* v, const LcbsaGrid* gq, const LcbsaGrid* gk,
                   const int32_t* idx, const int32_t* cnt, int cap, float sm_scale, const LcbsaTensor* out, float* lse,
                   int impl, void* stream) {
    if (!grid_ok(gq) || !grid_ok(gk)) return fail(LCBSA_EINVAL, "attn_fwd: bad grid");
    if (int rc = check_tensor("q", q, gq)) return rc;
    if (int rc = check_tensor("k", k, gk)) return rc;
    if (int rc = check_tensor("v", v, gk)) return rc;
    if (int rc = check_tensor("out", out, gq)) return rc;
    if (!idx || !cnt || cap < 1) return fail(LCBSA_EINVAL, "attn_fwd: null block lists or zero capacity");
    if (q->dtype != k->dtype || q->dtype != v->dtype || q->dtype != out->dtype) return fail(LCBSA_EINVAL, "attn_fwd: dtypes differ");
    if (q->dtype == LCBSA_FP32) return fail(LCBSA_EUNSUPPORTED, "attn_fwd: attention kernels take bf16 or fp16");
    for (int i : {0, 1, 3}) {
        if (q->size[i] != k->size[i] || q->size[i] != v->size[i] || q->size[i] != out->size[i])
            return fail(LCBSA_EINVAL, "attn_fwd: q, k, v, out disagree on batch, heads or head_dim");
    }
    if (!std::isfinite(sm_scale)) return fail(LCBSA_EINVAL, "attn_fwd: sm_scale is not finite");
    if (q->size[0] * q->size[1] > 65535) return fail(LCBSA_EUNSUPPORTED, "attn_fwd: batch*heads above 65535");

    lcbsa::AttnArgs a;
    a.dtype = q->dtype;
    a.q = view_of(q); a.k = view_of(k); a.v = view_of(v); a.o = view_of(out);
    a.B = (int)q->size[0]; a.H = (int)q->size[1]; a.D = (int)q->size[3];
    a.gq = lcbsa::make_geom(*gq); a.gk = lcbsa::make_geom(*gk);
    a.idx = idx; a.cnt = cnt; a.cap = cap; a.sm_scale = sm_scale; a.lse = lse;
    a.status = device_status_ptr();
    if (!a.status) return fail(LCBSA_ECUDA, "attn_fwd: cannot resolve the device status words");

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const char* why = "";
    cudaError_t e;
    // two tcgen05 kernels: one for 64-token blocks, one for 128-token blocks (the reference's default [4, 4, 8])
    const char* why128 = "";
    const bool tc64 = lcbsa::attn_tc_supported(a, &why), tc128 = !tc64 && lcbsa::attn_tc128_supported(a, &why128);
    if (impl == LCBSA_ATTN_AUTO) impl = (tc64 || tc128) ? LCBSA_ATTN_TC : LCBSA_ATTN_MMA;
    if (impl == LCBSA_ATTN_TC) {
        if (!tc64 && !tc128) return fail(LCBSA_EUNSUPPORTED, "attn_fwd (tcgen05): %s", a.gq.bs == 128 ? why128 : why);
        e = tc64 ? lcbsa::launch_attn_tc(a, st, &why) : lcbsa::launch_attn_tc128(a, st, &why);
    } else if (impl == LCBSA_ATTN_MMA) {
        e = lcbsa::launch_attn_mma(a, st, &why);
    } else {
        return fail(LCBSA_EINVAL, "attn_fwd: unknown impl %d", impl);
    }
    if (e != cudaSuccess) return cuda_fail(e, "attn_fwd", why);
    return LCBSA_OK;
}

int lcbsa_attn_fwd_scatter(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaTensor* v, const LcbsaGrid* gq, const LcbsaGrid* gk,
                           const int32_t* idx, const int32_t* cnt, int cap, float sm_scale, void* const* out_dst, int n_dst,
                           int64_t out_head_stride, int64_t out_token_stride, void* stream) {
    if (!grid_ok(gq) || !grid_ok(gk)) return fail(LCBSA_EINVAL, "attn_fwd_scatter: bad grid");
    if (int rc = check_tensor("q", q, gq)) return rc;
    if (int rc = check_tensor("k", k, gk)) return rc;
    if (int rc = check_tensor("v", v, gk)) return rc;
    if (!idx || !cnt || cap < 1) return fail(LCBSA_EINVAL, "attn_fwd_scatter: null block lists or zero capacity");
    if (q->dtype != k->dtype || q->dtype != v->dtype) return fail(LCBSA_EINVAL, "attn_fwd_scatter: dtypes differ");
    if (q->dtype == LCBSA_FP32) return fail(LCBSA_EUNSUPPORTED, "attn_fwd_scatter: attention kernels take bf16 or fp16");
    for (int i : {0, 1, 3})
        if (q->size[i] != k->size[i] || q->size[i] != v->size[i]) return fail(LCBSA_EINVAL, "attn_fwd_scatter: q, k, v disagree on batch, heads or head_dim");
    if (!std::isfinite(sm_scale)) return fail(LCBSA_EINVAL, "attn_fwd_scatter: sm_scale is not finite");
    if (n_dst < 1 || n_dst > 8 || !out_dst) return fail(LCBSA_EINVAL, "attn_fwd_scatter: 1..8 destinations");
    const size_t es = elem_size(q->dtype);
    if (out_head_stride < 0 || out_token_stride < 0 || (out_head_stride * (long long)es) % 16 || (out_token_stride * (long long)es) % 16)
        return fail(LCBSA_EINVAL, "attn_fwd_scatter: output strides must be non-negative multiples of 16 bytes");
    lcbsa::AttnArgs a;
    a.dtype = q->dtype;
    a.q = view_of(q); a.k = view_of(k); a.v = view_of(v);
    a.o = lcbsa::View{nullptr, 0, out_head_stride, out_token_stride};
    a.B = (int)q->size[0]; a.H = (int)q->size[1]; a.D = (int)q->size[3];
    a.gq = lcbsa::make_geom(*gq); a.gk = lcbsa::make_geom(*gk);
    a.idx = idx; a.cnt = cnt; a.cap = cap; a.sm_scale = sm_scale; a.lse = nullptr;
    a.n_out_dst = n_dst;
    for (int r = 0; r < n_dst; ++r) {
        if (!out_dst[r] || reinterpret_cast<uintptr_t>(out_dst[r]) % 16) return fail(LCBSA_EINVAL, "attn_fwd_scatter: destination %d is null or not 16-byte aligned", r);
        a.out_dst[r] = out_dst[r];
    }
    a.status = device_status_ptr();
    if (!a.status) return fail(LCBSA_ECUDA, "attn_fwd_scatter: cannot resolve the device status words");
    const char* why = "";
    const char* why128 = "";
    const bool tc64 = lcbsa::attn_tc_supported(a, &why), tc128 = !tc64 && lcbsa::attn_tc128_supported(a, &why128);
    if (!tc64 && !tc128) return fail(LCBSA_EUNSUPPORTED, "attn_fwd_scatter (tcgen05): %s", a.gq.bs == 128 ? why128 : why);
    cudaError_t e = tc64 ? lcbsa::launch_attn_tc(a, static_cast<cudaStream_t>(stream), &why)
                         : lcbsa::launch_attn_tc128(a, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess) return cuda_fail(e, "attn_fwd_scatter", why);
    return LCBSA_OK;
}

size_t lcbsa_attn_bwd_workspace_bytes(const LcbsaTensor* q, const LcbsaGrid* gq, const LcbsaGrid* gk, int cap) {
    if (!q || !grid_ok(gq) || !grid_ok(gk) || cap < 1) return 0;
    for (int i = 0; i < 4; ++i)
        if (q->size[i] < 0) return 0;
    const lcbsa::Geom a = lcbsa::make_geom(*gq), b = lcbsa::make_geom(*gk);
    return lcbsa::attn_bwd_workspace_bytes((long long)q->size[0] * q->size[1], a, b, cap);
}

int lcbsa_attn_bwd(const LcbsaTensor* q, const LcbsaTensor* k, const LcbsaTensor* v, const LcbsaTensor* out, const LcbsaTensor* dout,
                   const LcbsaGrid* gq, const LcbsaGrid* gk, const int32_t* idx, const int32_t* cnt, int cap, float sm_scale,
                   const float* lse, const LcbsaTensor* dq, const LcbsaTensor* dk, const LcbsaTensor* dv, void* workspace,
                   size_t workspace_bytes, void* stream) {
    if (!grid_ok(gq) || !grid_ok(gk)) return fail(LCBSA_EINVAL, "attn_bwd: bad grid");
    if (int rc = check_tensor("q", q, gq)) return rc;
    if (int rc = check_tensor("k", k, gk)) return rc;
    if (int rc = check_tensor("v", v, gk)) return rc;
    if (int rc = check_tensor("out", out, gq)) return rc;
    if (int rc = check_tensor("dout", dout, gq)) return rc;
    if (int rc = check_tensor("dq", dq, gq)) return rc;
    if (int rc = check_tensor("dk", dk, gk)) return rc;
    if (int rc = check_tensor("dv", dv, gk)) return rc;
    if (!idx || !cnt || !lse || cap < 1) return fail(LCBSA_EINVAL, "attn_bwd: null block lists or lse, or zero capacity");
    const LcbsaTensor* all[8] = {q, k, v, out, dout, dq, dk, dv};
    for (const LcbsaTensor* t : all) {
        if (t->dtype != q->dtype) return fail(LCBSA_EINVAL, "attn_bwd: dtypes differ");
        for (int i : {0, 1, 3})
            if (t->size[i] != q->size[i]) return fail(LCBSA_EINVAL, "attn_bwd: tensors disagree on batch, heads or head_dim");
    }
    if (q->dtype == LCBSA_FP32) return fail(LCBSA_EUNSUPPORTED, "attn_bwd: takes bf16 or fp16");
    if (!std::isfinite(sm_scale)) return fail(LCBSA_EINVAL, "attn_bwd: sm_scale is not finite");
    if (q->size[0] * q->size[1] > 65535) return fail(LCBSA_EUNSUPPORTED, "attn_bwd: batch*heads above 65535");
    lcbsa::BwdArgs a{};
    a.dtype = q->dtype;
    a.D = (int)q->size[3];
    a.q = view_of(q); a.k = view_of(k); a.v = view_of(v); a.o = view_of(out); a.dout = view_of(dout);
    a.dq = view_of(dq); a.dk = view_of(dk); a.dv = view_of(dv);
    a.B = (int)q->size[0]; a.H = (int)q->size[1];
    a.gq = lcbsa::make_geom(*gq); a.gk = lcbsa::make_geom(*gk);
    a.idx = idx; a.cnt = cnt; a.cap = cap; a.sm_scale = sm_scale; a.lse = lse;
    const char* why = "";
    if (!lcbsa::attn_bwd_supported(a, &why)) return fail(LCBSA_EUNSUPPORTED, "attn_bwd: %s", why);
    const size_t need = lcbsa_attn_bwd_workspace_bytes(q, gq, gk, cap);
    if (!workspace || workspace_bytes < need) return fail(LCBSA_EWORKSPACE, "attn_bwd: workspace of %zu bytes, need %zu", workspace_bytes, need);
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(LCBSA_EINVAL, "attn_bwd: workspace not 256-byte aligned");
    a.status = device_status_ptr();
    if (!a.status) return fail(LCBSA_ECUDA, "attn_bwd: cannot resolve the device status words");
    cudaError_t e = lcbsa::launch_attn_bwd(a, workspace, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess) return cuda_fail(e, "attn_bwd", why);
    return LCBSA_OK;
}

int lcbsa_set_attn_sm_reserve(int n_sms) {
    if (n_sms < 0 || n_sms > 64) return fail(LCBSA_EINVAL, "sm reserve %d outside 0..64", n_sms);
    return lcbsa::set_attn_sm_reserve(n_sms);
}

int lcbsa_score_cdf(const void* q_cmp, const void* k_cmp, int dtype, int BH, int Nq, int Nk, int D, float sm_scale, float cdf_threshold,
                    int nsel_min, int32_t* idx, int32_t* cnt, void* keys_ws, size_t keys_bytes, void* stream) {
    if (!q_cmp || !k_cmp || !idx || !cnt) return fail(LCBSA_EINVAL, "score_cdf: null pointer");
    if (dtype != LCBSA_BF16 && dtype != LCBSA_FP16) return fail(LCBSA_EUNSUPPORTED, "score_cdf: bf16 or fp16 only");
    if (BH < 0 || Nq < 0 || Nk <= 0) return fail(LCBSA_EINVAL, "score_cdf: bad sizes");
    if (Nk > 4096) return fail(LCBSA_EUNSUPPORTED, "score_cdf: more than 4096 key blocks");
    if (nsel_min < 0 || nsel_min > Nk) return fail(LCBSA_EINVAL, "score_cdf: nsel_min %d outside [0, %d]", nsel_min, Nk);
    if (!(cdf_threshold == cdf_threshold)) return fail(LCBSA_EINVAL, "score_cdf: threshold is NaN");
    if (reinterpret_cast<uintptr_t>(q_cmp) % 16 || reinterpret_cast<uintptr_t>(k_cmp) % 16)
        return fail(LCBSA_EINVAL, "score_cdf: pooled tensors must be 16-byte aligned");
    const size_t need = lcbsa::score_keys_bytes(dtype, BH, Nq, Nk, D);
    if (need == 0) return fail(LCBSA_EUNSUPPORTED, "score_cdf: head_dim 64 or 128 and batch*heads up to 65535");
    if (!keys_ws || keys_bytes < need) return fail(LCBSA_EWORKSPACE, "score_cdf: workspace of %zu bytes, %zu needed", keys_bytes, need);
    if (reinterpret_cast<uintptr_t>(keys_ws) % 16) return fail(LCBSA_EINVAL, "score_cdf: workspace not 16-byte aligned");
    const char* why = "";
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = lcbsa::launch_score_keys(dtype, q_cmp, k_cmp, BH, Nq, Nk, D, keys_ws, st, &why);
    if (e == cudaSuccess)
        e = lcbsa::launch_cdf_rows(dtype, keys_ws, (long long)BH * Nq, Nk, sm_scale, cdf_threshold, nsel_min, idx, cnt, st, &why);
    if (e != cudaSuccess) return cuda_fail(e, "score_cdf", why);
    return LCBSA_OK;
}

size_t lcbsa_rope_table_floats(const LcbsaGrid* g, int D) {
    if (!grid_ok(g) || D <= 0 || D % 2 != 0) return 0;
    return lcbsa::rope_table_floats(g->T, g->H, g->W, D);
}

int lcbsa_norm_rope_ex(const LcbsaTensor* x, const void* weight, const LcbsaGrid* g, const float* rope_tab, int table_T, int t_offset,
                       float eps, const LcbsaTensor* out, void* stream) {
    if (!grid_ok(g)) return fail(LCBSA_EINVAL, "norm_rope: bad grid");
    if (int rc = check_tensor("norm_rope input", x, g)) return rc;
    if (int rc = check_tensor("norm_rope output", out, g)) return rc;
    if (!weight && !rope_tab) return fail(LCBSA_EINVAL, "norm_rope: null weight and null rope table: nothing to do");
    if (reinterpret_cast<uintptr_t>(rope_tab) % 16 != 0 || reinterpret_cast<uintptr_t>(weight) % 16 != 0)
        return fail(LCBSA_EINVAL, "norm_rope: weight and rope table must be 16-byte aligned");
    if (rope_tab && (t_offset < 0 || table_T < g->T + t_offset))
        return fail(LCBSA_EINVAL, "norm_rope: frames %d..%d outside the table's %d frames", t_offset, g->T + t_offset - 1, table_T);
    if (x->dtype != out->dtype) return fail(LCBSA_EINVAL, "norm_rope: input and output dtypes differ");
    for (int i = 0; i < 4; ++i)
        if (x->size[i] != out->size[i]) return fail(LCBSA_EINVAL, "norm_rope: input and output shapes differ");
    if (!(eps >= 0.f)) return fail(LCBSA_EINVAL, "norm_rope: eps must be non-negative");
    const char* why = "";
    cudaError_t e = lcbsa::launch_norm_rope(x->dtype, view_of(x), (int)x->size[0], (int)x->size[1], (int)x->size[2], (int)x->size[3], table_T,
                                            t_offset, g->H, g->W, weight, rope_tab, eps, out->data, out->stride[0], out->stride[1],
                                            out->stride[2], static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess) return cuda_fail(e, "norm_rope", why);
    return LCBSA_OK;
}

int lcbsa_norm_rope(const LcbsaTensor* x, const void* weight, const LcbsaGrid* g, const float* rope_tab, float eps,
                    const LcbsaTensor* out, void* stream) {
    if (!weight || !rope_tab) return fail(LCBSA_EINVAL, "norm_rope: null weight or rope table");
    return lcbsa_norm_rope_ex(x, weight, g, rope_tab, g ? g->T : 0, 0, eps, out, stream);
}

int lcbsa_copy_slabs(void* const* dst, const void* const* src, size_t nbytes, int count, void* stream) {
    if (count < 0 || (count > 0 && (!dst || !src))) return fail(LCBSA_EINVAL, "copy_slabs: null pointer array");
    for (int i = 0; i < count; ++i) {
        if (!dst[i] || !src[i]) return fail(LCBSA_EINVAL, "copy_slabs: null slab %d", i);
        cudaError_t e = cudaMemcpyAsync(dst[i], src[i], nbytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
        if (e != cudaSuccess) return fail(LCBSA_ECUDA, "copy_slabs: slab %d: %s", i, cudaGetErrorString(e));
    }
    return LCBSA_OK;
}

int lcbsa_check_device_status(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail(LCBSA_ECUDA, "device synchronize: %s", cudaGetErrorString(e));
    unsigned int h[4] = {0, 0, 0, 0};
    e = cudaMemcpyFromSymbol(h, g_device_status, sizeof(h));
    if (e != cudaSuccess) return fail(LCBSA_ECUDA, "status read: %s", cudaGetErrorString(e));
    if (h[0] != 0) {
        unsigned int z[4] = {0, 0, 0, 0};
        cudaMemcpyToSymbol(g_device_status, z, sizeof(z));
        if (h[0] == lcbsa::kStatusBadBlockIndex)
            return fail(LCBSA_EDEVICE, "attn_fwd: block list entry outside [0, Nk) at (batch*head %u, query block %u, position %u); "
                        "the entry was not dereferenced, the rows of that query block are unspecified", h[1], h[2], h[3]);
        if (h[0] == 1u) return fail(LCBSA_EDEVICE, "attn_fwd: dynamic shared memory base not 1024-byte aligned (CTA %u)", h[1]);
        return fail(LCBSA_EDEVICE, "a kernel gave up on a bounded wait: code %u at (%u, %u, %u)", h[0], h[1], h[2], h[3]);
    }
    return LCBSA_OK;
}

}  // extern "C"
