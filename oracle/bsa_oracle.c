/*
 * CPU oracle for LongCat-Video block-sparse attention (BSA) forward.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the algorithm of the
 * reference's BSA forward so that the CUDA path can be checked against it.  Nothing
 * in the shipped package may link, import or call it; only the tests, the smoke
 * check and the CPU-baseline leg of the benchmark do.
 *
 * Reference functions restated here (paths inside the LongCat-Video project):
 *   longcat_video/block_sparse_attention/bsa_interface.py
 *     :600-604  rearrange_THW_to_3d_block   -> block/token index maps (lco_token_of)
 *     :168-178  mean_pooling_compression    -> lco_pool
 *     :180-184  cal_score                   -> lco_score
 *     :212-224  get_select_indices_topk_from_score -> lco_topk
 *     :290-341  attn_fwd_bsa_varlen_triton  -> lco_attn (launcher semantics)
 *   longcat_video/block_sparse_attention/flash_attn_bsa_varlen_mask.py
 *     :172-285  _attn_fwd_bsa_varlen_align  -> lco_attn (mathematical result; the
 *               oracle evaluates the softmax exactly in double precision instead of
 *               the kernel's online form, which is the "fp32 reference" the
 *               tolerance is stated against)
 *
 * Arithmetic definitions (the reference leaves summation order to the library that
 * runs it; this restatement fixes one order so that results are reproducible bit
 * for bit, and the CUDA kernels implement the same order):
 *   pool : fp32 running sum over the present tokens of a block in (t,h,w) row-major
 *          order, then multiplied by fp32(1/block_size), then rounded (RNE) to the
 *          input dtype.  Absent tokens of a partial block add nothing; the divisor
 *          is the full block size (bsa_interface.py:175-177 zero-pads the tail).
 *   score: fp32 fused-multiply-add chain over d = 0..D-1 starting from 0, rounded
 *          (RNE) to the input dtype.
 *   topk : the nsel entries that come first when a row is ordered by (score
 *          descending, block index ascending); -0 equals +0; NaN ranks above +inf.
 *          Emitted in ascending block-index order.
 *
 * Layout: every tensor argument is a dense [BH, S, D] array in the latent grid's
 * T,H,W token order (the order the DiT hands to flash_attn_bsa_3d).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { LCO_BF16 = 0, LCO_FP16 = 1, LCO_FP32 = 2 };

typedef struct {
    int32_t T, H, W;    /* latent grid */
    int32_t ct, ch, cw; /* 3-D block (chunk) shape */
} lco_grid;

/* ---------------------------------------------------------------- dtype helpers */

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

static inline float fp16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_fp16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a >= 0x47800000u) { /* >= 65536 -> inf (65520 rounds to inf too, handled below) */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a < 0x38800000u) { /* subnormal half or zero */
        if (a < 0x33000000u) return (uint16_t)sign; /* < 2^-25 rounds to 0 */
        int e = (int)(a >> 23);
        uint32_t man = (a & 0x7fffffu) | 0x800000u;
        int shift = 126 - e; /* 14..24 */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u))) ++half_man;
        return (uint16_t)(sign | half_man);
    }
    uint32_t exp = (a >> 23) - 127 + 15;
    uint32_t man = a & 0x7fffffu;
    uint32_t h = (exp << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h; /* may carry into exponent / inf: correct */
    return (uint16_t)(sign | h);
}

static inline float load_elem(const void* p, int dtype, int64_t i) {
    switch (dtype) {
        case LCO_BF16: return bf16_to_f32(((const uint16_t*)p)[i]);
        case LCO_FP16: return fp16_to_f32(((const uint16_t*)p)[i]);
        default: return ((const float*)p)[i];
    }
}

static inline void store_elem(void* p, int dtype, int64_t i, float v) {
    switch (dtype) {
        case LCO_BF16: ((uint16_t*)p)[i] = f32_to_bf16(v); break;
        case LCO_FP16: ((uint16_t*)p)[i] = f32_to_fp16(v); break;
        default: ((float*)p)[i] = v; break;
    }
}

/* round a float through the storage dtype (what a store followed by a load does) */
static inline float round_to(int dtype, float v) {
    switch (dtype) {
        case LCO_BF16: return bf16_to_f32(f32_to_bf16(v));
        case LCO_FP16: return fp16_to_f32(f32_to_fp16(v));
        default: return v;
    }
}

/* ---------------------------------------------------------------- block geometry */

static inline int cdiv(int a, int b) { return (a + b - 1) / b; }

int lco_num_blocks(const lco_grid* g) {
    return cdiv(g->T, g->ct) * cdiv(g->H, g->ch) * cdiv(g->W, g->cw);
}

int lco_block_size(const lco_grid* g) { return g->ct * g->ch * g->cw; }

/*
 * Token (position in the T,H,W-ordered sequence) of local slot `r` of block `blk`,
 * or -1 when that slot lies outside the grid (partial block on a ragged grid).
 * Blocks are numbered row-major over (Nt,Nh,Nw) and slots row-major over (t,h,w):
 * the permutation of bsa_interface.py:600-604.
 */
int64_t lco_token_of(const lco_grid* g, int blk, int r) {
    int Nh = cdiv(g->H, g->ch), Nw = cdiv(g->W, g->cw);
    int bw = blk % Nw, bh = (blk / Nw) % Nh, bt = blk / (Nw * Nh);
    int lw = r % g->cw, lh = (r / g->cw) % g->ch, lt = r / (g->cw * g->ch);
    int t = bt * g->ct + lt, h = bh * g->ch + lh, w = bw * g->cw + lw;
    if (t >= g->T || h >= g->H || w >= g->W) return -1;
    return ((int64_t)t * g->H + h) * g->W + w;
}

/* ---------------------------------------------------------------- pool */

/* x: [BH, S, D] (S = T*H*W) -> out: [BH, Nblk, D], same dtype. */
void lco_pool(const void* x, int dtype, int BH, const lco_grid* g, int D, void* out) {
    const int nblk = lco_num_blocks(g), bs = lco_block_size(g);
    const int64_t S = (int64_t)g->T * g->H * g->W;
    const float inv = 1.0f / (float)bs;
#pragma omp parallel for collapse(2) schedule(static)
    for (int bh = 0; bh < BH; ++bh) {
        for (int blk = 0; blk < nblk; ++blk) {
            float acc[512];
            for (int d = 0; d < D; ++d) acc[d] = 0.0f;
            for (int r = 0; r < bs; ++r) {
                int64_t tok = lco_token_of(g, blk, r);
                if (tok < 0) continue;
                int64_t base = ((int64_t)bh * S + tok) * D;
                for (int d = 0; d < D; ++d) acc[d] = acc[d] + load_elem(x, dtype, base + d);
            }
            int64_t ob = ((int64_t)bh * nblk + blk) * D;
            for (int d = 0; d < D; ++d) store_elem(out, dtype, ob + d, acc[d] * inv);
        }
    }
}

/* ---------------------------------------------------------------- score */

/* qc: [BH, Nq, D], kc: [BH, Nk, D] -> score: [BH, Nq, Nk], same dtype. */
void lco_score(const void* qc, const void* kc, int dtype, int BH, int Nq, int Nk, int D, void* score) {
#pragma omp parallel for collapse(2) schedule(static)
    for (int bh = 0; bh < BH; ++bh) {
        for (int i = 0; i < Nq; ++i) {
            float qrow[512];
            for (int d = 0; d < D; ++d) qrow[d] = load_elem(qc, dtype, ((int64_t)bh * Nq + i) * D + d);
            for (int j = 0; j < Nk; ++j) {
                int64_t kb = ((int64_t)bh * Nk + j) * D;
                float acc = 0.0f;
                for (int d = 0; d < D; ++d) acc = fmaf(qrow[d], load_elem(kc, dtype, kb + d), acc);
                store_elem(score, dtype, ((int64_t)bh * Nq + i) * Nk + j, acc);
            }
        }
    }
}

/* ---------------------------------------------------------------- top-k */

/* order-preserving key of a float: larger key <=> larger value; -0 == +0; NaN on top */
static inline uint32_t order_key(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
    if (u == 0x80000000u) u = 0;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

typedef struct { uint32_t key; int32_t idx; } lco_kv;

static int cmp_desc(const void* a, const void* b) {
    const lco_kv* x = (const lco_kv*)a;
    const lco_kv* y = (const lco_kv*)b;
    if (x->key != y->key) return x->key > y->key ? -1 : 1;
    return x->idx < y->idx ? -1 : (x->idx > y->idx ? 1 : 0);
}

static int cmp_int(const void* a, const void* b) {
    int32_t x = *(const int32_t*)a, y = *(const int32_t*)b;
    return x < y ? -1 : (x > y ? 1 : 0);
}

/*
 * score: [BH, Nq, Nk] -> idx: [BH, Nq, cap] (first nsel entries valid, ascending),
 * cnt: [BH, Nq] = nsel.  boundary_ties (nullable): [BH, Nq], the number of entries
 * OUTSIDE the selected set whose score equals the lowest selected score (a row with a
 * non-zero value is one where another tie rule would pick a different set).
 */
void lco_topk(const void* score, int dtype, int BH, int Nq, int Nk, int nsel, int cap,
              int32_t* idx, int32_t* cnt, int32_t* boundary_ties) {
#pragma omp parallel
    {
        lco_kv* row = (lco_kv*)malloc(sizeof(lco_kv) * (size_t)(Nk > 0 ? Nk : 1));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < (int64_t)BH * Nq; ++r) {
            for (int j = 0; j < Nk; ++j) {
                row[j].key = order_key(load_elem(score, dtype, r * Nk + j));
                row[j].idx = j;
            }
            qsort(row, (size_t)Nk, sizeof(lco_kv), cmp_desc);
            int32_t* o = idx + r * cap;
            for (int j = 0; j < nsel; ++j) o[j] = row[j].idx;
            qsort(o, (size_t)nsel, sizeof(int32_t), cmp_int);
            for (int j = nsel; j < cap; ++j) o[j] = -1;
            cnt[r] = nsel;
            if (boundary_ties) {
                int t = 0;
                if (nsel > 0)
                    for (int j = nsel; j < Nk && row[j].key == row[nsel - 1].key; ++j) ++t;
                boundary_ties[r] = t;
            }
        }
        free(row);
    }
}

/* ---------------------------------------------------------------- CDF-threshold selection */

/* exp(t) for t <= 0 from fp32 operations whose results do not depend on the machine (fmaf, rintf, one scaling by a
 * power of two), so that a GPU kernel written with the same operations returns the same bits: n = rint(t * log2 e),
 * r = t - n ln 2 in two fmaf steps, the degree-7 Taylor polynomial in Horner form, times 2^n.  Below -87: 0. */
static inline float lco_exp(float t) {
    if (!(t >= -87.0f)) return 0.0f;
    const float n = rintf(t * 1.44269504f);
    float r = fmaf(-n, 0.693145751953125f, t);
    r = fmaf(-n, 1.42860677e-6f, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    const uint32_t bits = (uint32_t)((int)n + 127) << 23; /* 2^n, n in [-126, 0] */
    float scale;
    memcpy(&scale, &bits, 4);
    return p * scale;
}

static int cmp_u32_desc(const void* a, const void* b) {
    const uint32_t x = *(const uint32_t*)a, y = *(const uint32_t*)b;
    return x > y ? -1 : (x < y ? 1 : 0);
}

/*
 * The cdf_threshold selectors (longcat_video/block_sparse_attention/bsa_interface.py:234-244 and :253-266):
 *   weights = softmax(score * sm_scale) in the score dtype (fp32 inside), sorted in descending order,
 *   cdf = cumsum(sorted weights) (fp32 running sum, every entry rounded to the dtype),
 *   count = number of entries with cdf <= threshold (searchsorted, right=True), raised to nsel_min for the combined
 *   "max(cdf, topk)" selector; the list is the whole sorted index row, of which the first `count` entries are used.
 * What the reference leaves to the library is fixed here: exp is lco_exp; the softmax denominator is summed as 256
 * partial sums (partial t takes the E consecutive entries t E .. t E + E - 1 in ascending order, E = 8 up to 2048
 * entries and 16 above) combined by a butterfly over each group
 * of 32 (xor 16, 8, 4, 2, 1) and then over the 8 group sums (xor 4, 2, 1); equal weights are ordered by ascending
 * index (torch.sort leaves the order of ties open); the comparison with the threshold is done in fp32.
 * score: [rows, Nk] in dtype (bf16 / fp16); idx: [rows, Nk]; cnt: [rows].
 */
void lco_cdf_select(const void* score, int dtype, int64_t rows, int Nk, float sm_scale, float threshold, int nsel_min,
                    int32_t* idx, int32_t* cnt) {
#pragma omp parallel
    {
        float* e = (float*)malloc(sizeof(float) * (size_t)(Nk > 0 ? Nk : 1));
        uint32_t* key = (uint32_t*)malloc(sizeof(uint32_t) * (size_t)(Nk > 0 ? Nk : 1));
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            float m = -INFINITY;
            for (int j = 0; j < Nk; ++j) {
                e[j] = round_to(dtype, load_elem(score, dtype, r * Nk + j) * sm_scale);
                if (e[j] > m) m = e[j];
            }
            float part[256];
            for (int t = 0; t < 256; ++t) part[t] = 0.0f;
            const int E = Nk <= 2048 ? 8 : 16;
            for (int j = 0; j < Nk; ++j) {
                e[j] = lco_exp(e[j] - m);
                part[j / E] += e[j];
            }
            for (int o = 16; o > 0; o >>= 1) {
                float nxt[256];
                for (int t = 0; t < 256; ++t) nxt[t] = part[t] + part[t ^ o];
                memcpy(part, nxt, sizeof(part));
            }
            float grp[8];
            for (int g = 0; g < 8; ++g) grp[g] = part[32 * g];
            for (int o = 4; o > 0; o >>= 1) {
                float nxt[8];
                for (int g = 0; g < 8; ++g) nxt[g] = grp[g] + grp[g ^ o];
                memcpy(grp, nxt, sizeof(grp));
            }
            const float sum = grp[0];
            for (int j = 0; j < Nk; ++j) {
                const float w = e[j] / sum;
                uint32_t wb = dtype == LCO_BF16 ? f32_to_bf16(w) : f32_to_fp16(w);
                key[j] = (wb << 16) | (uint32_t)(0xffff - j);
            }
            qsort(key, (size_t)Nk, sizeof(uint32_t), cmp_u32_desc);
            float acc = 0.0f;
            int n = 0, open = 1;
            for (int j = 0; j < Nk; ++j) {
                idx[r * Nk + j] = (int32_t)(0xffff - (key[j] & 0xffffu));
                const uint16_t wb = (uint16_t)(key[j] >> 16);
                acc += dtype == LCO_BF16 ? bf16_to_f32(wb) : fp16_to_f32(wb);
                if (open && round_to(dtype, acc) <= threshold) ++n; else open = 0;
            }
            cnt[r] = n > nsel_min ? n : nsel_min;
        }
        free(e);
        free(key);
    }
}

/* ---------------------------------------------------------------- attention */

/*
 * q: [BH, Sq, D], k,v: [BH, Sk, D] in T,H,W order; idx: [BH, Nq, cap], cnt: [BH, Nq].
 * out: fp32 [BH, Sq, D]; lse (nullable): fp32 [BH, Sq], natural log.
 * A query block with an empty list yields zeros and lse = -inf
 * (flash_attn_bsa_varlen_mask.py:242-244, 281-285 with zero iterations).
 */
void lco_attn(const void* q, const void* k, const void* v, int dtype, int BH, const lco_grid* gq,
              const lco_grid* gk, int D, const int32_t* idx, const int32_t* cnt, int cap, float sm_scale,
              float* out, float* lse) {
    const int nq = lco_num_blocks(gq), bsq = lco_block_size(gq), bsk = lco_block_size(gk);
    const int64_t Sq = (int64_t)gq->T * gq->H * gq->W, Sk = (int64_t)gk->T * gk->H * gk->W;
#pragma omp parallel
    {
        double* s = (double*)malloc(sizeof(double) * (size_t)cap * bsk + 8);
        int64_t* tokk = (int64_t*)malloc(sizeof(int64_t) * (size_t)cap * bsk + 8);
        double* acc = (double*)malloc(sizeof(double) * (size_t)D);
        float* qrow = (float*)malloc(sizeof(float) * (size_t)D);
#pragma omp for collapse(2) schedule(dynamic, 1)
        for (int bh = 0; bh < BH; ++bh) {
            for (int qb = 0; qb < nq; ++qb) {
                const int32_t* list = idx + ((int64_t)bh * nq + qb) * cap;
                const int n = cnt[(int64_t)bh * nq + qb];
                int nkeys = 0;
                for (int e = 0; e < n; ++e)
                    for (int r = 0; r < bsk; ++r) {
                        int64_t t = lco_token_of(gk, list[e], r);
                        if (t >= 0) tokk[nkeys++] = t;
                    }
                for (int r = 0; r < bsq; ++r) {
                    int64_t tq = lco_token_of(gq, qb, r);
                    if (tq < 0) continue;
                    float* o = out + ((int64_t)bh * Sq + tq) * D;
                    if (nkeys == 0) {
                        for (int d = 0; d < D; ++d) o[d] = 0.0f;
                        if (lse) lse[(int64_t)bh * Sq + tq] = -INFINITY;
                        continue;
                    }
                    for (int d = 0; d < D; ++d) qrow[d] = load_elem(q, dtype, ((int64_t)bh * Sq + tq) * D + d);
                    double m = -INFINITY;
                    for (int j = 0; j < nkeys; ++j) {
                        int64_t kb = ((int64_t)bh * Sk + tokk[j]) * D;
                        double a = 0.0;
                        for (int d = 0; d < D; ++d) a += (double)qrow[d] * (double)load_elem(k, dtype, kb + d);
                        a *= (double)sm_scale;
                        s[j] = a;
                        if (a > m) m = a;
                    }
                    double l = 0.0;
                    for (int d = 0; d < D; ++d) acc[d] = 0.0;
                    for (int j = 0; j < nkeys; ++j) {
                        double p = exp(s[j] - m);
                        l += p;
                        int64_t vb = ((int64_t)bh * Sk + tokk[j]) * D;
                        for (int d = 0; d < D; ++d) acc[d] += p * (double)load_elem(v, dtype, vb + d);
                    }
                    for (int d = 0; d < D; ++d) o[d] = (float)(acc[d] / l);
                    if (lse) lse[(int64_t)bh * Sq + tq] = (float)(m + log(l));
                }
            }
        }
        free(s);
        free(tokk);
        free(acc);
        free(qrow);
    }
}

/* round an fp32 array through a storage dtype (so tests can compare like with like) */
void lco_round_through(float* x, int64_t n, int dtype) {
    for (int64_t i = 0; i < n; ++i) x[i] = round_to(dtype, x[i]);
}

/* ---- the step before the path: q/k RMSNorm (fp32) + 3-D rotary embedding --------------------------------
 * Restates, per row x[D] of q or k (longcat_video/modules/attention.py:116,121):
 *   RMSNorm_FP32.forward (longcat_video/modules/blocks.py:42-53):
 *       y = T( float(x) * rsqrt(mean(float(x)^2) + eps) );   z = T( y * weight )
 *   RotaryPositionalEmbedding.forward (longcat_video/modules/rope_3d.py:99-120):
 *       o = T( float(z) * cos + rotate_half(float(z)) * sin ),  rotate_half: (x1, x2) -> (-x2, x1) per pair
 * cos/sin are the fp32 tables [S, D] the caller built from precompute_freqs_cis_3d (rope_3d.py:60-97).
 * What the reference leaves to the library is fixed here:
 *   the sum of squares is taken as 8 partial sums (partial p owns the D/8 consecutive elements p*(D/8) ..,
 *   accumulated in ascending order with fmaf) combined by the butterfly
 *   p[i] += p[i ^ o] for o = 4, 2, 1; mean = sum * (1/D); rsqrt(v) = 1 / sqrtf(v) (both correctly rounded);
 *   the two products of the rotation are rounded separately before the addition (no fused multiply-add).
 * x: [rows, D] with row stride xs elements; cos, sin: row index = row % S; out: dense [rows, D].
 * weight == NULL: no normalisation (z = x); cos_tab == NULL: no rotary embedding (o = z) -- the two halves as the
 * KV-cache path applies them (attention.py:118-119, 149-171). */
void lco_norm_rope(const void* x, int64_t xs, int dtype, int64_t rows, int D, int64_t S, const void* weight,
                   const float* cos_tab, const float* sin_tab, float eps, void* out) {
    const int per = D / 8;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        float part[8];
        for (int p = 0; p < 8; ++p) {
            float s = 0.f;
            for (int e = 0; e < per; ++e) {
                const float v = load_elem(x, dtype, r * xs + p * per + e);
                s = fmaf(v, v, s);
            }
            part[p] = s;
        }
        for (int o = 4; o > 0; o >>= 1) {
            float nxt[8];
            for (int i = 0; i < 8; ++i) nxt[i] = part[i] + part[i ^ o];
            memcpy(part, nxt, sizeof(part));
        }
        const float mean = part[0] * (1.0f / (float)D);
        const float rinv = 1.0f / sqrtf(mean + eps);
        const int norm = weight != NULL, rope = cos_tab != NULL;
        const int64_t pos = r % S;
        for (int d = 0; d < D; d += 2) {
            float z[2];
            for (int e = 0; e < 2; ++e) {
                z[e] = load_elem(x, dtype, r * xs + d + e);
                if (norm) {
                    const float y = round_to(dtype, z[e] * rinv);
                    z[e] = round_to(dtype, y * load_elem(weight, dtype, d + e));
                }
            }
            if (!rope) {
                store_elem(out, dtype, r * D + d, z[0]);
                store_elem(out, dtype, r * D + d + 1, z[1]);
                continue;
            }
            const float c0 = cos_tab[pos * D + d], c1 = cos_tab[pos * D + d + 1];
            const float s0 = sin_tab[pos * D + d], s1 = sin_tab[pos * D + d + 1];
            const float a0 = z[0] * c0, b0 = (-z[1]) * s0;
            const float a1 = z[1] * c1, b1 = z[0] * s1;
            store_elem(out, dtype, r * D + d, a0 + b0);
            store_elem(out, dtype, r * D + d + 1, a1 + b1);
        }
    }
}
