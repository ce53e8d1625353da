/*
 * CPU oracle for ChatOKF's block-quantized matvec / matmul path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's CPU ("--cpu") engine so the CUDA kernels can be checked
 * against it and so a CPU baseline can be timed beside them.  Nothing in the
 * shipped library calls it; only the tests, the smoke check and the bench's
 * CPU-baseline leg load it.
 *
 * Pinning.  The reference ships no known-answer vectors for these codecs (its
 * codec tests compare against ggml re-expansions of model files that are not in
 * its tree).  The Q8_0, Q4_K, IQ2_XXS, Q4_0, IQ4_NL, Q5_K and Q6_K decoders here are pinned instead
 * against gguf-py 0.19.0's dequantize -- the same ggml arithmetic the
 * reference's LLMTests/IQ1CodecTests.swift:15-102 compares to -- bit for bit on
 * random and edge-case blocks (tests/test_oracle.py, fixtures in
 * tests/golden/).  Q2_0 (ggml type 42) is unknown to gguf-py: for that type
 * parity is UNPINNED, the Swift source is the only authority.
 *
 * Build with -ffp-contract=off: the Swift code has separate multiplies and
 * subtracts (Quantize/KQuants.swift:118-119) and no fused multiply-add, so the
 * decoders must round twice to stay bit-comparable.
 *
 * Every function cites the reference lines it follows, by path inside the
 * reference project.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "iq2xxs_tables.h"

#define OKF_API __attribute__((visibility("default")))

/* LLM/Base/GGUF.swift:3-14 */
enum { T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ4_NL = 20, T_Q2_0 = 42 };

static inline float h2f(const uint8_t *p) {
    uint16_t bits;
    memcpy(&bits, p, 2);
    _Float16 h;
    memcpy(&h, &bits, 2);
    return (float)h; /* exact */
}

/* LLM/Gemma/Gemma4Quant.swift:77-87 (GQ.blockElems) */
OKF_API int okf_ref_block_elems(int type) {
    switch (type) {
    case T_Q4_K:
    case T_Q5_K:
    case T_Q6_K:
    case T_IQ2_XXS: return 256;
    case T_Q2_0: return 128;
    case T_Q4_0:
    case T_IQ4_NL:
    case T_Q8_0: return 32;
    default: return 0;
    }
}

/* LLM/Base/GGUF.swift:160-188 (GGUF.rowByteCount) */
OKF_API int okf_ref_block_bytes(int type) {
    switch (type) {
    case T_Q4_K: return 144;
    case T_Q5_K: return 176;
    case T_Q6_K: return 210;
    case T_Q4_0:
    case T_IQ4_NL: return 18;
    case T_IQ2_XXS: return 66;
    case T_Q2_0: return 34;
    case T_Q8_0: return 34;
    default: return 0;
    }
}

OKF_API size_t okf_ref_row_bytes(int type, size_t k) {
    int per = okf_ref_block_elems(type);
    return per ? k / (size_t)per * (size_t)okf_ref_block_bytes(type) : 0;
}

/* ---- block decoders ------------------------------------------------------ */

/* LLM/Gemma/Gemma4Quant.swift:51-69 (Q8_0.dequant): Float(q) * d */
static void dq_q8_0(const uint8_t *p, float *out) {
    float d = h2f(p);
    for (int j = 0; j < 32; j++) out[j] = (float)(int8_t)p[2 + j] * d;
}

/* LLM/Base/Quant.swift:10-25 (Q2_0.dequant): codes LSB first, (code-1)*d */
static void dq_q2_0(const uint8_t *p, float *out) {
    float d = h2f(p);
    const uint8_t *qs = p + 2;
    for (int j = 0; j < 128; j++) {
        int code = (qs[j >> 2] >> ((j & 3) << 1)) & 3;
        out[j] = (float)(code - 1) * d;
    }
}

/* LLM/Quantize/KQuants.swift:86-101 (scaleMin): ggml's get_scale_min_k4 */
static void q4k_scale_min(const uint8_t *b, int j, float *sc, float *mn) {
    const uint8_t *s = b + 4;
    uint8_t a, m;
    if (j < 4) {
        a = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        a = (uint8_t)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
    *sc = (float)a;
    *mn = (float)m;
}

/* LLM/Quantize/KQuants.swift:104-125 (KQuant.q4K): d1*q - o1, two roundings */
static void dq_q4_k(const uint8_t *b, float *out) {
    float d = h2f(b), dmin = h2f(b + 2);
    int y = 0, qoff = 16, isc = 0;
    for (int g = 0; g < 4; g++) {
        float s1, m1, s2, m2;
        q4k_scale_min(b, isc, &s1, &m1);
        q4k_scale_min(b, isc + 1, &s2, &m2);
        float d1 = d * s1, o1 = dmin * m1;
        float d2 = d * s2, o2 = dmin * m2;
        for (int l = 0; l < 32; l++) {
            uint8_t q = b[qoff + l];
            out[y + l] = d1 * (float)(q & 0xF) - o1;
            out[y + 32 + l] = d2 * (float)(q >> 4) - o2;
        }
        y += 64;
        qoff += 32;
        isc += 2;
    }
}

/* LLM/Quantize/IQ2XXS.swift:34-53 (IQ2XXS.dequant): db = d*(0.5+s)*0.25 left to
 * right; out = db * g * sign, also left to right (the sign multiply is exact). */
static void dq_iq2_xxs(const uint8_t *b, float *out) {
    float d = h2f(b);
    for (int ib = 0; ib < 8; ib++) {
        uint32_t a0, a1;
        memcpy(&a0, b + 2 + ib * 8, 4);
        memcpy(&a1, b + 2 + ib * 8 + 4, 4);
        float db = d * (0.5f + (float)(a1 >> 28)) * 0.25f;
        for (int l = 0; l < 4; l++) {
            uint64_t entry = okf_iq2xxs_grid[(a0 >> (8 * l)) & 0xFF];
            uint8_t signs = okf_iq2xxs_ksigns[(a1 >> (7 * l)) & 127];
            for (int j = 0; j < 8; j++) {
                float g = (float)((entry >> (8 * j)) & 0xFF);
                float s = (signs & (1u << j)) ? -1.0f : 1.0f;
                out[ib * 32 + l * 8 + j] = db * g * s;
            }
        }
    }
}

/* LLM/Gemma/Gemma4Quant.swift:30-49 (Q4_0.dequant): (Float(nibble) - 8) * d, byte j ->
 * elements j (low) and j + 16 (high) */
static void dq_q4_0(const uint8_t *p, float *out) {
    float d = h2f(p);
    for (int j = 0; j < 16; j++) {
        uint8_t b = p[2 + j];
        out[j] = ((float)(b & 0x0F) - 8) * d;
        out[j + 16] = ((float)(b >> 4) - 8) * d;
    }
}

/* LLM/Gemma/Gemma4Quant.swift:5-28 (IQ4_NL.kvalues / dequant): kvalues[nibble] * d */
static const float iq4nl_kvalues[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
static void dq_iq4_nl(const uint8_t *p, float *out) {
    float d = h2f(p);
    for (int j = 0; j < 16; j++) {
        uint8_t b = p[2 + j];
        out[j] = iq4nl_kvalues[b & 0x0F] * d;
        out[j + 16] = iq4nl_kvalues[b >> 4] * d;
    }
}

/* LLM/Quantize/KQuants.swift:127-158 (KQuant.q5K): {d, dmin, scales[12], qh[32] at 16,
 * qs[128] at 48}; the fifth bit of sub-block j is bit j of qh[l]; d1 * q - o1 */
static void dq_q5_k(const uint8_t *b, float *out) {
    float d = h2f(b), dmin = h2f(b + 2);
    int y = 0, qoff = 48, isc = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int g = 0; g < 4; g++) {
        float s1, m1, s2, m2;
        q4k_scale_min(b, isc, &s1, &m1);
        q4k_scale_min(b, isc + 1, &s2, &m2);
        float d1 = d * s1, o1 = dmin * m1;
        float d2 = d * s2, o2 = dmin * m2;
        for (int l = 0; l < 32; l++) {
            uint8_t q = b[qoff + l], h = b[16 + l];
            float lo = (float)((q & 0xF) + ((h & u1) ? 16 : 0));
            float hi = (float)((q >> 4) + ((h & u2) ? 16 : 0));
            out[y + l] = d1 * lo - o1;
            out[y + 32 + l] = d2 * hi - o2;
        }
        y += 64;
        qoff += 32;
        isc += 2;
        u1 = (uint8_t)(u1 << 2);
        u2 = (uint8_t)(u2 << 2);
    }
}

/* LLM/Quantize/KQuants.swift:160-177 (KQuant.q6K): {ql[128], qh[64] at 128, i8 scales[16]
 * at 192, f16 d at 208}; d * Float(s) * Float(q - 32), left to right */
static void dq_q6_k(const uint8_t *b, float *out) {
    float d = h2f(b + 208);
    for (int n = 0; n < 2; n++) {
        for (int l = 0; l < 32; l++) {
            int h = b[128 + n * 32 + l];
            int a = b[n * 64 + l], c = b[n * 64 + l + 32];
            for (int r = 0; r < 4; r++) {
                int byte = (r % 2) == 0 ? a : c;
                int nib = r < 2 ? (byte & 0xF) : (byte >> 4);
                int q = nib | (((h >> (2 * r)) & 3) << 4);
                int s = (int8_t)b[192 + n * 8 + 2 * r + l / 16];
                out[n * 128 + r * 32 + l] = d * (float)s * (float)(q - 32);
            }
        }
    }
}

typedef void (*decode_fn)(const uint8_t *, float *);

/* LLM/Quantize/Blocks.swift:10-29 (Blocks.decoder) plus the two packed types
 * that GQ.gather routes separately (Gemma4Quant.swift:320-349). */
static decode_fn decoder(int type) {
    switch (type) {
    case T_Q8_0: return dq_q8_0;
    case T_Q4_K: return dq_q4_k;
    case T_IQ2_XXS: return dq_iq2_xxs;
    case T_Q2_0: return dq_q2_0;
    case T_Q4_0: return dq_q4_0;
    case T_IQ4_NL: return dq_iq4_nl;
    case T_Q5_K: return dq_q5_k;
    case T_Q6_K: return dq_q6_k;
    default: return NULL;
    }
}

/* GQ.gather / QB.dequant (Gemma4Quant.swift:320-364, Base/Quant.swift:73-76):
 * `count` weights starting at a block boundary.  count must be a multiple of
 * the block size.  Returns 0, or -1 for an unsupported type / ragged count. */
OKF_API int okf_ref_dequant(int type, const void *blocks, size_t count, float *out) {
    decode_fn f = decoder(type);
    int per = okf_ref_block_elems(type), bb = okf_ref_block_bytes(type);
    if (!f || count % (size_t)per) return -1;
    const uint8_t *p = (const uint8_t *)blocks;
    for (size_t b = 0; b < count / (size_t)per; b++) f(p + b * bb, out + b * per);
    return 0;
}

/* ---- per-block dot products, in the reference's operation order ---------- */

/* Gemma4Quant.swift:115-124: integer-valued dot first, scale after */
static float dot_q8_0(const uint8_t *p, const float *x, int faithful) {
    (void)faithful;
    float acc = 0, d = h2f(p);
    for (int j = 0; j < 32; j++) acc += (float)(int8_t)p[2 + j] * x[j];
    return acc * d;
}

/* Base/Quant.swift:44-58 (Q2_0.matvec block body): d*(lo + 2*hi - sum) */
static float dot_q2_0(const uint8_t *p, const float *x, int faithful) {
    (void)faithful;
    float d = h2f(p);
    const uint8_t *qs = p + 2;
    float lo = 0, hi = 0, sy = 0;
    for (int j = 0; j < 128; j++) {
        int code = (qs[j >> 2] >> ((j & 3) << 1)) & 3;
        float xv = x[j];
        sy += xv;
        if (code & 1) lo += xv;
        if (code & 2) hi += xv;
    }
    return d * (lo + 2 * hi - sy);
}

/* Gemma4Quant.swift:125-136: decode the super-block into 256 floats, then a
 * sequential 256-long dot.  `faithful` reproduces the per-block heap scratch the
 * Swift closure allocates (`[Float](repeating: 0, count: 256)`). */
static float dot_super(decode_fn f, const uint8_t *p, const float *x, int faithful) {
    float stack[256];
    float *w = stack;
    if (faithful) w = (float *)calloc(256, sizeof(float));
    f(p, w);
    float acc = 0;
    for (int i = 0; i < 256; i++) acc += w[i] * x[i];
    if (faithful) free(w);
    return acc;
}

static float dot_q4_k(const uint8_t *p, const float *x, int faithful) {
    return dot_super(dq_q4_k, p, x, faithful);
}
static float dot_iq2_xxs(const uint8_t *p, const float *x, int faithful) {
    return dot_super(dq_iq2_xxs, p, x, faithful);
}

static float dot_q5_k(const uint8_t *p, const float *x, int faithful) {
    return dot_super(dq_q5_k, p, x, faithful);
}
static float dot_q6_k(const uint8_t *p, const float *x, int faithful) {
    return dot_super(dq_q6_k, p, x, faithful);
}

/* Gemma4Quant.swift:93-103 (GQ.matvec, q4_0 arm): low and high nibble products added in
 * turn, the block scale after */
static float dot_q4_0(const uint8_t *p, const float *x, int faithful) {
    (void)faithful;
    float acc = 0, d = h2f(p);
    for (int j = 0; j < 16; j++) {
        uint8_t b = p[2 + j];
        acc += ((float)(b & 0x0F) - 8) * x[j];
        acc += ((float)(b >> 4) - 8) * x[j + 16];
    }
    return acc * d;
}

/* Gemma4Quant.swift:104-114 (GQ.matvec, iq4_nl arm) */
static float dot_iq4_nl(const uint8_t *p, const float *x, int faithful) {
    (void)faithful;
    float acc = 0, d = h2f(p);
    for (int j = 0; j < 16; j++) {
        uint8_t b = p[2 + j];
        acc += iq4nl_kvalues[b & 0x0F] * x[j];
        acc += iq4nl_kvalues[b >> 4] * x[j + 16];
    }
    return acc * d;
}

typedef float (*dot_fn)(const uint8_t *, const float *, int);

static dot_fn dotter(int type) {
    switch (type) {
    case T_Q8_0: return dot_q8_0;
    case T_Q4_K: return dot_q4_k;
    case T_IQ2_XXS: return dot_iq2_xxs;
    case T_Q2_0: return dot_q2_0;
    case T_Q4_0: return dot_q4_0;
    case T_IQ4_NL: return dot_iq4_nl;
    case T_Q5_K: return dot_q5_k;
    case T_Q6_K: return dot_q6_k;
    default: return NULL;
    }
}

/* ---- row-parallel drivers ------------------------------------------------ */

typedef struct {
    int type, faithful;
    const uint8_t *w;
    size_t k, m, n;
    const float *x; /* [n][k] */
    float *out;     /* [n][m] */
    double *out64;  /* optional float64 yardstick */
    size_t row0, row1;
    int mode; /* 0 matvec per column, 1 q8_0 blockMatmul, 2 float64 */
} job_t;

/* GQ.rowParallel (Gemma4Quant.swift:250-279) and Q2_0.matvec (Quant.swift:41-62):
 * per row, block partials added sequentially in fp32. */
static void run_rows(const job_t *j) {
    int per = okf_ref_block_elems(j->type), bb = okf_ref_block_bytes(j->type);
    size_t nblk = j->k / (size_t)per, stride = nblk * (size_t)bb;
    dot_fn dot = dotter(j->type);
    decode_fn dec = decoder(j->type);
    for (size_t r = j->row0; r < j->row1; r++) {
        const uint8_t *row = j->w + r * stride;
        if (j->mode == 0) {
            for (size_t c = 0; c < j->n; c++) {
                const float *xp = j->x + c * j->k;
                float acc = 0;
                for (size_t b = 0; b < nblk; b++) acc += dot(row + b * bb, xp + b * per, j->faithful);
                j->out[c * j->m + r] = acc;
            }
        } else if (j->mode == 1) {
            /* GQ.blockMatmul (Gemma4Quant.swift:172-223): block decoded once,
             * acc[n] += w_j * x[n][k] walking k in order, no per-block partial. */
            float blk[32];
            float *acc = (float *)calloc(j->n, sizeof(float));
            for (size_t b = 0; b < nblk; b++) {
                dec(row + b * bb, blk);
                for (int e = 0; e < per; e++) {
                    float wj = blk[e];
                    size_t kk = b * per + e;
                    for (size_t c = 0; c < j->n; c++) acc[c] += wj * j->x[c * j->k + kk];
                }
            }
            for (size_t c = 0; c < j->n; c++) j->out[c * j->m + r] = acc[c];
            free(acc);
        } else {
            float blk[256];
            for (size_t c = 0; c < j->n; c++) {
                const float *xp = j->x + c * j->k;
                double acc = 0;
                for (size_t b = 0; b < nblk; b++) {
                    dec(row + b * bb, blk);
                    for (int e = 0; e < per; e++) acc += (double)blk[e] * (double)xp[b * per + e];
                }
                j->out64[c * j->m + r] = acc;
            }
        }
    }
}

static void *thread_main(void *arg) {
    run_rows((const job_t *)arg);
    return NULL;
}

/* DispatchQueue.concurrentPerform(iterations: M) hands rows to worker threads;
 * here each of `threads` workers takes one contiguous range of rows.  Results
 * do not depend on the split: every row is computed by one thread in one order. */
static int run_parallel(job_t base, int threads) {
    if (!dotter(base.type)) return -1;
    int per = okf_ref_block_elems(base.type);
    if (base.k % (size_t)per) return -1;
    if (threads < 1) threads = 1;
    if ((size_t)threads > base.m) threads = base.m ? (int)base.m : 1;
    if (threads == 1) {
        base.row0 = 0;
        base.row1 = base.m;
        run_rows(&base);
        return 0;
    }
    pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    job_t *jobs = (job_t *)malloc(sizeof(job_t) * (size_t)threads);
    for (int t = 0; t < threads; t++) {
        jobs[t] = base;
        jobs[t].row0 = base.m * (size_t)t / (size_t)threads;
        jobs[t].row1 = base.m * (size_t)(t + 1) / (size_t)threads;
        pthread_create(&tid[t], NULL, thread_main, &jobs[t]);
    }
    for (int t = 0; t < threads; t++) pthread_join(tid[t], NULL);
    free(tid);
    free(jobs);
    return 0;
}

/* GQ.matvec / QB.matvec (Gemma4Quant.swift:89-146, Base/Quant.swift:68-71).
 * w: M rows of K/per blocks, x: fp32 [K], out: fp32 [M]. */
OKF_API int okf_ref_matvec(int type, const void *w, size_t k, size_t m, const float *x,
                           float *out, int threads, int faithful) {
    job_t j = {0};
    j.type = type; j.faithful = faithful; j.w = (const uint8_t *)w;
    j.k = k; j.m = m; j.n = 1; j.x = x; j.out = out; j.mode = 0;
    return run_parallel(j, threads);
}

/* GQ.matmul (Gemma4Quant.swift:150-170): X [N][K] fp32, out[n*M + m].  Q8_0 and Q4_0
 * take the dequant-reuse path; the other types have no batched twin and answer as N
 * independent matvecs. */
OKF_API int okf_ref_matmul(int type, const void *w, size_t k, size_t m, const float *x,
                           size_t n, float *out, int threads) {
    job_t j = {0};
    j.type = type; j.w = (const uint8_t *)w;
    j.k = k; j.m = m; j.n = n; j.x = x; j.out = out;
    j.mode = (type == T_Q8_0 || type == T_Q4_0) ? 1 : 0;
    return run_parallel(j, threads);
}

/* Not in the reference: the same products accumulated in float64, as an
 * accuracy yardstick for both the fp32 oracle and the GPU kernels. */
OKF_API int okf_ref_matmul_f64(int type, const void *w, size_t k, size_t m, const float *x,
                               size_t n, double *out, int threads) {
    job_t j = {0};
    j.type = type; j.w = (const uint8_t *)w;
    j.k = k; j.m = m; j.n = n; j.x = x; j.out64 = out; j.mode = 2;
    return run_parallel(j, threads);
}

/* ---- the linears' neighbours (CPU engine restatements) ---------------------------- */

/* Kernels.rmsnorm (LLM/Base/Kernels.swift:12-20) after the residual add the GPU twin fuses
 * (add_rmsnorm_batch, LLM/metal/Kernels.metal:2839-2864): x += r (r may be NULL); sequential
 * fp32 sum of squares; y = x * scale * w, left to right. */
OKF_API void okf_ref_add_rmsnorm(float *x, const float *r, const float *w, float *y, size_t n, size_t rows,
                                 float eps, size_t x_stride, size_t y_stride) {
    for (size_t row = 0; row < rows; row++) {
        float *xr = x + row * x_stride, *yr = y + row * y_stride;
        const float *rr = r ? r + row * x_stride : NULL;
        float ss = 0;
        for (size_t i = 0; i < n; i++) {
            if (rr) xr[i] = xr[i] + rr[i];
            ss += xr[i] * xr[i];
        }
        float scale = 1 / sqrtf(ss / (float)n + eps);
        for (size_t i = 0; i < n; i++) yr[i] = xr[i] * scale * w[i];
    }
}

/* QwenEngine.ffn (LLM/Qwen/QwenEngine.swift:78-87): gate[i] = silu(gate[i]) * up[i],
 * silu(x) = x / (1 + exp(-x)) */
OKF_API void okf_ref_silu_mul(float *a, const float *b, size_t n) {
    for (size_t i = 0; i < n; i++) a[i] = a[i] / (1.0f + expf(-a[i])) * b[i];
}

/* SRQ.apply (LLM/Gemma/Gemma4Quant.swift:413-427) */
OKF_API void okf_ref_srq(const float *src, float *dst, size_t n, float scale, float lo, float hi) {
    if (scale != 0) {
        float inv = 1 / scale;
        for (size_t i = 0; i < n; i++) {
            float q = rintf(src[i] * inv); /* round half to even in the default mode */
            dst[i] = fminf(fmaxf(q, -128), 127) * scale;
        }
    } else if (lo < hi) {
        for (size_t i = 0; i < n; i++) dst[i] = fminf(fmaxf(src[i], lo), hi);
    } else {
        for (size_t i = 0; i < n; i++) dst[i] = src[i];
    }
}

/* The host arg-max argmax_rows replaces (LLM/metal/Kernels.metal:2754-2794): first largest
 * value, a strict > so ties keep the lower index and NaNs never win. */
OKF_API void okf_ref_argmax_rows(const float *x, size_t n, size_t rows, int *out) {
    for (size_t r = 0; r < rows; r++) {
        float bv = -INFINITY;
        int bi = 0;
        for (size_t i = 0; i < n; i++)
            if (x[r * n + i] > bv) { bv = x[r * n + i]; bi = (int)i; }
        out[r] = bi;
    }
}
