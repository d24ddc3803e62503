/*
 * CPU oracle: plain-C restatement of microkimi's quantized decode hot path.
 * TEST INFRASTRUCTURE ONLY - see mk_oracle.h.  Citations are file:line of the
 * reference project (Rust).  Build with -ffp-contract=off: the reference never
 * fuses a multiply with an add, and several checks are bit-level.
 */
#define _GNU_SOURCE
#include "mk_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#ifndef M_PI
#define M_PI 3.14159265358979323846
#endif

#define FLASH_KV 64 /* model.rs:1348 */

static const float E2M1[16] = { /* mxfp4.rs:5-7 */
    0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
    -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f };
static const int8_t E2M1_X2[16] = { /* q8.rs:22 */
    0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12 };
static const float BOUNDS[7] = { 0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f }; /* mxfp4.rs:52,99 */

int or_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
/* Thread count of the loops that carry no explicit count (the quantizers).  A launcher may have set
 * OMP_NUM_THREADS=1 for its children; a caller that wants all cores says so here. */
void or_set_num_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* exp / tanh / log of the reference are f32 libm calls (Rust's f32::exp, ::tanh, ::ln), whose last bit depends on the
 * platform's libm.  With or_set_cr_math(1) they are taken in double precision and rounded once - the correctly rounded
 * value up to double rounding, which is also what the CUDA kernels compute - so that a comparison can separate "same
 * algorithm, same order" (bit-level agreement under this switch) from the last-ulp freedom of a libm. */
static int g_cr_math = 0;
void or_set_cr_math(int on) { g_cr_math = on != 0; }
float or_m_expf(float x) { return g_cr_math ? (float)exp((double)x) : expf(x); }
float or_m_tanhf(float x) { return g_cr_math ? (float)tanh((double)x) : tanhf(x); }
float or_m_logf(float x) { return g_cr_math ? (float)log((double)x) : logf(x); }

static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* ------------------------------------------------------------------ RNG */
/* build.rs:16 SEED_BASE, :24-31 FNV-1a name hash, :32-39 xorshift64*,
 * :40-47 uniform + Box-Muller (cosine branch only). */
#define SEED_BASE 0x4B494D495EED0001ULL
void or_rng_for_tensor(or_rng *r, const char *name) {
    uint64_t h = 0xcbf29ce484222325ULL;
    for (const unsigned char *p = (const unsigned char *)name; *p; ++p) {
        h ^= (uint64_t)*p;
        h *= 0x00000100000001b3ULL;
    }
    r->s = (h ^ SEED_BASE) | 1ULL;
}
uint64_t or_rng_next_u64(or_rng *r) {
    uint64_t x = r->s;
    x ^= x >> 12;
    x ^= x << 25;
    x ^= x >> 27;
    r->s = x;
    return x * 0x2545F4914F6CDD1DULL;
}
double or_rng_uniform(or_rng *r) {
    return (double)(or_rng_next_u64(r) >> 11) / (double)(1ULL << 53);
}
float or_rng_gauss(or_rng *r) {
    double u1 = or_rng_uniform(r);
    if (u1 < 1e-300) u1 = 1e-300;
    double u2 = or_rng_uniform(r);
    return (float)(sqrt(-2.0 * log(u1)) * cos(2.0 * M_PI * u2));
}
void or_rng_fill_gauss(const char *name, float sigma, float *out, size_t n) {
    or_rng r;
    or_rng_for_tensor(&r, name);
    for (size_t i = 0; i < n; ++i) out[i] = or_rng_gauss(&r) * sigma; /* build.rs:332 */
}

/* ------------------------------------------------------------------ MXFP4 */
float or_exp2_i(int e) { /* mxfp4.rs:10-16 */
    if (e < -126) return ldexpf(1.0f, e); /* subnormal, exact */
    return bits_f32((uint32_t)(e + 127) << 23);
}
float or_scale_from_byte(uint8_t sb) { /* mxfp4.rs:340-346 */
    return sb == 0 ? bits_f32(0x00400000u) : bits_f32((uint32_t)sb << 23);
}

void or_mxfp4_dequant(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols, float *out) {
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t *prow = packed + r * cols / 2;
        const uint8_t *srow = scales + r * cols / 32;
        for (size_t c = 0; c < cols; ++c) {
            uint8_t byte = prow[c / 2];
            uint8_t nib = (c % 2 == 0) ? (byte & 0x0F) : (byte >> 4);
            out[r * cols + c] = E2M1[nib] * or_exp2_i((int)srow[c / 32] - 127);
        }
    }
}

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* mxfp4.rs:51-69 */
static double group_sse(const float *group, int e) {
    float inv = 1.0f / or_exp2_i(e);
    double s = (double)or_exp2_i(e);
    double sse = 0.0;
    for (int i = 0; i < 32; ++i) {
        float v = group[i];
        float q = clampf(v * inv, -6.0f, 6.0f);
        float mag = fabsf(q);
        int idx = 0;
        while (idx < 7 && mag >= BOUNDS[idx]) idx++;
        double lvl = (double)E2M1[idx];
        double dq = (signbit(q) ? -lvl : lvl) * s;
        double d = (double)v - dq;
        sse += d * d;
    }
    return sse;
}
/* mxfp4.rs:77-92 */
static int search_mx_scale(const float *group, int e) {
    int best = e;
    double best_sse = group_sse(group, e);
    int cands[2] = { e - 1, e + 1 };
    for (int k = 0; k < 2; ++k) {
        int cand = cands[k];
        if (cand < -127 || cand > 128) continue;
        double sse = group_sse(group, cand);
        if (sse < best_sse) { best_sse = sse; best = cand; }
    }
    return best;
}
/* mxfp4.rs:94-138 */
void or_mxfp4_quantize(const float *w, size_t rows, size_t cols, int search, uint8_t *packed, uint8_t *scales) {
    memset(packed, 0, rows * cols / 2);
    /* rows are independent: the split over threads does not change any byte */
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        const float *row = w + r * cols;
        for (size_t g = 0; g < cols / 32; ++g) {
            const float *group = row + g * 32;
            float maxabs = 0.0f;
            for (int j = 0; j < 32; ++j) maxabs = fmaxf(maxabs, fabsf(group[j]));
            int e;
            if (maxabs == 0.0f) e = -127;
            else {
                float c = ceilf(log2f(maxabs / 6.0f));
                /* Rust `as i32` saturates; the values here are far from the limits */
                e = (int)c;
            }
            if (e < -127) e = -127;
            if (e > 128) e = 128;
            if (search && maxabs != 0.0f) e = search_mx_scale(group, e);
            int sb = e + 127;
            if (sb < 0) sb = 0;
            if (sb > 255) sb = 255;
            scales[r * cols / 32 + g] = (uint8_t)sb;
            float inv = 1.0f / or_exp2_i(e);
            for (int j = 0; j < 32; ++j) {
                float q = clampf(group[j] * inv, -6.0f, 6.0f);
                float mag = fabsf(q);
                int idx = 0;
                while (idx < 7 && mag >= BOUNDS[idx]) idx++;
                if (signbit(q)) idx += 8;
                size_t c = g * 32 + j;
                uint8_t *byte = &packed[r * cols / 2 + c / 2];
                if (c % 2 == 0) *byte |= (uint8_t)idx; else *byte |= (uint8_t)(idx << 4);
            }
        }
    }
}

/* ---- MXFP4SQ: quadratic scale byte against a per-tensor smax (mxfp4.rs:140-240) ---- */
float or_scale_sq(uint8_t q, float smax) { /* :153-158 */
    float t = ((float)q + 1.0f) * (1.0f / 256.0f);
    return t * t * smax;
}
float or_mxfp4sq_quantize(const float *w, size_t rows, size_t cols, uint8_t *packed, uint8_t *scales) { /* :160-210; returns smax */
    size_t ng = rows * cols / 32;
    float *ideal = (float *)malloc(sizeof(float) * ng);
    float smax = 0.0f;
    for (size_t gi = 0; gi < ng; ++gi) {
        float maxabs = 0.0f;
        for (int j = 0; j < 32; ++j) maxabs = fmaxf(maxabs, fabsf(w[gi * 32 + j]));
        ideal[gi] = maxabs / 6.0f;
    }
    for (size_t gi = 0; gi < ng; ++gi) smax = fmaxf(smax, ideal[gi]);
    memset(packed, 0, rows * cols / 2);
    for (size_t gi = 0; gi < ng; ++gi) {
        uint8_t q = 0;
        if (!(smax == 0.0f || ideal[gi] == 0.0f)) {
            int v = (int)ceilf(256.0f * sqrtf(ideal[gi] / smax)) - 1;
            q = (uint8_t)(v < 0 ? 0 : (v > 255 ? 255 : v));
        }
        scales[gi] = q;
        float inv = 1.0f / or_scale_sq(q, smax);
        for (int j = 0; j < 32; ++j) {
            float qv = clampf(w[gi * 32 + j] * inv, -6.0f, 6.0f);
            float mag = fabsf(qv);
            int idx = 0;
            while (idx < 7 && mag >= BOUNDS[idx]) idx++;
            if (signbit(qv)) idx += 8;
            size_t c = gi * 32 + j;
            if (c % 2 == 0) packed[c / 2] |= (uint8_t)idx; else packed[c / 2] |= (uint8_t)(idx << 4);
        }
    }
    free(ideal);
    return smax;
}
void or_mxfp4sq_dequant(const uint8_t *packed, const uint8_t *scales, float smax, size_t rows, size_t cols, float *out) { /* :213-226 */
    for (size_t i = 0; i < rows * cols; ++i) {
        uint8_t byte = packed[i / 2];
        uint8_t nib = (i % 2 == 0) ? (byte & 0x0F) : (byte >> 4);
        out[i] = E2M1[nib] * or_scale_sq(scales[i / 32], smax);
    }
}

/* mxfp4.rs:494-505 (one row of the exact f32 path) */
static inline float mxfp4_row_f32(const uint8_t *prow, const uint8_t *srow, size_t cols, const float *x) {
    float sum = 0.0f;
    for (size_t g = 0; g < cols / 32; ++g) {
        float gsum = 0.0f;
        for (size_t j = 0; j < 32; ++j) {
            size_t c = g * 32 + j;
            uint8_t byte = prow[c / 2];
            uint8_t nib = (c % 2 == 0) ? (byte & 0x0F) : (byte >> 4);
            gsum += E2M1[nib] * x[c];
        }
        sum += gsum * or_exp2_i((int)srow[g] - 127);
    }
    return sum;
}
/* Row split: the reference cuts rows into n_threads contiguous chunks
 * (mxfp4.rs:509-538); results do not depend on the split. */
void or_mxfp4_matvec_f32(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                         const float *x, float *out, int n_threads) {
    if (n_threads <= 1) {
        for (size_t r = 0; r < rows; ++r)
            out[r] = mxfp4_row_f32(packed + r * cols / 2, scales + r * cols / 32, cols, x);
        return;
    }
#pragma omp parallel for schedule(static) num_threads(n_threads)
    for (long r = 0; r < (long)rows; ++r)
        out[r] = mxfp4_row_f32(packed + r * cols / 2, scales + r * cols / 32, cols, x);
}

int32_t or_block_dot(const uint8_t *packed16, const int8_t *x32) { /* q8.rs:194-202 */
    int32_t s = 0;
    for (int j = 0; j < 16; ++j) {
        uint8_t b = packed16[j];
        s += (int32_t)E2M1_X2[b & 0x0F] * (int32_t)x32[2 * j];
        s += (int32_t)E2M1_X2[b >> 4] * (int32_t)x32[2 * j + 1];
    }
    return s;
}
int32_t or_block_dot_i8(const int8_t *w32, const int8_t *x32) { /* q8.rs:119-125 */
    int32_t s = 0;
    for (int j = 0; j < 32; ++j) s += (int32_t)w32[j] * (int32_t)x32[j];
    return s;
}

/* mxfp4.rs:409-418 */
static inline float mxfp4_row_q8(const uint8_t *prow, const uint8_t *srow, size_t cols, const int8_t *xq, const float *xs) {
    float sum = 0.0f;
    for (size_t g = 0; g < cols / 32; ++g) {
        int32_t idot = or_block_dot(prow + g * 16, xq + g * 32);
        sum += (float)idot * (or_exp2_i((int)srow[g] - 128) * xs[g]);
    }
    return sum;
}
void or_mxfp4_matvec_q8(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                        const int8_t *xq, const float *xs, float *out, int n_threads) {
    if (n_threads <= 1) {
        for (size_t r = 0; r < rows; ++r)
            out[r] = mxfp4_row_q8(packed + r * cols / 2, scales + r * cols / 32, cols, xq, xs);
        return;
    }
#pragma omp parallel for schedule(static) num_threads(n_threads)
    for (long r = 0; r < (long)rows; ++r)
        out[r] = mxfp4_row_q8(packed + r * cols / 2, scales + r * cols / 32, cols, xq, xs);
}

/* mxfp4.rs:458-539 : q8 activation path by default, exact f32 path otherwise */
void or_mxfp4_matvec(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                     const float *x, float *out, int n_threads, int use_q8) {
    if (use_q8) {
        int8_t *xq = (int8_t *)malloc(cols);
        float *xs = (float *)malloc(sizeof(float) * (cols / 32));
        or_q8_quantize(x, cols, xq, xs);
        or_mxfp4_matvec_q8(packed, scales, rows, cols, xq, xs, out, n_threads);
        free(xq);
        free(xs);
    } else {
        or_mxfp4_matvec_f32(packed, scales, rows, cols, x, out, n_threads);
    }
}

/* mxfp4.rs:357-393 */
static float tree_sum(float *v, size_t n) {
    while (n > 1) {
        for (size_t i = 0; i < n / 2; ++i) v[i] += v[n / 2 + i];
        n /= 2;
    }
    return v[0];
}
void or_mxfp4_matvec_shader_emul(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                                 const float *x, float *out, size_t lanes) {
    float *part = (float *)malloc(sizeof(float) * lanes);
    float *sg = (float *)malloc(sizeof(float) * (lanes / 32));
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t *prow = packed + r * cols / 2;
        const uint8_t *srow = scales + r * cols / 32;
        for (size_t lane = 0; lane < lanes; ++lane) {
            float acc = 0.0f;
            for (size_t c = lane; c < cols; c += lanes) {
                uint8_t byte = prow[c / 2];
                uint8_t nib = (c % 2 == 0) ? (byte & 0x0F) : (byte >> 4);
                acc += E2M1[nib] * or_scale_from_byte(srow[c / 32]) * x[c];
            }
            part[lane] = acc;
        }
        for (size_t s = 0; s < lanes / 32; ++s) sg[s] = tree_sum(part + s * 32, 32);
        out[r] = tree_sum(sg, lanes / 32);
    }
    free(part);
    free(sg);
}

/* model.rs:2412-2447 */
void or_mxfp4_matvec_nt(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                        const float *xt, size_t m, float *out) {
    float *wrow = (float *)malloc(sizeof(float) * cols);
    for (size_t r = 0; r < rows; ++r) {
        const uint8_t *prow = packed + r * cols / 2;
        const uint8_t *srow = scales + r * cols / 32;
        for (size_t c = 0; c < cols; ++c) {
            uint8_t byte = prow[c / 2];
            uint8_t nib = (c % 2 == 0) ? (byte & 0x0F) : (byte >> 4);
            wrow[c] = E2M1[nib];
        }
        for (size_t t0 = 0; t0 < m; t0 += 8) {
            float sum[8] = { 0 };
            for (size_t g = 0; g < cols / 32; ++g) {
                float gsum[8] = { 0 };
                for (size_t j = 0; j < 32; ++j) {
                    size_t c = g * 32 + j;
                    float wv = wrow[c];
                    const float *xc = xt + c * m + t0;
                    for (int p = 0; p < 8; ++p) gsum[p] += wv * xc[p];
                }
                float sc = or_exp2_i((int)srow[g] - 127);
                for (int p = 0; p < 8; ++p) sum[p] += gsum[p] * sc;
            }
            for (int p = 0; p < 8; ++p) out[(t0 + p) * rows + r] = sum[p];
        }
    }
    free(wrow);
}

/* ------------------------------------------------------------------ q8_0 */
void or_q8_quantize(const float *x, size_t n, int8_t *q, float *scales) { /* q8.rs:49-69 */
    size_t nb = n / 32;
    memset(q, 0, n);
    for (size_t g = 0; g < nb; ++g) {
        const float *b = x + g * 32;
        float max = 0.0f;
        for (int j = 0; j < 32; ++j) max = fmaxf(max, fabsf(b[j]));
        float dx = max / 127.0f;
        scales[g] = dx;
        if (dx == 0.0f) continue;
        for (int j = 0; j < 32; ++j)
            q[g * 32 + j] = (int8_t)clampf(roundf(b[j] / dx), -127.0f, 127.0f);
    }
}

/* ------------------------------------------------------------------ f32 kernels */
float or_dot(const float *a, const float *b, size_t n) { /* model.rs:63-82 */
    float acc[8] = { 0 };
    size_t i = 0;
    for (; i + 8 <= n; i += 8)
        for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
    float s = (acc[0] + acc[1]) + (acc[2] + acc[3]) + (acc[4] + acc[5]) + (acc[6] + acc[7]);
    for (; i < n; ++i) s += a[i] * b[i];
    return s;
}
void or_matvec_f32(const float *w, size_t rows, size_t cols, const float *x, float *out, int n_threads) {
    if (n_threads <= 1) {
        for (size_t r = 0; r < rows; ++r) out[r] = or_dot(w + r * cols, x, cols);
        return;
    }
#pragma omp parallel for schedule(static) num_threads(n_threads)
    for (long r = 0; r < (long)rows; ++r) out[r] = or_dot(w + r * cols, x, cols);
}
void or_rmsnorm(const float *x, const float *w, size_t n, float eps, float *out) { /* model.rs:599-605 */
    float ss = or_dot(x, x, n) / (float)n;
    float inv = 1.0f / sqrtf(ss + eps);
    for (size_t i = 0; i < n; ++i) out[i] = x[i] * inv * w[i];
}
float or_sigmoid(float x) { return 1.0f / (1.0f + or_m_expf(-x)); } /* model.rs:607-610 */
float or_situ(float g, float u) { /* model.rs:617-621 */
    return 4.0f * or_m_tanhf(g / 4.0f) * or_sigmoid(g) * (25.0f * or_m_tanhf(u / 25.0f));
}
int or_argmax(const float *v, size_t n) { /* model.rs:3277-3290 with k = 1: first strict maximum */
    int best = 0;
    for (size_t i = 1; i < n; ++i)
        if (v[i] > v[best]) best = (int)i;
    return best;
}

/* ------------------------------------------------------------------ q8 lm_head */
void or_q8head_from_f32(const float *w, size_t rows, size_t cols, int8_t *q, float *scales) { /* model.rs:274-286 */
    size_t nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r)
        or_q8_quantize(w + (size_t)r * cols, cols, q + (size_t)r * cols, scales + (size_t)r * nb);
}
void or_q8head_matvec(const int8_t *q, const float *scales, size_t rows, size_t cols,
                      const float *x, float *out, int n_threads) { /* model.rs:290-335 */
    size_t nb = cols / 32;
    int8_t *xq = (int8_t *)malloc(cols);
    float *xs = (float *)malloc(sizeof(float) * nb);
    or_q8_quantize(x, cols, xq, xs);
    if (n_threads < 1) n_threads = 1;
#pragma omp parallel for schedule(static) num_threads(n_threads)
    for (long r = 0; r < (long)rows; ++r) {
        const int8_t *wq = q + (size_t)r * cols;
        const float *ws = scales + (size_t)r * nb;
        float acc = 0.0f;
        for (size_t g = 0; g < nb; ++g) {
            int32_t idot = or_block_dot_i8(wq + g * 32, xq + g * 32);
            acc += ws[g] * xs[g] * (float)idot;
        }
        out[r] = acc;
    }
    free(xq);
    free(xs);
}

/* ------------------------------------------------------------------ KDA decode step, AttnRes */
static float or_silu(float x) { return x * or_sigmoid(x); } /* model.rs:612-615 */

void or_kda_conv_step(size_t proj, size_t kconv, const float *w_conv, float *vec, float *cache_raw) { /* model.rs:1070-1085 */
    float *out = (float *)malloc(sizeof(float) * proj);
    size_t prev = kconv - 1;
    for (size_t c = 0; c < proj; ++c) {
        float acc = 0.0f;
        for (size_t j = 0; j < prev; ++j) acc += w_conv[c * kconv + j] * cache_raw[j * proj + c];
        acc += w_conv[c * kconv + prev] * vec[c];
        out[c] = or_silu(acc);
    }
    memmove(cache_raw, cache_raw + proj, sizeof(float) * (prev - 1) * proj);
    memcpy(cache_raw + (prev - 1) * proj, vec, sizeof(float) * proj);
    memcpy(vec, out, sizeof(float) * proj);
    free(out);
}
void or_kda_norm_head(size_t heads, size_t dim, float *vec, float scale) { /* model.rs:1088-1097 */
    for (size_t h = 0; h < heads; ++h) {
        float *head = vec + h * dim;
        float n2 = or_dot(head, head, dim);
        float inv = scale / fmaxf(sqrtf(n2), 1e-12f);
        for (size_t i = 0; i < dim; ++i) head[i] *= inv;
    }
}
void or_kda_gate(size_t heads, size_t dim, float gate_lb, const float *a_log, const float *dt_bias, const float *g_low, float *g) {
    for (size_t h = 0; h < heads; ++h) /* model.rs:1100-1109 */
        for (size_t c = 0; c < dim; ++c) {
            size_t i = h * dim + c;
            g[i] = gate_lb * or_sigmoid(or_m_expf(a_log[c]) * (g_low[i] + dt_bias[i]));
        }
}
void or_kda_recur_step(size_t heads, size_t dim, float *s, const float *q, const float *k, const float *v, const float *g,
                       const float *beta, float *o) { /* model.rs:1114-1156 */
    float *delta = (float *)malloc(sizeof(float) * dim);
    for (size_t h = 0; h < heads; ++h) {
        float *sh = s + h * dim * dim;
        const float *gh = g + h * dim, *kh = k + h * dim, *vh = v + h * dim, *qh = q + h * dim;
        for (size_t i = 0; i < dim; ++i) {
            float decay = or_m_expf(gh[i]);
            for (size_t j = 0; j < dim; ++j) sh[i * dim + j] *= decay;
        }
        memcpy(delta, vh, sizeof(float) * dim);
        for (size_t i = 0; i < dim; ++i)
            for (size_t j = 0; j < dim; ++j) delta[j] -= kh[i] * sh[i * dim + j];
        float bh = beta[h];
        float *oh = o + h * dim;
        for (size_t j = 0; j < dim; ++j) oh[j] = 0.0f;
        for (size_t i = 0; i < dim; ++i) {
            float bk = bh * kh[i], qi = qh[i];
            for (size_t j = 0; j < dim; ++j) sh[i * dim + j] += bk * delta[j];
            for (size_t j = 0; j < dim; ++j) oh[j] += qi * sh[i * dim + j];
        }
    }
    free(delta);
}
void or_kda_gated_onorm(size_t heads, size_t dim, float eps, float *o, const float *o_norm, const float *g2) { /* model.rs:1167-1176 */
    for (size_t h = 0; h < heads; ++h) {
        float *oh = o + h * dim;
        float ss = or_dot(oh, oh, dim) / (float)dim;
        float inv = 1.0f / sqrtf(ss + eps);
        for (size_t c = 0; c < dim; ++c) oh[c] = oh[c] * inv * o_norm[c] * or_sigmoid(g2[h * dim + c]);
    }
}
void or_kda_step(const or_kda_desc *d, float *conv_q, float *conv_k, float *conv_v, float *s, const float *q_raw,
                 const float *k_raw, const float *v_raw, const float *g_low, const float *beta_raw, const float *g2, float *o) {
    size_t proj = d->heads * d->dim; /* model.rs:1203-1228 */
    float *q = (float *)malloc(sizeof(float) * proj), *k = (float *)malloc(sizeof(float) * proj);
    float *v = (float *)malloc(sizeof(float) * proj), *g = (float *)malloc(sizeof(float) * proj);
    float *beta = (float *)malloc(sizeof(float) * d->heads);
    memcpy(q, q_raw, sizeof(float) * proj);
    memcpy(k, k_raw, sizeof(float) * proj);
    memcpy(v, v_raw, sizeof(float) * proj);
    for (size_t h = 0; h < d->heads; ++h) beta[h] = or_sigmoid(beta_raw[h]);
    or_kda_conv_step(proj, d->kconv, d->q_conv, q, conv_q);
    or_kda_conv_step(proj, d->kconv, d->k_conv, k, conv_k);
    or_kda_conv_step(proj, d->kconv, d->v_conv, v, conv_v);
    or_kda_norm_head(d->heads, d->dim, q, powf((float)d->dim, -0.5f));
    or_kda_norm_head(d->heads, d->dim, k, 1.0f);
    or_kda_gate(d->heads, d->dim, d->gate_lb, d->a_log, d->dt_bias, g_low, g);
    or_kda_recur_step(d->heads, d->dim, s, q, k, v, g, beta, o);
    or_kda_gated_onorm(d->heads, d->dim, d->rms_eps, o, d->o_norm, g2);
    free(q); free(k); free(v); free(g); free(beta);
}
void or_kda_core(const float *q, const float *k, const float *v, const float *g, const float *beta, const float *a_log,
                 const float *dt_bias, size_t t_steps, size_t heads, size_t dim, float *o, float *s) { /* selftest.rs:48-113 */
    float scale = powf((float)dim, -0.5f);
    float *qn = (float *)malloc(sizeof(float) * dim), *kn = (float *)malloc(sizeof(float) * dim);
    float *gg = (float *)malloc(sizeof(float) * dim), *delta = (float *)malloc(sizeof(float) * dim);
    memset(s, 0, sizeof(float) * heads * dim * dim);
    for (size_t t = 0; t < t_steps; ++t)
        for (size_t h = 0; h < heads; ++h) {
            size_t base = (t * heads + h) * dim;
            const float *qh = q + base, *kh = k + base, *vh = v + base, *gh = g + base;
            float bh = 1.0f / (1.0f + or_m_expf(-beta[t * heads + h]));
            float nq = 0.0f, nk = 0.0f;
            for (size_t i = 0; i < dim; ++i) nq += qh[i] * qh[i];
            for (size_t i = 0; i < dim; ++i) nk += kh[i] * kh[i];
            nq = fmaxf(sqrtf(nq), 1e-12f);
            nk = fmaxf(sqrtf(nk), 1e-12f);
            for (size_t i = 0; i < dim; ++i) qn[i] = qh[i] / nq * scale;
            for (size_t i = 0; i < dim; ++i) kn[i] = kh[i] / nk;
            for (size_t c = 0; c < dim; ++c) {
                float a = or_m_expf(a_log[c]), x = gh[c] + dt_bias[h * dim + c];
                gg[c] = -5.0f / (1.0f + or_m_expf(-a * x));
            }
            float *sh = s + h * dim * dim;
            for (size_t i = 0; i < dim; ++i) {
                float decay = or_m_expf(gg[i]);
                for (size_t j = 0; j < dim; ++j) sh[i * dim + j] *= decay;
            }
            memcpy(delta, vh, sizeof(float) * dim);
            for (size_t i = 0; i < dim; ++i)
                for (size_t j = 0; j < dim; ++j) delta[j] -= kn[i] * sh[i * dim + j];
            float *oh = o + base;
            for (size_t j = 0; j < dim; ++j) oh[j] = 0.0f;
            for (size_t i = 0; i < dim; ++i) {
                float bk = bh * kn[i];
                for (size_t j = 0; j < dim; ++j) sh[i * dim + j] += bk * delta[j];
                for (size_t j = 0; j < dim; ++j) oh[j] += qn[i] * sh[i * dim + j];
            }
        }
    free(qn); free(kn); free(gg); free(delta);
}
void or_attn_res(size_t d, float eps, const float *prefix, const float *blocks, size_t b, const float *w, float *out) {
    float *scores = (float *)malloc(sizeof(float) * (b + 1)); /* model.rs:632-669 */
    float *kbuf = (float *)malloc(sizeof(float) * d);
    for (size_t i = 0; i <= b; ++i) {
        const float *v = i < b ? blocks + i * d : prefix;
        float ss = or_dot(v, v, d) / (float)d;
        float inv = 1.0f / sqrtf(ss + eps);
        for (size_t j = 0; j < d; ++j) kbuf[j] = v[j] * inv;
        scores[i] = or_dot(kbuf, w, d);
    }
    float m = -INFINITY;
    for (size_t i = 0; i <= b; ++i) m = fmaxf(m, scores[i]);
    float z = 0.0f;
    for (size_t i = 0; i <= b; ++i) {
        scores[i] = or_m_expf(scores[i] - m);
        z += scores[i];
    }
    for (size_t i = 0; i <= b; ++i) scores[i] /= z;
    for (size_t j = 0; j < d; ++j) out[j] = 0.0f;
    for (size_t i = 0; i < b; ++i)
        for (size_t j = 0; j < d; ++j) out[j] += scores[i] * blocks[i * d + j];
    for (size_t j = 0; j < d; ++j) out[j] += scores[b] * prefix[j];
    free(scores); free(kbuf);
}

uint16_t or_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? 0x200u : 0)); /* inf/nan */
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);                                      /* overflow -> inf */
    if (ax < 0x33000001u) return (uint16_t)sign;                                                   /* underflow -> 0 */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    uint32_t shift, half;
    if (e < -14) shift = (uint32_t)(13 + (-14 - e)); else shift = 13;
    uint32_t res = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    half = 1u << (shift - 1);
    if (rem > half || (rem == half && (res & 1u))) res++;
    if (e < -14) return (uint16_t)(sign | res); /* subnormal (res may carry into exp=1, still right) */
    res += ((uint32_t)(e + 15 - 1)) << 10;      /* res holds implicit 1 at bit 10 -> adds 1 to exponent */
    return (uint16_t)(sign | res);
}
float or_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF;
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        float v = ldexpf((float)m, -24);
        return sign ? -v : v;
    }
    if (e == 31) return bits_f32(sign | 0x7F800000u | (m << 13));
    return bits_f32(sign | ((e + 112) << 23) | (m << 13));
}
/* f16-scale variant: dx is rounded to half FIRST, then q = round(x / dx_h). */
void or_q8head_from_f32_f16s(const float *w, size_t rows, size_t cols, int8_t *q, uint16_t *scales_h) {
    size_t nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < (long)rows; ++r) {
        for (size_t g = 0; g < nb; ++g) {
            const float *b = w + (size_t)r * cols + g * 32;
            int8_t *qq = q + (size_t)r * cols + g * 32;
            float max = 0.0f;
            for (int j = 0; j < 32; ++j) max = fmaxf(max, fabsf(b[j]));
            uint16_t hs = or_f32_to_f16(max / 127.0f);
            float dx = or_f16_to_f32(hs);
            scales_h[(size_t)r * nb + g] = hs;
            for (int j = 0; j < 32; ++j)
                qq[j] = (dx == 0.0f) ? 0 : (int8_t)clampf(roundf(b[j] / dx), -127.0f, 127.0f);
        }
    }
}
void or_q8head_matvec_f16s(const int8_t *q, const uint16_t *scales_h, size_t rows, size_t cols,
                           const float *x, float *out, int n_threads) {
    size_t nb = cols / 32;
    int8_t *xq = (int8_t *)malloc(cols);
    float *xs = (float *)malloc(sizeof(float) * nb);
    or_q8_quantize(x, cols, xq, xs);
    if (n_threads < 1) n_threads = 1;
#pragma omp parallel for schedule(static) num_threads(n_threads)
    for (long r = 0; r < (long)rows; ++r) {
        float acc = 0.0f;
        for (size_t g = 0; g < nb; ++g) {
            int32_t idot = or_block_dot_i8(q + (size_t)r * cols + g * 32, xq + g * 32);
            acc += or_f16_to_f32(scales_h[(size_t)r * nb + g]) * xs[g] * (float)idot;
        }
        out[r] = acc;
    }
    free(xq);
    free(xs);
}

/* ------------------------------------------------------------------ routers */
typedef struct { int32_t id; float score; float key; } sel_t;
/* Rust's sort_by is stable; k is small, insertion sort keeps stability. */
static void stable_sort_desc(sel_t *s, size_t n) {
    for (size_t i = 1; i < n; ++i) {
        sel_t v = s[i];
        size_t j = i;
        while (j > 0 && s[j - 1].key < v.key) { s[j] = s[j - 1]; --j; }
        s[j] = v;
    }
}
static void topk_stream(const float *score, const float *key, size_t n, size_t k, sel_t *sel) {
    size_t len = 0;
    for (size_t i = 0; i < n; ++i) { /* model.rs:2158-2171 */
        sel_t item = { (int32_t)i, score[i], key[i] };
        if (len < k) {
            sel[len++] = item;
            if (len == k) stable_sort_desc(sel, k);
        } else if (item.key > sel[k - 1].key) {
            sel[k - 1] = item;
            stable_sort_desc(sel, k);
        }
    }
}
void or_router_k3(const float *gate_w, const float *gate_b, size_t n_experts, size_t d, size_t top_k,
                  const float *x, int32_t *ids, float *weights, float *logits_out) {
    float *logits = (float *)malloc(sizeof(float) * n_experts);
    float *sc = (float *)malloc(sizeof(float) * n_experts);
    float *key = (float *)malloc(sizeof(float) * n_experts);
    sel_t *sel = (sel_t *)malloc(sizeof(sel_t) * top_k);
    or_matvec_f32(gate_w, n_experts, d, x, logits, 1);
    for (size_t i = 0; i < n_experts; ++i) {
        sc[i] = or_sigmoid(logits[i]);
        key[i] = sc[i] + gate_b[i];
    }
    topk_stream(sc, key, n_experts, top_k, sel);
    float sumw = 0.0f;
    for (size_t i = 0; i < top_k; ++i) sumw += sel[i].score; /* model.rs:2172 */
    sumw += 1e-20f;
    for (size_t i = 0; i < top_k; ++i) {
        ids[i] = sel[i].id;
        weights[i] = sel[i].score / sumw;
    }
    if (logits_out) memcpy(logits_out, logits, sizeof(float) * n_experts);
    free(logits); free(sc); free(key); free(sel);
}
static float softplus(float x) { return x > 20.0f ? x : or_m_logf(1.0f + or_m_expf(x)); } /* deepseek.rs:60-68 */
void or_gate_ds(const float *gate_w, const float *bias, size_t n_experts, size_t d, size_t top_k,
                float route_scale, const float *x, int32_t *ids, float *weights) {
    float *logits = (float *)malloc(sizeof(float) * n_experts);
    float *orig = (float *)malloc(sizeof(float) * n_experts);
    float *key = (float *)malloc(sizeof(float) * n_experts);
    sel_t *sel = (sel_t *)malloc(sizeof(sel_t) * top_k);
    or_matvec_f32(gate_w, n_experts, d, x, logits, 1);
    for (size_t i = 0; i < n_experts; ++i) {
        orig[i] = sqrtf(softplus(logits[i]));
        key[i] = orig[i] + (bias ? bias[i] : 0.0f);
    }
    topk_stream(orig, key, n_experts, top_k, sel);
    float sum = 0.0f;
    for (size_t i = 0; i < top_k; ++i) sum += orig[sel[i].id];
    for (size_t i = 0; i < top_k; ++i) {
        ids[i] = sel[i].id;
        weights[i] = orig[sel[i].id] / sum * route_scale; /* deepseek.rs:52-56 */
    }
    free(logits); free(orig); free(key); free(sel);
}

/* ------------------------------------------------------------------ experts */
void or_expert_ds_f32(const float *w1, const float *w2, const float *w3, const float *x,
                      size_t d, size_t inter, float limit, float *out) { /* deepseek.rs:74-95 */
    float *gate = (float *)malloc(sizeof(float) * inter);
    float *up = (float *)malloc(sizeof(float) * inter);
    float *act = (float *)malloc(sizeof(float) * inter);
    or_matvec_f32(w1, inter, d, x, gate, 1);
    or_matvec_f32(w3, inter, d, x, up, 1);
    for (size_t i = 0; i < inter; ++i) {
        float g = fminf(gate[i], limit);
        float u = clampf(up[i], -limit, limit);
        act[i] = (g / (1.0f + or_m_expf(-g))) * u; /* deepseek.rs:97-100 silu */
    }
    or_matvec_f32(w2, d, inter, act, out, 1);
    free(gate); free(up); free(act);
}

/* deepseek.rs:1069-1093 : one routed expert, routing weight folded before w2 */
static void expert_ds_mxfp4(const uint8_t *const p[3], const uint8_t *const s[3], size_t d, size_t inter,
                            float limit, float wgt, int use_q8, const float *x, float *o) {
    float *gate = (float *)malloc(sizeof(float) * inter);
    float *up = (float *)malloc(sizeof(float) * inter);
    float *act = (float *)malloc(sizeof(float) * inter);
    or_mxfp4_matvec(p[0], s[0], inter, d, x, gate, 1, use_q8);
    or_mxfp4_matvec(p[2], s[2], inter, d, x, up, 1, use_q8);
    for (size_t j = 0; j < inter; ++j) {
        float g = fminf(gate[j], limit);
        float u = clampf(up[j], -limit, limit);
        act[j] = wgt * (g / (1.0f + or_m_expf(-g))) * u;
    }
    or_mxfp4_matvec(p[1], s[1], d, inter, act, o, 1, use_q8);
    free(gate); free(up); free(act);
}
void or_moe_ds_forward(const or_moe_ds_desc *m, const float *x, float *out,
                       int32_t *ids_out, float *w_out, int n_threads) {
    size_t k = m->top_k, d = m->d;
    int32_t *ids = (int32_t *)malloc(sizeof(int32_t) * k);
    float *wts = (float *)malloc(sizeof(float) * k);
    float *outs = (float *)malloc(sizeof(float) * (k + 1) * d);
    or_router_k3(m->gate_w, m->gate_b, m->n_experts, d, k, x, ids, wts, NULL);
    if (n_threads < 1) n_threads = 1;
    /* one job per selected expert (deepseek.rs:1069-1094) + the shared expert */
#pragma omp parallel for schedule(dynamic, 1) num_threads(n_threads)
    for (long ei = 0; ei <= (long)k; ++ei) {
        if (ei < (long)k) {
            const uint8_t *p[3], *s[3];
            for (int j = 0; j < 3; ++j) {
                p[j] = m->packed[(size_t)ids[ei] * 3 + j];
                s[j] = m->scales[(size_t)ids[ei] * 3 + j];
            }
            expert_ds_mxfp4(p, s, d, m->inter, m->limit, wts[ei], m->use_q8, x, outs + (size_t)ei * d);
        } else {
            /* shared expert, unweighted (deepseek.rs:1101-1103); wgt = 1.0 is exact */
            expert_ds_mxfp4(m->sh_packed, m->sh_scales, d, m->inter, m->limit, 1.0f, m->use_q8, x, outs + k * d);
        }
    }
    for (size_t j = 0; j < d; ++j) out[j] = 0.0f;
    for (size_t ei = 0; ei < k; ++ei) /* deepseek.rs:1095-1100, slot order */
        for (size_t j = 0; j < d; ++j) out[j] += outs[ei * d + j];
    for (size_t j = 0; j < d; ++j) out[j] += outs[k * d + j]; /* deepseek.rs:1104-1106 */
    if (ids_out) memcpy(ids_out, ids, sizeof(int32_t) * k);
    if (w_out) memcpy(w_out, wts, sizeof(float) * k);
    free(ids); free(wts); free(outs);
}

/* ------------------------------------------------------------------ FP8 e4m3fn dequant */
float or_e4m3_to_f32(uint8_t b) { /* dequant.rs:12-23 */
    float sign = (b & 0x80) ? -1.0f : 1.0f;
    int e = (b >> 3) & 0x0F;
    float m = (float)(b & 0x07);
    if (e == 15 && (b & 0x07) == 7) return NAN;
    if (e == 0) return sign * (m / 8.0f) * 0.015625f; /* 2^-6 */
    return sign * (1.0f + m / 8.0f) * or_exp2_i(e - 7);
}
void or_dequant_fp8(const uint8_t *w, const uint8_t *scales, size_t rows, size_t cols, float *out) { /* dequant.rs:27-41 */
    size_t scols = (cols + 127) / 128;
    for (size_t r = 0; r < rows; ++r)
        for (size_t c = 0; c < cols; ++c) {
            float s = or_exp2_i((int)scales[(r / 128) * scols + c / 128] - 127);
            out[r * cols + c] = or_e4m3_to_f32(w[r * cols + c]) * s;
        }
}

/* ------------------------------------------------------------------ VQ1 codebook matvec */
void or_matvec_vq_gather(const float *codebook, const uint8_t *indices, size_t rows, size_t cols, const float *x, float *out) {
    size_t vpr = cols / 16; /* quant.rs:317-335 */
    for (size_t r = 0; r < rows; ++r) {
        float sum = 0.0f;
        for (size_t v = 0; v < vpr; ++v) {
            const float *cb = codebook + (size_t)indices[r * vpr + v] * 16, *xs = x + v * 16;
            float s = 0.0f;
            for (size_t j = 0; j < 16; ++j) s += cb[j] * xs[j];
            sum += s;
        }
        out[r] = sum;
    }
}
void or_matvec_vq_lut(const float *codebook, const uint8_t *indices, size_t rows, size_t cols, const float *x, float *out) {
    size_t vpr = cols / 16; /* lutgemv.rs:208-238, tiles of 16 groups */
    float *lut = (float *)malloc(sizeof(float) * 16 * 256);
    for (size_t r = 0; r < rows; ++r) out[r] = 0.0f;
    for (size_t g0 = 0; g0 < vpr; g0 += 16) {
        size_t groups = vpr - g0 < 16 ? vpr - g0 : 16;
        for (size_t g = 0; g < groups; ++g)
            for (size_t k = 0; k < 256; ++k) { /* lutgemv.rs:116-125 */
                float s = 0.0f;
                for (size_t j = 0; j < 16; ++j) s += codebook[k * 16 + j] * x[(g0 + g) * 16 + j];
                lut[g * 256 + k] = s;
            }
        for (size_t r = 0; r < rows; ++r) { /* lutgemv.rs:67-92 */
            float a = out[r];
            for (size_t g = 0; g < groups; ++g) a += lut[g * 256 + indices[r * vpr + g0 + g]];
            out[r] = a;
        }
    }
    free(lut);
}

/* model.rs:2150-2380 : K3 latent MoE layer, one token */
void or_moe_k3_forward(const or_moe_k3_desc *m, const float *x, float *out, int32_t *ids_out, float *w_out) {
    size_t k = m->top_k, d = m->d, rh = m->rh, I = m->inter;
    int32_t *ids = (int32_t *)malloc(sizeof(int32_t) * k);
    float *wts = (float *)malloc(sizeof(float) * k);
    float *h = (float *)malloc(sizeof(float) * rh);
    float *outs = (float *)malloc(sizeof(float) * k * rh);
    float *a = (float *)malloc(sizeof(float) * I), *u = (float *)malloc(sizeof(float) * I), *act = (float *)malloc(sizeof(float) * I);
    float *y = (float *)calloc(rh, sizeof(float)), *yn = (float *)malloc(sizeof(float) * rh);
    or_router_k3(m->gate_w, m->gate_b, m->n_experts, d, k, x, ids, wts, NULL);   /* :2152-2173 */
    or_matvec_f32(m->routed_down, rh, d, x, h, 1);                               /* :2202-2203 */
    for (size_t ei = 0; ei < k; ++ei) {                                          /* :2227-2260 */
        const uint8_t *const *p = m->packed + (size_t)ids[ei] * 3, *const *s = m->scales + (size_t)ids[ei] * 3;
        or_mxfp4_matvec(p[0], s[0], I, rh, h, a, 1, m->use_q8);
        or_mxfp4_matvec(p[2], s[2], I, rh, h, u, 1, m->use_q8);
        for (size_t j = 0; j < I; ++j) act[j] = or_situ(a[j], u[j]);
        or_mxfp4_matvec(p[1], s[1], rh, I, act, outs + ei * rh, 1, m->use_q8);
    }
    for (size_t ei = 0; ei < k; ++ei)                                            /* :2346-2351 */
        for (size_t j = 0; j < rh; ++j) y[j] += wts[ei] * outs[ei * rh + j];
    or_rmsnorm(y, m->routed_norm, rh, m->rms_eps, yn);                           /* :2352-2354 */
    or_matvec_f32(m->routed_up, d, rh, yn, out, 1);                              /* :2355-2356 */
    if (m->shared_gate) {                                                        /* :2357-2378 */
        size_t si = m->shared_inter;
        float *sa = (float *)malloc(sizeof(float) * si), *su = (float *)malloc(sizeof(float) * si);
        float *sout = (float *)malloc(sizeof(float) * d);
        or_matvec_f32(m->shared_gate, si, d, x, sa, 1);
        or_matvec_f32(m->shared_up, si, d, x, su, 1);
        for (size_t j = 0; j < si; ++j) sa[j] = or_situ(sa[j], su[j]);
        or_matvec_f32(m->shared_down, d, si, sa, sout, 1);
        for (size_t j = 0; j < d; ++j) out[j] += sout[j];
        free(sa); free(su); free(sout);
    }
    if (ids_out) memcpy(ids_out, ids, sizeof(int32_t) * k);
    if (w_out) memcpy(w_out, wts, sizeof(float) * k);
    free(ids); free(wts); free(h); free(outs); free(a); free(u); free(act); free(y); free(yn);
}

/* ------------------------------------------------------------------ MLA, per-head layout */
or_mla_cache *or_mla_new(size_t nh, size_t nope, size_t rope, size_t vd, size_t cap) {
    or_mla_cache *c = (or_mla_cache *)calloc(1, sizeof(*c));
    c->nh = nh; c->nope = nope; c->rope = rope; c->vd = vd; c->cap = cap; c->n = 0;
    c->kq = (int8_t *)malloc(cap * nh * nope);
    c->ks = (float *)malloc(sizeof(float) * cap * nh * (nope / 32));
    c->kr = (float *)malloc(sizeof(float) * cap * rope);
    c->vq = (int8_t *)malloc(cap * nh * vd);
    c->vs = (float *)malloc(sizeof(float) * cap * nh * (vd / 32));
    return c;
}
void or_mla_free(or_mla_cache *c) {
    if (!c) return;
    free(c->kq); free(c->ks); free(c->kr); free(c->vq); free(c->vs); free(c);
}
void or_mla_push(or_mla_cache *c, const float *k_row, const float *v_row) { /* model.rs:1583-1618 */
    size_t nh = c->nh, nope = c->nope, rope = c->rope, vd = c->vd, qh = nope + rope, j = c->n;
    if (j >= c->cap) return;
    memcpy(c->kr + j * rope, k_row + nope, sizeof(float) * rope); /* rope from head 0 */
    for (size_t h = 0; h < nh; ++h) {
        or_q8_quantize(k_row + h * qh, nope, c->kq + (j * nh + h) * nope, c->ks + (j * nh + h) * (nope / 32));
        or_q8_quantize(v_row + h * vd, vd, c->vq + (j * nh + h) * vd, c->vs + (j * nh + h) * (vd / 32));
    }
    c->n = j + 1;
}
void or_mla_to_f32(const or_mla_cache *c, float *k, float *v) { /* model.rs:1623-1676 */
    size_t nh = c->nh, nope = c->nope, rope = c->rope, vd = c->vd, qh = nope + rope;
    for (size_t j = 0; j < c->n; ++j)
        for (size_t h = 0; h < nh; ++h) {
            for (size_t i = 0; i < nope; ++i)
                k[(j * nh + h) * qh + i] = (float)c->kq[(j * nh + h) * nope + i] * c->ks[(j * nh + h) * (nope / 32) + i / 32];
            memcpy(k + (j * nh + h) * qh + nope, c->kr + j * rope, sizeof(float) * rope);
            for (size_t i = 0; i < vd; ++i)
                v[(j * nh + h) * vd + i] = (float)c->vq[(j * nh + h) * vd + i] * c->vs[(j * nh + h) * (vd / 32) + i / 32];
        }
}
void or_mla_attn_flash_q8(const or_mla_cache *c, const float *qh, size_t h, size_t pos, float scale, float *oh) {
    size_t nh = c->nh, nope = c->nope, rope = c->rope, vd = c->vd, nb = nope / 32;
    int8_t *qq = (int8_t *)malloc(nope);
    float *qs = (float *)malloc(sizeof(float) * nb);
    float *vtile = (float *)malloc(sizeof(float) * FLASH_KV * vd);
    or_q8_quantize(qh, nope, qq, qs);
    const float *q_rope = qh + nope;
    float m = -INFINITY, l = 0.0f, scores[FLASH_KV];
    for (size_t d = 0; d < vd; ++d) oh[d] = 0.0f;
    size_t t = 0;
    while (t <= pos) {
        size_t end = t + FLASH_KV - 1 < pos ? t + FLASH_KV - 1 : pos;
        size_t tn = end - t + 1;
        float tm = -INFINITY;
        for (size_t i = 0; i < tn; ++i) {
            size_t j = t + i;
            float s = or_dot(q_rope, c->kr + j * rope, rope);
            float acc = 0.0f;
            size_t bq = (j * nh + h) * nope, bs = (j * nh + h) * nb;
            for (size_t g = 0; g < nb; ++g) {
                int32_t d = or_block_dot_i8(c->kq + bq + g * 32, qq + g * 32);
                acc += qs[g] * c->ks[bs + g] * (float)d;
            }
            s += 1.0f * acc;
            s = s * scale;
            scores[i] = s;
            tm = fmaxf(tm, s);
        }
        float m_new = fmaxf(m, tm);
        float corr = or_m_expf(m - m_new);
        float tile_l = 0.0f;
        for (size_t i = 0; i < tn; ++i) { scores[i] = or_m_expf(scores[i] - m_new); tile_l += scores[i]; }
        for (size_t d = 0; d < vd; ++d) oh[d] *= corr;
        l = l * corr + tile_l;
        for (size_t i = 0; i < tn; ++i) {
            size_t j = t + i;
            size_t bq = (j * nh + h) * vd, bs = (j * nh + h) * (vd / 32);
            float *out = vtile + i * vd;
            for (size_t g = 0; g < vd / 32; ++g) {
                float sc = c->vs[bs + g];
                for (size_t d2 = 0; d2 < 32; ++d2) out[g * 32 + d2] = (float)c->vq[bq + g * 32 + d2] * sc;
            }
            float p = scores[i];
            for (size_t d = 0; d < vd; ++d) oh[d] += p * out[d];
        }
        m = m_new;
        t = end + 1;
    }
    for (size_t d = 0; d < vd; ++d) oh[d] /= l;
    free(qq); free(qs); free(vtile);
}
void or_mla_attn_flash_q8_mqa(const or_mla_cache *c, const float *q, size_t pos, float scale, float *attn) {
    size_t nh = c->nh, nope = c->nope, rope = c->rope, vd = c->vd, hd = nope + rope, nb = nope / 32, nbv = vd / 32;
    int8_t *qq = (int8_t *)malloc(nh * nope);
    float *qs = (float *)malloc(sizeof(float) * nh * nb);
    float *m = (float *)malloc(sizeof(float) * nh);
    float *l = (float *)malloc(sizeof(float) * nh);
    float *scores = (float *)malloc(sizeof(float) * nh * FLASH_KV);
    float *vtile = (float *)malloc(sizeof(float) * vd);
    for (size_t h = 0; h < nh; ++h) {
        or_q8_quantize(q + h * hd, nope, qq + h * nope, qs + h * nb);
        m[h] = -INFINITY;
        l[h] = 0.0f;
    }
    for (size_t i = 0; i < nh * vd; ++i) attn[i] = 0.0f;
    size_t t = 0;
    while (t <= pos) {
        size_t end = t + FLASH_KV - 1 < pos ? t + FLASH_KV - 1 : pos;
        size_t tn = end - t + 1;
        for (size_t i = 0; i < tn; ++i) {
            size_t j = t + i;
            const float *kr = c->kr + j * rope;
            const int8_t *kq = c->kq + j * nh * nope;
            const float *ks = c->ks + j * nh * nb;
            for (size_t h = 0; h < nh; ++h) {
                float s = or_dot(q + h * hd + nope, kr, rope);
                float acc = 0.0f;
                for (size_t g = 0; g < nb; ++g) {
                    int32_t d = or_block_dot_i8(kq + h * nope + g * 32, qq + h * nope + g * 32);
                    acc += qs[h * nb + g] * ks[h * nb + g] * (float)d;
                }
                s += 1.0f * acc;
                scores[h * FLASH_KV + i] = s * scale;
            }
        }
        for (size_t h = 0; h < nh; ++h) {
            float *sh = scores + h * FLASH_KV;
            float tm = -INFINITY;
            for (size_t i = 0; i < tn; ++i) tm = fmaxf(tm, sh[i]);
            float m_new = fmaxf(m[h], tm);
            float corr = or_m_expf(m[h] - m_new);
            float tile_l = 0.0f;
            for (size_t i = 0; i < tn; ++i) { sh[i] = or_m_expf(sh[i] - m_new); tile_l += sh[i]; }
            float *oh = attn + h * vd;
            for (size_t d = 0; d < vd; ++d) oh[d] *= corr;
            l[h] = l[h] * corr + tile_l;
            m[h] = m_new;
        }
        for (size_t i = 0; i < tn; ++i) {
            size_t j = t + i;
            const int8_t *vq = c->vq + j * nh * vd;
            const float *vs = c->vs + j * nh * nbv;
            for (size_t h = 0; h < nh; ++h) {
                for (size_t g = 0; g < nbv; ++g) {
                    float sc = vs[h * nbv + g];
                    for (size_t d2 = 0; d2 < 32; ++d2) vtile[g * 32 + d2] = (float)vq[h * vd + g * 32 + d2] * sc;
                }
                float p = scores[h * FLASH_KV + i];
                float *oh = attn + h * vd;
                for (size_t d = 0; d < vd; ++d) oh[d] += p * vtile[d];
            }
        }
        t = end + 1;
    }
    for (size_t h = 0; h < nh; ++h)
        for (size_t d = 0; d < vd; ++d) attn[h * vd + d] /= l[h];
    free(qq); free(qs); free(m); free(l); free(scores); free(vtile);
}
void or_mla_attn_ref_q8(const or_mla_cache *c, const float *qh, size_t h, size_t pos, float scale, float *oh) {
    size_t nh = c->nh, hd = c->nope + c->rope, vd = c->vd;
    float *k = (float *)malloc(sizeof(float) * c->n * nh * hd);
    float *v = (float *)malloc(sizeof(float) * c->n * nh * vd);
    or_mla_to_f32(c, k, v);
    or_mla_attn_ref_f32(k, v, nh, hd, vd, qh, h, pos, scale, oh);
    free(k); free(v);
}
void or_mla_attn_ref_f32(const float *k, const float *v, size_t nh, size_t hd, size_t vd,
                         const float *qh, size_t h, size_t pos, float scale, float *oh) { /* model.rs:1353-1375 */
    float *scores = (float *)malloc(sizeof(float) * (pos + 1));
    for (size_t j = 0; j <= pos; ++j) scores[j] = or_dot(qh, k + (j * nh + h) * hd, hd) * scale;
    float m = -INFINITY;
    for (size_t j = 0; j <= pos; ++j) m = fmaxf(m, scores[j]);
    float z = 0.0f;
    for (size_t j = 0; j <= pos; ++j) { scores[j] = or_m_expf(scores[j] - m); z += scores[j]; }
    for (size_t j = 0; j <= pos; ++j) scores[j] /= z;
    for (size_t d = 0; d < vd; ++d) oh[d] = 0.0f;
    for (size_t j = 0; j <= pos; ++j) {
        const float *vj = v + (j * nh + h) * vd;
        float p = scores[j];
        for (size_t d = 0; d < vd; ++d) oh[d] += p * vj[d];
    }
    free(scores);
}
void or_mla_attn_flash_f32(const float *k, const float *v, size_t nh, size_t hd, size_t vd,
                           const float *qh, size_t h, size_t pos, float scale, float *oh) { /* model.rs:1385-1425 */
    float m = -INFINITY, l = 0.0f, scores[FLASH_KV];
    for (size_t d = 0; d < vd; ++d) oh[d] = 0.0f;
    size_t t = 0;
    while (t <= pos) {
        size_t end = t + FLASH_KV - 1 < pos ? t + FLASH_KV - 1 : pos;
        size_t tn = end - t + 1;
        float tm = -INFINITY;
        for (size_t i = 0; i < tn; ++i) {
            float s = or_dot(qh, k + ((t + i) * nh + h) * hd, hd) * scale;
            scores[i] = s;
            tm = fmaxf(tm, s);
        }
        float m_new = fmaxf(m, tm);
        float corr = or_m_expf(m - m_new);
        float tile_l = 0.0f;
        for (size_t i = 0; i < tn; ++i) { scores[i] = or_m_expf(scores[i] - m_new); tile_l += scores[i]; }
        for (size_t d = 0; d < vd; ++d) oh[d] *= corr;
        l = l * corr + tile_l;
        for (size_t i = 0; i < tn; ++i) {
            const float *vj = v + ((t + i) * nh + h) * vd;
            float p = scores[i];
            for (size_t d = 0; d < vd; ++d) oh[d] += p * vj[d];
        }
        m = m_new;
        t = end + 1;
    }
    for (size_t d = 0; d < vd; ++d) oh[d] /= l;
}

/* ------------------------------------------------------------------ MLA, absorbed shared-latent layout */
or_mla_abs_cache *or_mla_abs_new(size_t lat, size_t vd, size_t cap) {
    or_mla_abs_cache *c = (or_mla_abs_cache *)calloc(1, sizeof(*c));
    c->lat = lat; c->vd = vd; c->cap = cap; c->n = 0;
    c->q = (int8_t *)malloc(cap * lat);
    c->s = (float *)malloc(sizeof(float) * cap * (lat / 32));
    return c;
}
void or_mla_abs_free(or_mla_abs_cache *c) { if (c) { free(c->q); free(c->s); free(c); } }
void or_mla_abs_push(or_mla_abs_cache *c, const float *row) {
    if (c->n >= c->cap) return;
    or_q8_quantize(row, c->lat, c->q + c->n * c->lat, c->s + c->n * (c->lat / 32));
    c->n++;
}
/* Per head: the query row (all `lat` columns, rope part included - the layout
 * quantizes rope too) -> q8; score = (sum_g (qs[g]*ks[g])*idot) * scale as in
 * model.rs:1843-1849; online softmax in 64-position tiles (:1854-1870); V row =
 * first vd columns dequantized (int8 * block scale) then o += p*v (:1874-1890);
 * final o /= l (:1903-1907). */
void or_mla_abs_attn(const or_mla_abs_cache *c, const float *q, size_t nh, size_t pos, float scale, float *out) {
    size_t lat = c->lat, vd = c->vd, nb = lat / 32, nbv = vd / 32;
    int8_t *qq = (int8_t *)malloc(nh * lat);
    float *qs = (float *)malloc(sizeof(float) * nh * nb);
    float *m = (float *)malloc(sizeof(float) * nh);
    float *l = (float *)malloc(sizeof(float) * nh);
    float *scores = (float *)malloc(sizeof(float) * nh * FLASH_KV);
    float *vtile = (float *)malloc(sizeof(float) * vd);
    for (size_t h = 0; h < nh; ++h) {
        or_q8_quantize(q + h * lat, lat, qq + h * lat, qs + h * nb);
        m[h] = -INFINITY;
        l[h] = 0.0f;
    }
    for (size_t i = 0; i < nh * vd; ++i) out[i] = 0.0f;
    size_t t = 0;
    while (t <= pos) {
        size_t end = t + FLASH_KV - 1 < pos ? t + FLASH_KV - 1 : pos;
        size_t tn = end - t + 1;
        for (size_t i = 0; i < tn; ++i) {
            const int8_t *kq = c->q + (t + i) * lat;
            const float *ks = c->s + (t + i) * nb;
            for (size_t h = 0; h < nh; ++h) {
                float acc = 0.0f;
                for (size_t g = 0; g < nb; ++g) {
                    int32_t d = or_block_dot_i8(kq + g * 32, qq + h * lat + g * 32);
                    acc += qs[h * nb + g] * ks[g] * (float)d;
                }
                scores[h * FLASH_KV + i] = acc * scale;
            }
        }
        for (size_t h = 0; h < nh; ++h) {
            float *sh = scores + h * FLASH_KV;
            float tm = -INFINITY;
            for (size_t i = 0; i < tn; ++i) tm = fmaxf(tm, sh[i]);
            float m_new = fmaxf(m[h], tm);
            float corr = or_m_expf(m[h] - m_new);
            float tile_l = 0.0f;
            for (size_t i = 0; i < tn; ++i) { sh[i] = or_m_expf(sh[i] - m_new); tile_l += sh[i]; }
            float *oh = out + h * vd;
            for (size_t d = 0; d < vd; ++d) oh[d] *= corr;
            l[h] = l[h] * corr + tile_l;
            m[h] = m_new;
        }
        for (size_t i = 0; i < tn; ++i) {
            const int8_t *vq = c->q + (t + i) * lat;
            const float *vs = c->s + (t + i) * nb;
            for (size_t g = 0; g < nbv; ++g)
                for (size_t d2 = 0; d2 < 32; ++d2) vtile[g * 32 + d2] = (float)vq[g * 32 + d2] * vs[g];
            for (size_t h = 0; h < nh; ++h) {
                float p = scores[h * FLASH_KV + i];
                float *oh = out + h * vd;
                for (size_t d = 0; d < vd; ++d) oh[d] += p * vtile[d];
            }
        }
        t = end + 1;
    }
    for (size_t h = 0; h < nh; ++h)
        for (size_t d = 0; d < vd; ++d) out[h * vd + d] /= l[h];
    free(qq); free(qs); free(m); free(l); free(scores); free(vtile);
}
void or_mla_abs_attn_f64(const or_mla_abs_cache *c, const float *q, size_t nh, size_t pos, float scale, double *out) {
    size_t lat = c->lat, vd = c->vd, nb = lat / 32;
    double *sc = (double *)malloc(sizeof(double) * (pos + 1));
    for (size_t h = 0; h < nh; ++h) {
        double mx = -INFINITY;
        for (size_t j = 0; j <= pos; ++j) {
            double s = 0.0;
            for (size_t i = 0; i < lat; ++i)
                s += (double)q[h * lat + i] * ((double)c->q[j * lat + i] * (double)c->s[j * nb + i / 32]);
            sc[j] = s * (double)scale;
            if (sc[j] > mx) mx = sc[j];
        }
        double z = 0.0;
        for (size_t j = 0; j <= pos; ++j) { sc[j] = exp(sc[j] - mx); z += sc[j]; }
        for (size_t d = 0; d < vd; ++d) {
            double o = 0.0;
            for (size_t j = 0; j <= pos; ++j) o += sc[j] * ((double)c->q[j * lat + d] * (double)c->s[j * nb + d / 32]);
            out[h * vd + d] = o / z;
        }
    }
    free(sc);
}
