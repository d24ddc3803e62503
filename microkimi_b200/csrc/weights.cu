// Weight registration kernels: natural row-major blobs <-> the fragment-major
// device layout described at mk_weight (mk_common.cuh), the bit-exact q8_0 row
// quantizer (Q8Head::from_f32, src/model.rs:274-286) and the MXFP4 dequantizer
// (mxfp4::dequant, src/mxfp4.rs:19-31).  All of them only move or re-encode
// bytes; values are unchanged and mk_weight_export() undoes the tiling.
#include <cuda_fp16.h>

#include "mk_common.cuh"

namespace {

__constant__ float c_e2m1[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                 -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

// ---- MXFP4: one thread per tiled 32-bit word (8 codes)
__global__ void retile_mxfp4_kernel(const uint8_t *__restrict__ packed, const uint8_t *__restrict__ scales,
                                    uint32_t *__restrict__ tv, uint8_t *__restrict__ ts, int64_t rows, int64_t cols,
                                    int64_t nrt, int64_t nb, int64_t nbp) {
    const int64_t nwords = nrt * (nbp / 2) * 128;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < nwords) {
        const int64_t chunk = idx >> 7;
        const int within = (int)(idx & 127);
        const int lane = within >> 2, j = within & 3;
        const int g = lane >> 2, t = lane & 3;
        const int64_t rt = chunk / (nbp / 2), bp = chunk % (nbp / 2);
        const int64_t row = rt * 16 + g + ((j & 1) ? 8 : 0);
        const int64_t b = bp * 2 + (j >> 1);
        uint32_t v = 0;
        if (row < rows && b < nb) v = *(const uint32_t *)(packed + row * (cols / 2) + b * 16 + t * 4);
        tv[idx] = v;
    }
    const int64_t nsc = nrt * nbp * 16;
    if (idx < nsc) {
        const int r16 = (int)(idx & 15);
        const int64_t rb = idx >> 4;
        const int64_t rt = rb / nbp, b = rb % nbp;
        const int64_t row = rt * 16 + r16;
        ts[mk_scale_off(rt, nbp, b, r16)] = (row < rows && b < nb) ? scales[row * nb + b] : (uint8_t)0;
    }
}
__global__ void untile_mxfp4_kernel(const uint32_t *__restrict__ tv, const uint8_t *__restrict__ ts,
                                    uint8_t *__restrict__ packed, uint8_t *__restrict__ scales, int64_t rows,
                                    int64_t cols, int64_t nrt, int64_t nb, int64_t nbp) {
    const int64_t nwords = nrt * (nbp / 2) * 128;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < nwords) {
        const int64_t chunk = idx >> 7;
        const int within = (int)(idx & 127);
        const int lane = within >> 2, j = within & 3;
        const int g = lane >> 2, t = lane & 3;
        const int64_t rt = chunk / (nbp / 2), bp = chunk % (nbp / 2);
        const int64_t row = rt * 16 + g + ((j & 1) ? 8 : 0);
        const int64_t b = bp * 2 + (j >> 1);
        if (row < rows && b < nb) *(uint32_t *)(packed + row * (cols / 2) + b * 16 + t * 4) = tv[idx];
    }
    const int64_t nsc = nrt * nbp * 16;
    if (idx < nsc) {
        const int r16 = (int)(idx & 15);
        const int64_t rb = idx >> 4;
        const int64_t rt = rb / nbp, b = rb % nbp;
        const int64_t row = rt * 16 + r16;
        if (row < rows && b < nb) scales[row * nb + b] = ts[mk_scale_off(rt, nbp, b, r16)];
    }
}
// one thread per element: W[r,c] = E2M1[code] * 2^(sb-127), bit-exact (-0.0 and subnormals included)
__global__ void dequant_mxfp4_kernel(const uint32_t *__restrict__ tv, const uint8_t *__restrict__ ts,
                                     float *__restrict__ out, int64_t rows, int64_t cols, int64_t nbp) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * cols) return;
    const int64_t row = idx / cols, col = idx % cols;
    const int64_t rt = row >> 4;
    const int r16 = (int)(row & 15), g = r16 & 7, hi = r16 >> 3;
    const int64_t b = col >> 5;
    const int jc = (int)(col & 31), t = jc >> 3, jj = jc & 7;
    const int64_t chunk = rt * (nbp / 2) + (b >> 1);
    const uint32_t w = tv[chunk * 128 + (g * 4 + t) * 4 + (int)(b & 1) * 2 + hi];
    const uint32_t code = (w >> (4 * jj)) & 15u;
    const uint32_t sb = ts[mk_scale_off(rt, nbp, b, r16)];
    out[idx] = c_e2m1[code] * mk_e8m0(sb);
}

// ---- q8_0
// byte offset of element (r16, column j of the block) inside its 512-byte chunk
__device__ __forceinline__ int q8_chunk_off(int r16, int j) {
    const int g = r16 & 7, hi = r16 >> 3, t = j >> 3, jj = j & 7;
    return (g * 4 + t) * 16 + ((jj >> 2) * 2 + hi) * 4 + (jj & 3);
}
template <typename ST> __device__ __forceinline__ ST to_scale(float v);
template <> __device__ __forceinline__ float to_scale<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_scale<__half>(float v) { return __float2half_rn(v); }
__device__ __forceinline__ float from_scale(float v) { return v; }
__device__ __forceinline__ float from_scale(__half v) { return __half2float(v); }

// One warp per (row, block) of the f32 source: q8::quantize_q8_into per row
// (src/q8.rs:49-69).  With half scales the scale is rounded to half FIRST and the
// values are quantized against the rounded scale.
template <typename ST>
__global__ void __launch_bounds__(256)
quantize_weight_q8_kernel(const float *__restrict__ w, int64_t row0, int64_t nrows, int64_t cols, int64_t nb,
                          int64_t nbp, int8_t *__restrict__ tv, ST *__restrict__ ts) {
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wid >= nrows * nb) return;
    const int64_t rl = wid / nb, b = wid % nb;
    const int64_t row = row0 + rl;
    const float v = w[rl * cols + b * 32 + lane];
    float mx = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    const ST st = to_scale<ST>(__fdiv_rn(mx, 127.0f));
    const float dx = from_scale(st);
    int q = 0;
    if (dx != 0.0f) q = (int)fminf(fmaxf(roundf(__fdiv_rn(v, dx)), -127.0f), 127.0f);
    const uint32_t qb = (uint32_t)q & 0xFFu;
    const uint32_t pk = qb | (__shfl_down_sync(0xFFFFFFFFu, qb, 1) << 8) | (__shfl_down_sync(0xFFFFFFFFu, qb, 2) << 16) |
                        (__shfl_down_sync(0xFFFFFFFFu, qb, 3) << 24);
    const int64_t rt = row >> 4;
    const int r16 = (int)(row & 15);
    if ((lane & 3) == 0) *(uint32_t *)(tv + (rt * nbp + b) * 512 + q8_chunk_off(r16, lane)) = pk;
    if (lane == 0) ts[mk_scale_off(rt, nbp, b, r16)] = st;
}
// natural q8 rows -> tiled; one thread per 4 bytes
template <typename ST>
__global__ void retile_q8_kernel(const int8_t *__restrict__ q, const ST *__restrict__ s, int8_t *__restrict__ tv,
                                 ST *__restrict__ ts, int64_t rows, int64_t cols, int64_t nb, int64_t nbp, bool inverse,
                                 int8_t *__restrict__ q_out, ST *__restrict__ s_out) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nquads = rows * (cols / 4);
    if (idx < nquads) {
        const int64_t row = idx / (cols / 4);
        const int64_t c4 = (idx % (cols / 4)) * 4;
        const int64_t b = c4 >> 5;
        const int j = (int)(c4 & 31);
        const int64_t off = ((row >> 4) * nbp + b) * 512 + q8_chunk_off((int)(row & 15), j);
        if (!inverse) *(uint32_t *)(tv + off) = *(const uint32_t *)(q + row * cols + c4);
        else *(uint32_t *)(q_out + row * cols + c4) = *(const uint32_t *)(tv + off);
    }
    if (idx < rows * nb) {
        const int64_t row = idx / nb, b = idx % nb;
        const int64_t off = mk_scale_off(row >> 4, nbp, b, (int)(row & 15));
        if (!inverse) ts[off] = s[idx];
        else s_out[idx] = ts[off];
    }
}

// one thread per element: W[r,c] = e4m3fn(w[r,c]) * 2^(scale[r/128, c/128] - 127), bit-exact (src/dequant.rs:12-41)
__global__ void dequant_fp8_kernel(const uint8_t *__restrict__ w, const uint8_t *__restrict__ scales, float *__restrict__ out,
                                   int64_t rows, int64_t cols) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * cols) return;
    const int64_t r = idx / cols, c = idx % cols;
    const uint32_t b = w[idx];
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    float v;
    if (e == 15u && m == 7u) v = __uint_as_float(0x7FC00000u);                 // the format's NaN
    else if (e == 0u) v = (float)m * 0.001953125f;                             // m / 8 * 2^-6 = m * 2^-9, exact
    else v = __uint_as_float(((e + 120u) << 23) | (m << 20));                  // 2^(e-7) * (1 + m/8)
    if (b & 0x80u) v = -v;
    out[idx] = v * mk_e8m0(scales[(r >> 7) * ((cols + 127) >> 7) + (c >> 7)]);
}

} // namespace

static unsigned grid_for(int64_t n, int block) { return (unsigned)mk_ceil_div(n > 0 ? n : 1, block); }

int32_t mk_launch_retile_mxfp4(mk_ctx *ctx, const uint8_t *packed, const uint8_t *scales, mk_weight *w) {
    const int64_t n = w->nrt * (w->nbp / 2) * 128; // >= nrt*nbp*16
    retile_mxfp4_kernel<<<grid_for(n, 256), 256, 0, ctx->stream>>>(packed, scales, (uint32_t *)w->values,
                                                                  (uint8_t *)w->scales, w->rows, w->cols, w->nrt, w->nb, w->nbp);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}
int32_t mk_launch_untile_mxfp4(mk_ctx *ctx, const mk_weight *w, uint8_t *packed, uint8_t *scales) {
    const int64_t n = w->nrt * (w->nbp / 2) * 128;
    untile_mxfp4_kernel<<<grid_for(n, 256), 256, 0, ctx->stream>>>((const uint32_t *)w->values, (const uint8_t *)w->scales,
                                                                  packed, scales, w->rows, w->cols, w->nrt, w->nb, w->nbp);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}
int32_t mk_launch_dequant_mxfp4(mk_ctx *ctx, const mk_weight *w, float *out) {
    dequant_mxfp4_kernel<<<grid_for(w->rows * w->cols, 256), 256, 0, ctx->stream>>>(
        (const uint32_t *)w->values, (const uint8_t *)w->scales, out, w->rows, w->cols, w->nbp);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}
int32_t mk_launch_quantize_weight_q8(mk_ctx *ctx, const float *wf32, int64_t row0, int64_t nrows, mk_weight *w) {
    const int64_t warps = nrows * w->nb;
    if (w->scale_type == MK_SCALE_F16)
        quantize_weight_q8_kernel<__half><<<grid_for(warps * 32, 256), 256, 0, ctx->stream>>>(
            wf32, row0, nrows, w->cols, w->nb, w->nbp, (int8_t *)w->values, (__half *)w->scales);
    else
        quantize_weight_q8_kernel<float><<<grid_for(warps * 32, 256), 256, 0, ctx->stream>>>(
            wf32, row0, nrows, w->cols, w->nb, w->nbp, (int8_t *)w->values, (float *)w->scales);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}
int32_t mk_launch_retile_q8(mk_ctx *ctx, const int8_t *q, const void *scales, mk_weight *w) {
    const int64_t n = w->rows * (w->cols / 4);
    if (w->scale_type == MK_SCALE_F16)
        retile_q8_kernel<__half><<<grid_for(n, 256), 256, 0, ctx->stream>>>(q, (const __half *)scales, (int8_t *)w->values,
                                                                         (__half *)w->scales, w->rows, w->cols, w->nb,
                                                                         w->nbp, false, nullptr, nullptr);
    else
        retile_q8_kernel<float><<<grid_for(n, 256), 256, 0, ctx->stream>>>(q, (const float *)scales, (int8_t *)w->values,
                                                                        (float *)w->scales, w->rows, w->cols, w->nb, w->nbp,
                                                                        false, nullptr, nullptr);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}
int32_t mk_launch_untile_q8(mk_ctx *ctx, const mk_weight *w, int8_t *q, void *scales) {
    const int64_t n = w->rows * (w->cols / 4);
    if (w->scale_type == MK_SCALE_F16)
        retile_q8_kernel<__half><<<grid_for(n, 256), 256, 0, ctx->stream>>>(nullptr, nullptr, (int8_t *)w->values,
                                                                         (__half *)w->scales, w->rows, w->cols, w->nb,
                                                                         w->nbp, true, q, (__half *)scales);
    else
        retile_q8_kernel<float><<<grid_for(n, 256), 256, 0, ctx->stream>>>(nullptr, nullptr, (int8_t *)w->values,
                                                                        (float *)w->scales, w->rows, w->cols, w->nb, w->nbp,
                                                                        true, q, (float *)scales);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

// e4m3fn weights + ue8m0 scales per 128 x 128 block -> f32, HOST in / HOST out (a check kernel like mk_dequant_mxfp4)
extern "C" int32_t mk_dequant_fp8(mk_ctx *ctx, const uint8_t *w, const uint8_t *scales, int64_t rows, int64_t cols, float *out) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && scales != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(rows > 0 && cols > 0, "rows and cols must be positive");
    MK_CUDA(cudaSetDevice(ctx->device));
    const size_t wb = (size_t)rows * cols, sb = (size_t)mk_ceil_div(rows, 128) * mk_ceil_div(cols, 128), ob = wb * 4;
    int32_t rc = mk_io_reserve(ctx, mk_align_up(wb, 256) + mk_align_up(sb, 256) + mk_align_up(ob, 256));
    if (rc != MK_OK) return rc;
    uint8_t *dw = (uint8_t *)ctx->io_dev, *ds = dw + mk_align_up(wb, 256);
    float *dout = (float *)(ds + mk_align_up(sb, 256));
    MK_CUDA(cudaMemcpyAsync(dw, w, wb, cudaMemcpyHostToDevice, ctx->stream));
    MK_CUDA(cudaMemcpyAsync(ds, scales, sb, cudaMemcpyHostToDevice, ctx->stream));
    dequant_fp8_kernel<<<grid_for((int64_t)wb, 256), 256, 0, ctx->stream>>>(dw, ds, dout, rows, cols);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    MK_CUDA(cudaMemcpyAsync(out, dout, ob, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

// ---------------------------------------------------------------- mxfp4::quantize (src/mxfp4.rs:38-138) on the GPU
// One warp per 32-wide block, lane = element.  Every step keeps the CPU's arithmetic: f32 maximum, the exponent
// e = ceil(log2(maxabs / 6)) clamped to [-127, 128], the three-candidate search by the f64 squared error summed in
// element order (the naive exponent first, replaced only by a strictly smaller error), nearest level by the
// midpoints, the sign taken from the sign bit (so -0.0 keeps code 8).
namespace {
__device__ __forceinline__ float q4_exp2_i(int e) {   // exp2_i (src/mxfp4.rs:10-16): exact bit patterns
    return e >= -126 ? __uint_as_float((uint32_t)(e + 127) << 23) : __uint_as_float(0x00400000u);
}
__device__ __forceinline__ int q4_level(float q) {     // count of the midpoints 0.25 .. 5 that |q| reaches
    const float mag = fabsf(q);
    return (mag >= 0.25f) + (mag >= 0.75f) + (mag >= 1.25f) + (mag >= 1.75f) + (mag >= 2.5f) + (mag >= 3.5f) + (mag >= 5.0f);
}
__device__ __forceinline__ float q4_clamp6(float q) { return q < -6.0f ? -6.0f : (q > 6.0f ? 6.0f : q); }
// group_sse (src/mxfp4.rs:51-69): the warp's 32 terms added in element order by every lane (same result in all)
__device__ __forceinline__ double q4_group_sse(float v, int e) {
    const float inv = __fdiv_rn(1.0f, q4_exp2_i(e));
    const double s = (double)q4_exp2_i(e);
    const float q = q4_clamp6(__fmul_rn(v, inv));
    const double lvl = (double)fabsf(c_e2m1[q4_level(q)]);
    const double dq = __dmul_rn((__float_as_uint(q) >> 31) ? -lvl : lvl, s);
    const double d = __dsub_rn((double)v, dq);
    const double term = __dmul_rn(d, d);
    double sse = 0.0;
#pragma unroll 8
    for (int i = 0; i < 32; ++i) sse = __dadd_rn(sse, __shfl_sync(0xFFFFFFFFu, term, i));
    return sse;
}
__global__ void __launch_bounds__(256)
quantize_mxfp4_kernel(const float *__restrict__ w, int64_t nblocks, int search, uint8_t *__restrict__ packed, uint8_t *__restrict__ scales) {
    const int64_t blk = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (blk >= nblocks) return;
    const float v = w[blk * 32 + lane];
    float maxabs = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) maxabs = fmaxf(maxabs, __shfl_xor_sync(0xFFFFFFFFu, maxabs, o));
    int e = -127;
    if (maxabs != 0.0f) {
        // f32 log2 of the CPU's libm, taken as the correctly rounded value: double log2 rounded once
        const float lg = (float)log2((double)__fdiv_rn(maxabs, 6.0f));
        const float c = ceilf(lg);
        e = c >= 2147483648.0f ? 2147483647 : (c <= -2147483648.0f ? (int)0x80000000 : (int)c);   // `as i32` saturates
        if (c != c) e = 0;
    }
    e = e < -127 ? -127 : (e > 128 ? 128 : e);
    if (search && maxabs != 0.0f) {   // search_mx_scale (src/mxfp4.rs:77-92)
        int best = e;
        double best_sse = q4_group_sse(v, e);
        if (e - 1 >= -127) { const double s1 = q4_group_sse(v, e - 1); if (s1 < best_sse) { best_sse = s1; best = e - 1; } }
        if (e + 1 <= 128) { const double s2 = q4_group_sse(v, e + 1); if (s2 < best_sse) { best_sse = s2; best = e + 1; } }
        e = best;
    }
    int sb = e + 127;
    sb = sb < 0 ? 0 : (sb > 255 ? 255 : sb);
    const float inv = __fdiv_rn(1.0f, q4_exp2_i(e));
    const float q = q4_clamp6(__fmul_rn(v, inv));
    uint32_t idx = (uint32_t)q4_level(q) + ((__float_as_uint(q) >> 31) ? 8u : 0u);
    const uint32_t hi = __shfl_down_sync(0xFFFFFFFFu, idx, 1);
    if ((lane & 1) == 0) packed[blk * 16 + (lane >> 1)] = (uint8_t)(idx | (hi << 4));
    if (lane == 0) scales[blk] = (uint8_t)sb;
}
} // namespace

extern "C" int32_t mk_quantize_mxfp4_dev(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols, int32_t search, uint8_t *packed,
                                         uint8_t *scales) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && packed != nullptr && scales != nullptr, "NULL argument");
    MK_CHECK_ARG(rows > 0 && cols > 0 && cols % 32 == 0, "rows > 0 and cols a positive multiple of 32 required");
    MK_CUDA(cudaSetDevice(ctx->device));
    const int64_t nblocks = rows * (cols / 32);
    quantize_mxfp4_kernel<<<grid_for(nblocks * 32, 256), 256, 0, ctx->stream>>>(w, nblocks, search, packed, scales);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

// ---------------------------------------------------------------- mxfp4::dequant_any (src/mxfp4.rs:228-240)
// A raw blob of either MXFP4 flavour -> f32, HOST in / HOST out: packed || scales for MK_DTYPE_MXFP4, packed || scales ||
// smax (one trailing f32) for MK_DTYPE_MXFP4SQ, whose scale byte decodes as ((q + 1) / 256)^2 * smax (scale_sq, :153-158).
namespace {
__global__ void __launch_bounds__(256) dequant_blob_kernel(const uint8_t *__restrict__ blob, int64_t n, int sq, float *__restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint8_t byte = blob[i >> 1], nib = (i & 1) ? (byte >> 4) : (byte & 0x0F);
    const uint8_t sb = blob[n / 2 + i / 32];
    float sc;
    if (sq) {
        const uint8_t *sp = blob + n / 2 + n / 32;     // the blob is only byte-aligned
        const float smax = __uint_as_float((uint32_t)sp[0] | ((uint32_t)sp[1] << 8) | ((uint32_t)sp[2] << 16) | ((uint32_t)sp[3] << 24));
        const float t = __fmul_rn(__fadd_rn((float)sb, 1.0f), 1.0f / 256.0f);
        sc = __fmul_rn(__fmul_rn(t, t), smax);
    } else {
        sc = mk_e8m0(sb);
    }
    out[i] = __fmul_rn(c_e2m1[nib], sc);
}
} // namespace
extern "C" int32_t mk_dequant_mxfp4_blob(mk_ctx *ctx, int32_t dtype, const uint8_t *blob, int64_t rows, int64_t cols, float *out) {
    MK_CHECK_ARG(ctx != nullptr && blob != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(dtype == MK_DTYPE_MXFP4 || dtype == MK_DTYPE_MXFP4SQ, "dtype is not an MXFP4 flavour");
    MK_CHECK_ARG(rows > 0 && cols > 0 && cols % 32 == 0, "rows > 0 and cols a positive multiple of 32 required");
    MK_CUDA(cudaSetDevice(ctx->device));
    const int64_t n = rows * cols;
    const size_t bb = (size_t)(n / 2 + n / 32 + (dtype == MK_DTYPE_MXFP4SQ ? 4 : 0)), ob = (size_t)n * 4;
    int32_t rc = mk_io_reserve(ctx, mk_align_up(bb, 256) + ob);
    if (rc != MK_OK) return rc;
    uint8_t *db = (uint8_t *)ctx->io_dev;
    float *dout = (float *)(db + mk_align_up(bb, 256));
    MK_CUDA(cudaMemcpyAsync(db, blob, bb, cudaMemcpyHostToDevice, ctx->stream));
    dequant_blob_kernel<<<grid_for(n, 256), 256, 0, ctx->stream>>>(db, n, dtype == MK_DTYPE_MXFP4SQ ? 1 : 0, dout);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    MK_CUDA(cudaMemcpyAsync(out, dout, ob, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}
