// f32 pieces of the decode path (sm_100a): the f32 matvec, rmsnorm and SiTU.
//
// Reference: matvec / matvec_cpu (src/model.rs:199-247; the Metal seam is
// gpu_matvec, src/metal.rs:750), rmsnorm (src/model.rs:599-605) and situ
// (src/model.rs:617-621).  The matvec and the rmsnorm reproduce the engine's dot()
// order (src/model.rs:63-82) and therefore its bits; SiTU evaluates tanh and exp in
// double precision and rounds once.
#include "f32gemv.cuh"

namespace {

// y[tok * ldy + row] (+)= dot(w[row], x[tok]); accumulate: y = y + dot (one add, as `out[j] += s[j]`)
template <class S>
__global__ void __launch_bounds__(256)
f32_gemv_tile_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ y, int rows, int d, int n,
                     int64_t ldy, int accumulate) {
    extern __shared__ __align__(16) float smem[];
    int row, tok;
    bool valid;
    const float v = mkf::tile_dot<S>(w, x, rows, d, n, blockIdx.x * S::NE, blockIdx.y * S::NT, smem, &row, &tok, &valid);
    if (valid) {
        float *o = y + (int64_t)tok * ldy + row;
        *o = accumulate ? __fadd_rn(*o, v) : v;
    }
}

// many tokens (a prompt's rows): 16 matrix rows x 16 tokens per CTA, every pair the engine's dot() (mkf::reg_tile_product)
__global__ void __launch_bounds__(mkf::RG_THREADS)
f32_gemm_reg_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ y, int rows, int d, int n, int64_t ldy,
                    int accumulate) {
    extern __shared__ __align__(16) float gsm[];
    mkf::reg_tile_product(w, x, rows, d, n, blockIdx.x * mkf::RG_TE, blockIdx.y * mkf::RG_TT, gsm, [&](int row, int tok, float v) {
        float *o = y + (int64_t)tok * ldy + row;
        *o = accumulate ? __fadd_rn(*o, v) : v;
    });
}

template <int T>
__global__ void __launch_bounds__(256)
f32_gemv_rows_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ y, int rows, int d, int n,
                     int64_t ldy, int accumulate) {
    const int warp_g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31, sub = lane >> 3, j = lane & 7;
    const int rwarps = (rows + 3) / 4;
    const int tok0 = (warp_g / rwarps) * T;
    const int row = (warp_g % rwarps) * 4 + sub;
    if (tok0 >= n) return;
    const bool rv = row < rows;
    float out[T];
    mkf::rows_dot<T>(w + (size_t)(rv ? row : 0) * d, x, d, n, tok0, rv, lane, out);
#pragma unroll
    for (int t = 0; t < T; ++t)
        if (j == 0 && rv && tok0 + t < n) {
            float *o = y + (int64_t)(tok0 + t) * ldy + row;
            *o = accumulate ? __fadd_rn(*o, out[t]) : out[t];
        }
}

// one warp per row: ss = dot(x, x) / len; inv = 1 / sqrt(ss + eps); out = (x * inv) * w
__global__ void __launch_bounds__(128) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ w, int n, int len, float eps,
                                                      float *__restrict__ out) {
    const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31, j = lane & 7;
    if (row >= n) return;
    const float *xr = x + (size_t)row * len;
    const int full = len & ~7;
    float acc = 0.0f;
    for (int c = 0; c < full; c += 8) {
        const float v = xr[c + j];
        acc = __fadd_rn(acc, __fmul_rn(v, v));
    }
    float ss = mkf::reduce8(acc, lane); // all four octets compute the same value
    for (int c = full; c < len; ++c) ss = __fadd_rn(ss, __fmul_rn(xr[c], xr[c]));
    ss = __fdiv_rn(ss, (float)len);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ss, eps)));
    for (int c = lane; c < len; c += 32) out[(size_t)row * len + c] = __fmul_rn(__fmul_rn(xr[c], inv), w[c]);
}

__global__ void __launch_bounds__(256) situ_kernel(const float *__restrict__ a, const float *__restrict__ u, int64_t count,
                                                   float *__restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = mk_situ(a[i], u[i]);
}

// a[i] *= sigmoid(g[i]) (the output gate of mla_forward, src/model.rs:2017-2019); exp in double precision, rounded once
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(float *__restrict__ a, const float *__restrict__ g, int64_t count) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) a[i] = __fmul_rn(a[i], __fdiv_rn(1.0f, __fadd_rn(1.0f, (float)exp((double)(-g[i])))));
}

using GemvB1 = mkf::TileShape<32, 1, 128, 4>;
using GemvB2 = mkf::TileShape<16, 2, 128, 4>;
using GemvB4 = mkf::TileShape<8, 4, 256, 3>;
using GemvB8 = mkf::TileShape<4, 8, 256, 3>;
using GemvB16 = mkf::TileShape<2, 16, 256, 3>;

template <class S>
int32_t launch_tile(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols, const float *x, int n, float *y, int64_t ldy, int accumulate) {
    static mk_once_per_device attr; // one per instantiation
    if (attr.pending(ctx->device)) {
        MK_CUDA(cudaFuncSetAttribute(f32_gemv_tile_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)S::SMEM));
        attr.mark(ctx->device);
    }
    const dim3 grid((unsigned)mk_ceil_div(rows, S::NE), (unsigned)mk_ceil_div(n, S::NT));
    f32_gemv_tile_kernel<S><<<grid, 256, S::SMEM, ctx->stream>>>(w, x, y, (int)rows, (int)cols, n, ldy, accumulate);
    return MK_OK;
}

} // namespace

int32_t mk_launch_f32_gemv(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols, const float *x, int n, float *y, int64_t ldy,
                           int accumulate) {
    MK_CHECK_ARG(rows > 0 && cols > 0 && rows < (1ll << 31) && cols < (1ll << 31) && n > 0, "f32 matvec: bad shape");
    mk_prof_scope prof(ctx, MK_PROF_OTHER);
    if (cols % 4 == 0 && (((uintptr_t)w | (uintptr_t)x) & 15) == 0) {
        int32_t rc;
        if (n == 1) rc = launch_tile<GemvB1>(ctx, w, rows, cols, x, n, y, ldy, accumulate);
        else if (n == 2) rc = launch_tile<GemvB2>(ctx, w, rows, cols, x, n, y, ldy, accumulate);
        else if (n <= 4) rc = launch_tile<GemvB4>(ctx, w, rows, cols, x, n, y, ldy, accumulate);
        else if (n <= 8) rc = launch_tile<GemvB8>(ctx, w, rows, cols, x, n, y, ldy, accumulate);
        else if (n >= 48) {
            static mk_once_per_device attr;
            if (attr.pending(ctx->device)) {
                MK_CUDA(cudaFuncSetAttribute(f32_gemm_reg_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mkf::RG_SMEM));
                attr.mark(ctx->device);
            }
            f32_gemm_reg_kernel<<<dim3((unsigned)mk_ceil_div(rows, mkf::RG_TE), (unsigned)mk_ceil_div(n, mkf::RG_TT)), mkf::RG_THREADS, mkf::RG_SMEM,
                                  ctx->stream>>>(w, x, y, (int)rows, (int)cols, n, ldy, accumulate);
            rc = MK_OK;
        } else rc = launch_tile<GemvB16>(ctx, w, rows, cols, x, n, y, ldy, accumulate);
        if (rc != MK_OK) return rc;
    } else if (n >= 4) {
        const int64_t warps = mk_ceil_div(rows, 4) * mk_ceil_div(n, 4);
        f32_gemv_rows_kernel<4><<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(w, x, y, (int)rows, (int)cols, n, ldy, accumulate);
    } else {
        const int64_t warps = mk_ceil_div(rows, 4) * n;
        f32_gemv_rows_kernel<1><<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(w, x, y, (int)rows, (int)cols, n, ldy, accumulate);
    }
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

int32_t mk_launch_rmsnorm(mk_ctx *ctx, const float *x, const float *w, int n, int len, float eps, float *out) {
    mk_prof_scope prof(ctx, MK_PROF_OTHER);
    rmsnorm_kernel<<<(unsigned)mk_ceil_div((int64_t)n * 32, 128), 128, 0, ctx->stream>>>(x, w, n, len, eps, out);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

int32_t mk_launch_situ(mk_ctx *ctx, const float *a, const float *u, int64_t count, float *out) {
    mk_prof_scope prof(ctx, MK_PROF_OTHER);
    situ_kernel<<<(unsigned)mk_ceil_div(count, 256), 256, 0, ctx->stream>>>(a, u, count, out);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

// ====================================================================== C ABI
#include <new>

extern "C" int32_t mk_weight_f32(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols, int32_t src_on_device, mk_weight **out) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(rows > 0 && cols > 0 && rows < (1ll << 31) && cols < (1ll << 31), "rows and cols must be in [1, 2^31)");
    *out = nullptr;
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_weight *h = new (std::nothrow) mk_weight();
    if (!h) return MK_ERR_OOM;
    memset(h, 0, sizeof(*h));
    h->fmt = MK_FMT_F32;
    h->rows = rows;
    h->cols = cols;
    h->values_bytes = (size_t)rows * cols * 4;
    cudaError_t e = cudaMalloc(&h->values, h->values_bytes);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(h->values, w, h->values_bytes, src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        mk_set_error("mk_weight_f32: %s (%zu bytes)", cudaGetErrorString(e), h->values_bytes);
        if (h->values) cudaFree(h->values);
        delete h;
        return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    *out = h;
    return MK_OK;
}

static int32_t f32_check(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && x != nullptr && y != nullptr, "NULL argument");
    MK_CHECK_ARG(w->fmt == MK_FMT_F32, "weight handle has the wrong format for this call");
    MK_CHECK_ARG(batch >= 1 && batch <= 4096, "batch must be in [1, 4096]");
    MK_CUDA(cudaSetDevice(ctx->device));
    return MK_OK;
}

extern "C" int32_t mk_matvec_f32_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch) {
    int32_t rc = f32_check(ctx, w, x, y, batch);
    if (rc != MK_OK) return rc;
    return mk_launch_f32_gemv(ctx, (const float *)w->values, w->rows, w->cols, x, batch, y, w->rows, 0);
}

extern "C" int32_t mk_matvec_f32(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch) {
    int32_t rc = f32_check(ctx, w, x, y, batch);
    if (rc != MK_OK) return rc;
    const size_t xb = (size_t)batch * w->cols * 4, yb = (size_t)batch * w->rows * 4;
    rc = mk_io_reserve(ctx, mk_align_up(xb, 256) + mk_align_up(yb, 256));
    if (rc != MK_OK) return rc;
    float *dx = (float *)ctx->io_dev;
    float *dy = (float *)((char *)ctx->io_dev + mk_align_up(xb, 256));
    MK_CUDA(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = mk_launch_f32_gemv(ctx, (const float *)w->values, w->rows, w->cols, dx, batch, dy, w->rows, 0);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(y, dy, yb, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_rmsnorm_dev(mk_ctx *ctx, const float *x, const float *w, int32_t n, int32_t len, float eps, float *out) {
    MK_CHECK_ARG(ctx != nullptr && x != nullptr && w != nullptr && out != nullptr && n > 0 && len > 0, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    return mk_launch_rmsnorm(ctx, x, w, n, len, eps, out);
}

extern "C" int32_t mk_sigmoid_gate_dev(mk_ctx *ctx, float *a, const float *g, int64_t count) {
    MK_CHECK_ARG(ctx != nullptr && a != nullptr && g != nullptr && count > 0, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_prof_scope prof(ctx, MK_PROF_OTHER);
    sigmoid_gate_kernel<<<(unsigned)mk_ceil_div(count, 256), 256, 0, ctx->stream>>>(a, g, count);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}
