// VQ1 codebook matvec by lookup table (sm_100a).
//
// Reference: quant::matvec_vq / matvec_vq_gather (src/quant.rs:313-346) and
// lutgemv::matvec_vq_lut (src/lutgemv.rs:208-238).  W[r, 16 v + j] = codebook[idx[r][v]][j]
// with a 256 x 16 f32 codebook and one index byte per 16 weights.  The products that can
// occur are formed once per activation group, lut[v][k] = dot(codebook[k], x[16 v ..]) with
// ascending j, a separate multiply and add, starting from 0; a row is then the sum of its
// table entries in ascending group order.  That is the engine's order, so the result is
// bit-identical to both of its paths (src/lutgemv.rs:22-27).
//
// Two launches per call: the table (cols / 16 x 256 floats, built once for all rows: it is
// 30 times the work of the sweep at 7168 x 2048) and the sweep: one thread per (row, token),
// index bytes staged through shared memory in coalesced tiles, the table read through L1.
#include "mk_common.cuh"

#include <new>

namespace {
constexpr int VQ_DIM = 16, VQ_K = 256;

// grid (groups, batch); thread k: lut[b][v][k] = dot(codebook[k], x[b][16 v ..])
__global__ void __launch_bounds__(VQ_K) vq_lut_kernel(const float *__restrict__ codebook, const float *__restrict__ x, int64_t cols,
                                                     float *__restrict__ lut) {
    const int v = blockIdx.x, b = blockIdx.y, k = threadIdx.x;
    const int64_t vpr = cols / VQ_DIM;
    __shared__ float xs[VQ_DIM];
    if (k < VQ_DIM) xs[k] = x[(int64_t)b * cols + (int64_t)v * VQ_DIM + k];
    __syncthreads();
    const float4 *cb = (const float4 *)(codebook + (size_t)k * VQ_DIM);
    float s = 0.0f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 c = __ldg(cb + q);
        s = __fadd_rn(s, __fmul_rn(c.x, xs[4 * q + 0]));
        s = __fadd_rn(s, __fmul_rn(c.y, xs[4 * q + 1]));
        s = __fadd_rn(s, __fmul_rn(c.z, xs[4 * q + 2]));
        s = __fadd_rn(s, __fmul_rn(c.w, xs[4 * q + 3]));
    }
    lut[((int64_t)b * vpr + v) * VQ_K + k] = s;
}

// CTA = 128 rows; index bytes in tiles of 64 groups; thread = row, loop over tokens inside
constexpr int SW_ROWS = 128, SW_TILE = 64, SW_LD = SW_TILE + 4; // +4: rows 17 words apart, conflict-free byte reads
__global__ void __launch_bounds__(SW_ROWS) vq_sweep_kernel(const uint8_t *__restrict__ indices, const float *__restrict__ lut, int64_t rows,
                                                          int64_t vpr, int batch, float *__restrict__ y) {
    __shared__ uint8_t tile[SW_ROWS * SW_LD];
    const int tid = threadIdx.x;
    const int64_t row0 = (int64_t)blockIdx.x * SW_ROWS, row = row0 + tid;
    float acc[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[b] = 0.0f;
    for (int64_t g0 = 0; g0 < vpr; g0 += SW_TILE) {
        const int groups = (int)min((int64_t)SW_TILE, vpr - g0);
        __syncthreads();
        // coalesced: consecutive threads take consecutive bytes of a row's tile
        for (int i = tid; i < SW_ROWS * SW_TILE; i += SW_ROWS) {
            const int r = i / SW_TILE, g = i % SW_TILE;
            if (row0 + r < rows && g < groups) tile[r * SW_LD + g] = indices[(row0 + r) * vpr + g0 + g];
        }
        __syncthreads();
        if (row < rows) {
            for (int g = 0; g < groups; ++g) {
                const int code = tile[tid * SW_LD + g];
#pragma unroll
                for (int b = 0; b < 8; ++b)
                    if (b < batch) acc[b] = __fadd_rn(acc[b], __ldg(lut + ((int64_t)b * vpr + g0 + g) * VQ_K + code));
            }
        }
    }
    if (row < rows)
        for (int b = 0; b < batch; ++b) y[(int64_t)b * rows + row] = acc[b];
}
} // namespace

// y [batch][rows]; lut scratch [batch][cols/16][256] floats; batch <= 8 per pass
static int32_t vq_launch(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int batch, float *lut) {
    mk_prof_scope prof(ctx, MK_PROF_OTHER);
    const int64_t vpr = w->cols / VQ_DIM;
    vq_lut_kernel<<<dim3((unsigned)vpr, (unsigned)batch), VQ_K, 0, ctx->stream>>>((const float *)w->scales, x, w->cols, lut);
    vq_sweep_kernel<<<(unsigned)mk_ceil_div(w->rows, SW_ROWS), SW_ROWS, 0, ctx->stream>>>((const uint8_t *)w->values, lut, w->rows, vpr,
                                                                                         batch, y);
    ctx->launches += 2;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

extern "C" int32_t mk_weight_vq1(mk_ctx *ctx, const float *codebook, const uint8_t *indices, int64_t rows, int64_t cols,
                                 int32_t src_on_device, mk_weight **out) {
    MK_CHECK_ARG(ctx != nullptr && codebook != nullptr && indices != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(rows > 0 && cols > 0 && cols % VQ_DIM == 0, "rows > 0 and cols a positive multiple of 16 required");
    *out = nullptr;
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_weight *h = new (std::nothrow) mk_weight();
    if (!h) return MK_ERR_OOM;
    memset(h, 0, sizeof(*h));
    h->fmt = MK_FMT_VQ1;
    h->rows = rows;
    h->cols = cols;
    h->values_bytes = (size_t)rows * (cols / VQ_DIM);
    h->scales_bytes = (size_t)VQ_K * VQ_DIM * 4; // the codebook
    const cudaMemcpyKind kind = src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    cudaError_t e = cudaMalloc(&h->values, h->values_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&h->scales, h->scales_bytes);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h->values, indices, h->values_bytes, kind, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h->scales, codebook, h->scales_bytes, kind, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        mk_set_error("mk_weight_vq1: %s", cudaGetErrorString(e));
        if (h->values) cudaFree(h->values);
        if (h->scales) cudaFree(h->scales);
        delete h;
        return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    *out = h;
    return MK_OK;
}

static int32_t vq_check(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && x != nullptr && y != nullptr, "NULL argument");
    MK_CHECK_ARG(w->fmt == MK_FMT_VQ1, "weight handle has the wrong format for this call");
    MK_CHECK_ARG(batch >= 1 && batch <= 4096, "batch must be in [1, 4096]");
    MK_CUDA(cudaSetDevice(ctx->device));
    return MK_OK;
}

extern "C" int32_t mk_matvec_vq1_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch) {
    int32_t rc = vq_check(ctx, w, x, y, batch);
    if (rc != MK_OK) return rc;
    const int per_pass = batch < 8 ? batch : 8;
    rc = mk_ws_reserve(ctx, (size_t)per_pass * (w->cols / VQ_DIM) * VQ_K * 4);
    if (rc != MK_OK) return rc;
    for (int t0 = 0; t0 < batch; t0 += 8) {
        const int nt = batch - t0 < 8 ? batch - t0 : 8;
        rc = vq_launch(ctx, w, x + (int64_t)t0 * w->cols, y + (int64_t)t0 * w->rows, nt, (float *)ctx->ws);
        if (rc != MK_OK) return rc;
    }
    return MK_OK;
}

extern "C" int32_t mk_matvec_vq1(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch) {
    int32_t rc = vq_check(ctx, w, x, y, batch);
    if (rc != MK_OK) return rc;
    const size_t xb = (size_t)batch * w->cols * 4, yb = (size_t)batch * w->rows * 4;
    rc = mk_io_reserve(ctx, mk_align_up(xb, 256) + mk_align_up(yb, 256));
    if (rc != MK_OK) return rc;
    float *dx = (float *)ctx->io_dev;
    float *dy = (float *)((char *)ctx->io_dev + mk_align_up(xb, 256));
    MK_CUDA(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = mk_matvec_vq1_dev(ctx, w, dx, dy, batch);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(y, dy, yb, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}
