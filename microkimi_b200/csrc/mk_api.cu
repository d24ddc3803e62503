// C-ABI entry points of libmk_b200 (see include/mk_cuda.h): context, weight
// registration, activation staging and the matvec calls.  Host-pointer variants
// stage through a pinned buffer and synchronize; `_dev` variants only enqueue.
#include <stdarg.h>

#include <new>

#include "mk_common.cuh"

// ---------------------------------------------------------------- errors
static thread_local char g_err[512] = "";

void mk_set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
extern "C" const char *mk_last_error(void) { return g_err; }

// ---------------------------------------------------------------- context
extern "C" int32_t mk_init(int32_t device, mk_ctx **out) {
    MK_CHECK_ARG(out != nullptr, "out is NULL");
    *out = nullptr;
    int n = 0;
    MK_CUDA(cudaGetDeviceCount(&n));
    MK_CHECK_ARG(device >= 0 && device < n, "no such CUDA device");
    cudaDeviceProp p;
    MK_CUDA(cudaGetDeviceProperties(&p, device));
    if (p.major != 10) {
        mk_set_error("mk_init: device %d is sm_%d%d; this library is built for sm_100a only", device, p.major, p.minor);
        return MK_ERR_UNSUPPORTED;
    }
    MK_CUDA(cudaSetDevice(device));
    mk_ctx *c = new (std::nothrow) mk_ctx();
    if (!c) return MK_ERR_OOM;
    memset(c, 0, sizeof(*c));
    c->device = device;
    c->pdl = 1;
    c->sm_count = p.multiProcessorCount;
    c->cc_major = p.major;
    c->cc_minor = p.minor;
    c->mem_bytes = p.totalGlobalMem;
    cudaError_t e = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&c->status_dev, sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemset(c->status_dev, 0, sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMalloc(&c->zeros_dev, 256);
    if (e == cudaSuccess) e = cudaMemset(c->zeros_dev, 0, 256);
    if (e == cudaSuccess) e = cudaMalloc(&c->argmax_count, 64 * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(c->argmax_count, 0, 64 * sizeof(unsigned));
    if (e != cudaSuccess) {
        mk_set_error("mk_init: %s", cudaGetErrorString(e));
        delete c;
        return MK_ERR_CUDA;
    }
    c->stream = c->own_stream;
    *out = c;
    return MK_OK;
}

extern "C" int32_t mk_shutdown(mk_ctx *ctx) {
    MK_CHECK_ARG(ctx != nullptr, "ctx is NULL");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->io_dev) cudaFree(ctx->io_dev);
    if (ctx->io_pinned) cudaFreeHost(ctx->io_pinned);
    if (ctx->status_dev) cudaFree(ctx->status_dev);
    if (ctx->zeros_dev) cudaFree(ctx->zeros_dev);
    if (ctx->argmax_count) cudaFree(ctx->argmax_count);
    if (ctx->prof_pairs) {
        for (int i = 0; i < ctx->prof_cap; ++i) {
            cudaEventDestroy(ctx->prof_pairs[i].a);
            cudaEventDestroy(ctx->prof_pairs[i].b);
        }
        delete[] ctx->prof_pairs;
    }
    if (ctx->side_ready) {
        for (int i = 0; i < 2; ++i) cudaStreamDestroy(ctx->side[i]);
        for (int i = 0; i < 4; ++i) cudaEventDestroy(ctx->side_ev[i]);
    }
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    delete ctx;
    return MK_OK;
}

static int32_t side_init(mk_ctx *ctx) {
    if (ctx->side_ready) return MK_OK;
    MK_CUDA(cudaSetDevice(ctx->device));
    for (int i = 0; i < 2; ++i) MK_CUDA(cudaStreamCreateWithFlags(&ctx->side[i], cudaStreamNonBlocking));
    for (int i = 0; i < 4; ++i) MK_CUDA(cudaEventCreateWithFlags(&ctx->side_ev[i], cudaEventDisableTiming));
    ctx->side_ready = 1;
    return MK_OK;
}
int32_t mk_fork(mk_ctx *ctx, int i) {
    int32_t rc = side_init(ctx);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaEventRecord(ctx->side_ev[i], ctx->stream));
    MK_CUDA(cudaStreamWaitEvent(ctx->side[i], ctx->side_ev[i], 0));
    return MK_OK;
}
int32_t mk_join(mk_ctx *ctx, int i) {
    MK_CUDA(cudaEventRecord(ctx->side_ev[2 + i], ctx->side[i]));
    MK_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->side_ev[2 + i], 0));
    return MK_OK;
}

extern "C" int32_t mk_set_stream(mk_ctx *ctx, void *cuda_stream) {
    MK_CHECK_ARG(ctx != nullptr, "ctx is NULL");
    ctx->stream = (cudaStream_t)cuda_stream;
    return MK_OK;
}
extern "C" int32_t mk_memcpy_dev(mk_ctx *ctx, void *dst, const void *src, uint64_t bytes) {
    MK_CHECK_ARG(ctx != nullptr && dst != nullptr && src != nullptr, "NULL argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    MK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return MK_OK;
}
extern "C" int32_t mk_sync(mk_ctx *ctx) {
    MK_CHECK_ARG(ctx != nullptr, "ctx is NULL");
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}
extern "C" int64_t mk_launch_count(mk_ctx *ctx) { return ctx ? ctx->launches : -1; }
extern "C" int32_t mk_device_info(mk_ctx *ctx, int32_t *sm_count, int32_t *cc_major, int32_t *cc_minor, uint64_t *mem_bytes) {
    MK_CHECK_ARG(ctx != nullptr, "ctx is NULL");
    if (sm_count) *sm_count = ctx->sm_count;
    if (cc_major) *cc_major = ctx->cc_major;
    if (cc_minor) *cc_minor = ctx->cc_minor;
    if (mem_bytes) *mem_bytes = ctx->mem_bytes;
    return MK_OK;
}
extern "C" int32_t mk_status_word(mk_ctx *ctx, int32_t *out) {
    MK_CHECK_ARG(ctx != nullptr && out != nullptr, "NULL argument");
    MK_CUDA(cudaMemcpyAsync(out, ctx->status_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaMemsetAsync(ctx->status_dev, 0, sizeof(int32_t), ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_set_option(mk_ctx *ctx, const char *name, int64_t value) {
    MK_CHECK_ARG(ctx != nullptr && name != nullptr, "NULL argument");
    if (strcmp(name, "force_ks") == 0) {
        MK_CHECK_ARG(value == 0 || value == 1 || value == 2 || value == 4 || value == 8, "force_ks must be 0, 1, 2, 4 or 8");
        ctx->force_ks = (int)value;
        return MK_OK;
    }
    if (strcmp(name, "pdl") == 0) {
        ctx->pdl = value != 0;
        return MK_OK;
    }
    if (strcmp(name, "moe_no_fuse") == 0) {
        ctx->moe_no_fuse = value != 0;
        return MK_OK;
    }
    if (strcmp(name, "mla_max_split") == 0) {
        MK_CHECK_ARG(value >= 0 && value <= 256, "mla_max_split must be in [0, 256]");
        ctx->mla_max_split = (int)value;
        return MK_OK;
    }
    if (strcmp(name, "kda_smem") == 0) {
        ctx->kda_smem = value != 0;
        return MK_OK;
    }
    if (strcmp(name, "mla_no_t5") == 0) {
        ctx->mla_no_t5 = value != 0;
        return MK_OK;
    }
    if (strcmp(name, "mla_strict") == 0) {
        ctx->mla_strict = value != 0;
        return MK_OK;
    }
    if (strcmp(name, "mla_no_tc") == 0) {
        ctx->mla_no_tc = value != 0;
        return MK_OK;
    }
    mk_set_error("mk_set_option: unknown option '%s'", name);
    return MK_ERR_ARG;
}

// ---------------------------------------------------------------- profiling
mk_prof_scope::mk_prof_scope(mk_ctx *c, int cat) : ctx(c), p(nullptr) {
    if (!c->prof_on) return;
    if (c->prof_used == c->prof_cap && mk_prof_drain(c) != MK_OK) return;
    p = &c->prof_pairs[c->prof_used++];
    p->cat = cat;
    cudaEventRecord(p->a, c->stream);
}
mk_prof_scope::~mk_prof_scope() {
    if (p) cudaEventRecord(p->b, ctx->stream);
}
int32_t mk_prof_drain(mk_ctx *ctx) {
    if (ctx->prof_used == 0) return MK_OK;
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < ctx->prof_used; ++i) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, ctx->prof_pairs[i].a, ctx->prof_pairs[i].b) == cudaSuccess) {
            ctx->prof_count[ctx->prof_pairs[i].cat]++;
            ctx->prof_ms[ctx->prof_pairs[i].cat] += ms;
        }
    }
    ctx->prof_used = 0;
    return MK_OK;
}
extern "C" int32_t mk_prof_enable(mk_ctx *ctx, int32_t on) {
    MK_CHECK_ARG(ctx != nullptr, "ctx is NULL");
    MK_CUDA(cudaSetDevice(ctx->device));
    if (on && !ctx->prof_pairs) {
        ctx->prof_cap = 1024;
        ctx->prof_pairs = new (std::nothrow) mk_prof_pair[ctx->prof_cap];
        if (!ctx->prof_pairs) return MK_ERR_OOM;
        for (int i = 0; i < ctx->prof_cap; ++i) {
            MK_CUDA(cudaEventCreate(&ctx->prof_pairs[i].a));
            MK_CUDA(cudaEventCreate(&ctx->prof_pairs[i].b));
        }
    }
    if (on) {
        int32_t rc = mk_prof_drain(ctx);
        if (rc != MK_OK) return rc;
        for (int i = 0; i < MK_PROF_NCAT; ++i) { ctx->prof_count[i] = 0; ctx->prof_ms[i] = 0.0; }
    }
    ctx->prof_on = on ? 1 : 0;
    return MK_OK;
}
extern "C" int32_t mk_prof_read(mk_ctx *ctx, int32_t category, int64_t *launches, double *total_ms) {
    MK_CHECK_ARG(ctx != nullptr, "ctx is NULL");
    MK_CHECK_ARG(category >= 0 && category < MK_PROF_NCAT, "bad category");
    int32_t rc = mk_prof_drain(ctx);
    if (rc != MK_OK) return rc;
    if (launches) *launches = ctx->prof_count[category];
    if (total_ms) *total_ms = ctx->prof_ms[category];
    return MK_OK;
}

static int32_t grow(void **p, size_t *have, size_t want, bool pinned, cudaStream_t st) {
    if (*have >= want) return MK_OK;
    MK_CUDA(cudaStreamSynchronize(st));
    if (*p) {
        if (pinned) cudaFreeHost(*p); else cudaFree(*p);
        *p = nullptr;
        *have = 0;
    }
    want = mk_align_up(want + want / 4, 1 << 16);
    if (pinned) MK_CUDA(cudaMallocHost(p, want));
    else MK_CUDA(cudaMalloc(p, want));
    *have = want;
    return MK_OK;
}
int32_t mk_ws_reserve(mk_ctx *ctx, size_t bytes) { return grow(&ctx->ws, &ctx->ws_bytes, bytes, false, ctx->stream); }
int32_t mk_io_reserve(mk_ctx *ctx, size_t bytes) { return grow(&ctx->io_dev, &ctx->io_bytes, bytes, false, ctx->stream); }
int32_t mk_pinned_reserve(mk_ctx *ctx, size_t bytes) {
    return grow(&ctx->io_pinned, &ctx->io_pinned_bytes, bytes, true, ctx->stream);
}

// ---------------------------------------------------------------- weights
static int32_t weight_alloc(mk_ctx *ctx, int fmt, int scale_type, int64_t rows, int64_t cols, mk_weight **out) {
    MK_CHECK_ARG(ctx != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(rows > 0 && cols > 0 && cols % 32 == 0, "rows > 0 and cols a positive multiple of 32 required");
    *out = nullptr;
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_weight *w = new (std::nothrow) mk_weight();
    if (!w) return MK_ERR_OOM;
    memset(w, 0, sizeof(*w));
    w->fmt = fmt;
    w->scale_type = scale_type;
    w->rows = rows;
    w->cols = cols;
    w->nrt = mk_ceil_div(rows, 16);
    w->nb = cols / 32;
    w->nbp = mk_ceil_div(w->nb, 4) * 4;
    if (fmt == MK_FMT_MXFP4) {
        w->values_bytes = (size_t)w->nrt * (w->nbp / 2) * 512;
        w->scales_bytes = (size_t)w->nrt * w->nbp * 16;
    } else {
        w->values_bytes = (size_t)w->nrt * w->nbp * 512;
        w->scales_bytes = (size_t)w->nrt * w->nbp * 16 * (scale_type == MK_SCALE_F16 ? 2 : 4);
    }
    cudaError_t e = cudaMalloc(&w->values, w->values_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&w->scales, w->scales_bytes);
    if (e == cudaSuccess) e = cudaMemsetAsync(w->values, 0, w->values_bytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(w->scales, 0, w->scales_bytes, ctx->stream);
    if (e != cudaSuccess) {
        mk_set_error("weight_alloc: %s (%zu + %zu bytes)", cudaGetErrorString(e), w->values_bytes, w->scales_bytes);
        if (w->values) cudaFree(w->values);
        if (w->scales) cudaFree(w->scales);
        delete w;
        return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    *out = w;
    return MK_OK;
}

extern "C" int32_t mk_weight_free(mk_ctx *ctx, mk_weight *w) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr, "NULL argument");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (w->values) cudaFree(w->values);
    if (w->scales) cudaFree(w->scales);
    delete w;
    return MK_OK;
}
extern "C" int64_t mk_weight_bytes(const mk_weight *w) { return w ? (int64_t)(w->values_bytes + w->scales_bytes) : -1; }

// temporary device copy of a host blob (registration only)
struct TmpDev {
    void *p = nullptr;
    ~TmpDev() { if (p) cudaFree(p); }
};

extern "C" int32_t mk_weight_mxfp4(mk_ctx *ctx, const uint8_t *packed, const uint8_t *scales, int64_t rows, int64_t cols,
                                   int32_t src_on_device, mk_weight **out) {
    MK_CHECK_ARG(packed != nullptr && scales != nullptr, "NULL blob");
    mk_weight *w = nullptr;
    int32_t rc = weight_alloc(ctx, MK_FMT_MXFP4, 0, rows, cols, &w);
    if (rc != MK_OK) return rc;
    const size_t pb = (size_t)rows * cols / 2, sb = (size_t)rows * cols / 32;
    TmpDev tp, ts;
    const uint8_t *dp = packed, *ds = scales;
    cudaError_t e = cudaSuccess;
    if (!src_on_device) {
        e = cudaMalloc(&tp.p, pb);
        if (e == cudaSuccess) e = cudaMalloc(&ts.p, sb);
        if (e == cudaSuccess) e = cudaMemcpyAsync(tp.p, packed, pb, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(ts.p, scales, sb, cudaMemcpyHostToDevice, ctx->stream);
        dp = (const uint8_t *)tp.p;
        ds = (const uint8_t *)ts.p;
    }
    if (e == cudaSuccess) {
        rc = mk_launch_retile_mxfp4(ctx, dp, ds, w);
        if (rc == MK_OK) e = cudaStreamSynchronize(ctx->stream);
    }
    if (e != cudaSuccess || rc != MK_OK) {
        if (e != cudaSuccess) mk_set_error("mk_weight_mxfp4: %s", cudaGetErrorString(e));
        mk_weight_free(ctx, w);
        return rc != MK_OK ? rc : (e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA);
    }
    *out = w;
    return MK_OK;
}

extern "C" int32_t mk_weight_q8_from_f32(mk_ctx *ctx, const float *wsrc, int64_t rows, int64_t cols, int32_t scale_type,
                                         int32_t src_on_device, mk_weight **out) {
    MK_CHECK_ARG(wsrc != nullptr, "NULL matrix");
    MK_CHECK_ARG(scale_type == MK_SCALE_F32 || scale_type == MK_SCALE_F16, "bad scale_type");
    mk_weight *w = nullptr;
    int32_t rc = weight_alloc(ctx, MK_FMT_Q8, scale_type, rows, cols, &w);
    if (rc != MK_OK) return rc;
    cudaError_t e = cudaSuccess;
    if (src_on_device) {
        rc = mk_launch_quantize_weight_q8(ctx, wsrc, 0, rows, w);
    } else {
        // stream the f32 source through a bounded staging buffer (<= 256 MiB)
        const int64_t chunk_rows = (int64_t)((256ull << 20) / ((size_t)cols * 4)) > 0 ? (int64_t)((256ull << 20) / ((size_t)cols * 4)) : 1;
        TmpDev stage;
        e = cudaMalloc(&stage.p, (size_t)(chunk_rows < rows ? chunk_rows : rows) * cols * 4);
        for (int64_t r0 = 0; e == cudaSuccess && rc == MK_OK && r0 < rows; r0 += chunk_rows) {
            const int64_t nr = rows - r0 < chunk_rows ? rows - r0 : chunk_rows;
            e = cudaMemcpyAsync(stage.p, wsrc + r0 * cols, (size_t)nr * cols * 4, cudaMemcpyHostToDevice, ctx->stream);
            if (e == cudaSuccess) rc = mk_launch_quantize_weight_q8(ctx, (const float *)stage.p, r0, nr, w);
            if (e == cudaSuccess && rc == MK_OK) e = cudaStreamSynchronize(ctx->stream);
        }
    }
    if (e == cudaSuccess && rc == MK_OK) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess || rc != MK_OK) {
        if (e != cudaSuccess) mk_set_error("mk_weight_q8_from_f32: %s", cudaGetErrorString(e));
        mk_weight_free(ctx, w);
        return rc != MK_OK ? rc : (e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA);
    }
    *out = w;
    return MK_OK;
}

extern "C" int32_t mk_weight_q8(mk_ctx *ctx, const int8_t *q, const void *scales, int64_t rows, int64_t cols,
                                int32_t scale_type, int32_t src_on_device, mk_weight **out) {
    MK_CHECK_ARG(q != nullptr && scales != nullptr, "NULL blob");
    MK_CHECK_ARG(scale_type == MK_SCALE_F32 || scale_type == MK_SCALE_F16, "bad scale_type");
    mk_weight *w = nullptr;
    int32_t rc = weight_alloc(ctx, MK_FMT_Q8, scale_type, rows, cols, &w);
    if (rc != MK_OK) return rc;
    const size_t qb = (size_t)rows * cols, sb = (size_t)rows * (cols / 32) * (scale_type == MK_SCALE_F16 ? 2 : 4);
    TmpDev tq, ts;
    const int8_t *dq = q;
    const void *ds = scales;
    cudaError_t e = cudaSuccess;
    if (!src_on_device) {
        e = cudaMalloc(&tq.p, qb);
        if (e == cudaSuccess) e = cudaMalloc(&ts.p, sb);
        if (e == cudaSuccess) e = cudaMemcpyAsync(tq.p, q, qb, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(ts.p, scales, sb, cudaMemcpyHostToDevice, ctx->stream);
        dq = (const int8_t *)tq.p;
        ds = ts.p;
    }
    if (e == cudaSuccess) {
        rc = mk_launch_retile_q8(ctx, dq, ds, w);
        if (rc == MK_OK) e = cudaStreamSynchronize(ctx->stream);
    }
    if (e != cudaSuccess || rc != MK_OK) {
        if (e != cudaSuccess) mk_set_error("mk_weight_q8: %s", cudaGetErrorString(e));
        mk_weight_free(ctx, w);
        return rc != MK_OK ? rc : (e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA);
    }
    *out = w;
    return MK_OK;
}

extern "C" int32_t mk_weight_export(mk_ctx *ctx, const mk_weight *w, void *values, void *scales) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr, "NULL argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const size_t vb = w->fmt == MK_FMT_MXFP4 ? (size_t)w->rows * w->cols / 2 : (size_t)w->rows * w->cols;
    const size_t sb = (size_t)w->rows * w->nb * (w->fmt == MK_FMT_MXFP4 ? 1 : (w->scale_type == MK_SCALE_F16 ? 2 : 4));
    TmpDev tv, ts;
    MK_CUDA(cudaMalloc(&tv.p, vb));
    MK_CUDA(cudaMalloc(&ts.p, sb));
    int32_t rc = w->fmt == MK_FMT_MXFP4 ? mk_launch_untile_mxfp4(ctx, w, (uint8_t *)tv.p, (uint8_t *)ts.p)
                                        : mk_launch_untile_q8(ctx, w, (int8_t *)tv.p, ts.p);
    if (rc != MK_OK) return rc;
    if (values) MK_CUDA(cudaMemcpyAsync(values, tv.p, vb, cudaMemcpyDeviceToHost, ctx->stream));
    if (scales) MK_CUDA(cudaMemcpyAsync(scales, ts.p, sb, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_dequant_mxfp4(mk_ctx *ctx, const mk_weight *w, float *out) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(w->fmt == MK_FMT_MXFP4, "not an MXFP4 weight");
    MK_CUDA(cudaSetDevice(ctx->device));
    TmpDev t;
    const size_t bytes = (size_t)w->rows * w->cols * 4;
    MK_CUDA(cudaMalloc(&t.p, bytes));
    int32_t rc = mk_launch_dequant_mxfp4(ctx, w, (float *)t.p);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(out, t.p, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

// ---------------------------------------------------------------- activations
extern "C" int32_t mk_quantize_q8(mk_ctx *ctx, const float *x, int64_t n, int8_t *q, float *scales) {
    MK_CHECK_ARG(ctx != nullptr && x != nullptr && q != nullptr && scales != nullptr, "NULL argument");
    MK_CHECK_ARG(n > 0 && n % 32 == 0, "n must be a positive multiple of 32");
    MK_CUDA(cudaSetDevice(ctx->device));
    const int64_t nb = n / 32;
    const size_t need = (size_t)n * 4 + (size_t)n + (size_t)nb * 4;
    int32_t rc = mk_io_reserve(ctx, need + 64);
    if (rc != MK_OK) return rc;
    float *dx = (float *)ctx->io_dev;
    float *ds = dx + n;
    int8_t *dq = (int8_t *)(ds + nb);
    MK_CUDA(cudaMemcpyAsync(dx, x, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = mk_launch_quantize_act(ctx, dx, 1, n, n, nb, 0, dq, ds);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(q, dq, (size_t)n, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaMemcpyAsync(scales, ds, (size_t)nb * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

// ---------------------------------------------------------------- matvec
// Device path shared by every matvec entry point: quantize the activations into
// the context workspace, then run the fused kernel in passes of <= 8 tokens.
static int32_t matvec_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode,
                          int32_t *argmax_dev) {
    const int x2 = (act_mode & 0xFF) == MK_ACT_Q8X2;
    const int strict = (act_mode & MK_ACT_STRICT) != 0;
    MK_CHECK_ARG((act_mode & 0xFF) == MK_ACT_Q8 || x2, "unknown act_mode");
    const int per_pass = x2 ? 4 : 8;
    const int64_t ldq = w->nbp * 32;
    const size_t xq_bytes = mk_align_up((size_t)(x2 ? 2 : 1) * per_pass * ldq, 256);
    const size_t xs_bytes = mk_align_up((size_t)per_pass * w->nbp * 4, 256);
    const size_t am_bytes = argmax_dev ? mk_align_up(mk_argmax_scratch_bytes(batch), 256) : 0;
    int32_t rc = mk_ws_reserve(ctx, xq_bytes + xs_bytes + am_bytes);
    if (rc != MK_OK) return rc;
    int8_t *xq = (int8_t *)ctx->ws;
    float *xs = (float *)((char *)ctx->ws + xq_bytes);
    void *am = (char *)ctx->ws + xq_bytes + xs_bytes;
    for (int t0 = 0; t0 < batch; t0 += per_pass) {
        const int nt = batch - t0 < per_pass ? batch - t0 : per_pass;
        rc = mk_launch_quantize_act(ctx, x + (int64_t)t0 * w->cols, nt, w->cols, w->cols, w->nbp, x2, xq, xs);
        if (rc != MK_OK) return rc;
        rc = mk_launch_qgemv(ctx, w, xq, xs, nt, x2, strict, y + (int64_t)t0 * w->rows, w->rows);
        if (rc != MK_OK) return rc;
    }
    if (argmax_dev) return mk_launch_argmax(ctx, y, w->rows, w->rows, batch, argmax_dev, am);
    return MK_OK;
}

static int32_t matvec_host(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode,
                           int32_t *argmax) {
    const size_t xb = (size_t)batch * w->cols * 4, yb = (size_t)batch * w->rows * 4, ab = argmax ? (size_t)batch * 4 : 0;
    int32_t rc = mk_io_reserve(ctx, mk_align_up(xb, 256) + mk_align_up(yb, 256) + mk_align_up(ab, 256));
    if (rc != MK_OK) return rc;
    float *dx = (float *)ctx->io_dev;
    float *dy = (float *)((char *)ctx->io_dev + mk_align_up(xb, 256));
    int32_t *da = argmax ? (int32_t *)((char *)dy + mk_align_up(yb, 256)) : nullptr;
    MK_CUDA(cudaMemcpyAsync(dx, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = matvec_dev(ctx, w, dx, dy, batch, act_mode, da);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(y, dy, yb, cudaMemcpyDeviceToHost, ctx->stream));
    if (argmax) MK_CUDA(cudaMemcpyAsync(argmax, da, ab, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

static int32_t matvec_check(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int fmt) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && x != nullptr && y != nullptr, "NULL argument");
    MK_CHECK_ARG(w->fmt == fmt, "weight handle has the wrong format for this call");
    MK_CHECK_ARG(batch >= 1 && batch <= 4096, "batch must be in [1, 4096]");
    MK_CUDA(cudaSetDevice(ctx->device));
    return MK_OK;
}

extern "C" int32_t mk_matvec_mxfp4(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode) {
    int32_t rc = matvec_check(ctx, w, x, y, batch, MK_FMT_MXFP4);
    return rc != MK_OK ? rc : matvec_host(ctx, w, x, y, batch, act_mode, nullptr);
}
extern "C" int32_t mk_matvec_mxfp4_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode) {
    int32_t rc = matvec_check(ctx, w, x, y, batch, MK_FMT_MXFP4);
    return rc != MK_OK ? rc : matvec_dev(ctx, w, x, y, batch, act_mode, nullptr);
}
extern "C" int32_t mk_matvec_q8(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode,
                                int32_t *argmax) {
    int32_t rc = matvec_check(ctx, w, x, y, batch, MK_FMT_Q8);
    return rc != MK_OK ? rc : matvec_host(ctx, w, x, y, batch, act_mode, argmax);
}
extern "C" int32_t mk_matvec_q8_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode,
                                    int32_t *argmax) {
    int32_t rc = matvec_check(ctx, w, x, y, batch, MK_FMT_Q8);
    return rc != MK_OK ? rc : matvec_dev(ctx, w, x, y, batch, act_mode, argmax);
}
