// Dequant-fused quantized matrix x vector for MXFP4 and q8_0 weights (sm_100a).
//
// What it computes, per output row r and token:
//   MXFP4 : sum_g  idot(r,g) * (2^(sb[r,g]-128) * xs[g])      (src/mxfp4.rs:409-418)
//   q8_0  : sum_g (ws[r,g] * xs[g]) * idot(r,g)                (src/model.rs:337-347)
// where idot is the EXACT int32 dot of one 32-wide block of the weight row with
// the q8_0-quantized activation (src/q8.rs:119-125, 194-202).
//
// How: the weights sit in HBM in mma.m16n8k32 fragment order (see mk_weight), so
// one warp streams a 16-row tile with one coalesced 16-byte load per lane.  The
// block dot runs on the tensor cores as int8 x int8 -> int32 (exact).  E2M1
// codes are decoded in registers with byte permutes: a code's 3 magnitude bits
// select one of the 8 bytes {0,1,2,3,4,6,8,12} (= E2M1 x 2); a set sign bit makes
// the permute return 0, so one pass yields the positive part and a second pass
// over the sign-flipped word yields the negative part; idot = dot(pos) - dot(neg).
//
// Two schedules:
//   "spread"  (<= 2 activation columns): the MMA's 8 output columns are used for
//             4 consecutive weight blocks x 2 columns, so the per-block scaling
//             runs once per 4 blocks with all lanes busy.
//   "batched" (<= 8 tokens): the 8 columns are 8 tokens; each lane owns 4 outputs
//             and adds the block terms in ascending block order with separate
//             multiply and add.  With no K split that reproduces the CPU sums
//             bit for bit (MK_ACT_STRICT).
#include "qgemv_core.cuh"

namespace {
using namespace mkq;

// ------------------------------------------------------------------ one matrix, "spread" schedule
// CTA = 8 warps = (8/KS) row tiles x KS K-slices.
template <int WF, int KS, int NSLOT, bool X2>
__global__ void __launch_bounds__(256)
qgemv_spread_kernel(const void *__restrict__ wt, const void *__restrict__ wscale, const int8_t *__restrict__ xq,
                    const float *__restrict__ xs, int64_t ldq, int64_t nbp, float *__restrict__ y, int64_t ldy,
                    int64_t rows, int64_t nrt, const Consts k) {
    constexpr int RT = 8 / KS;
    constexpr int NOUT = X2 ? 1 : NSLOT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rt_local = warp / KS, ks = warp % KS;
    const int64_t rt = (int64_t)blockIdx.x * RT + rt_local;
    float acc[2][NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) acc[0][o] = acc[1][o] = 0.0f;
    // a small kernel launched behind this one with programmatic stream serialization (the greedy pick, the exchange of a
    // sharded head) may become resident now; it waits for this grid's results itself
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (rt < nrt) {
        const int slot = g & 1;
        const int8_t *xrow = slot < NSLOT ? xq + (int64_t)slot * ldq : nullptr;
        warp_tile_spread<WF, NSLOT, X2>(tile_values<WF>(wt, rt, nbp), tile_scales<WF>(wscale, rt, nbp), nbp >> 2, ks, KS,
                                        lane, xrow, xs, xs + nbp, k, acc);
    }
    if constexpr (KS > 1) {
        __shared__ float red[8][16][NOUT];
        if (t == 0) {
#pragma unroll
            for (int o = 0; o < NOUT; ++o) {
                red[warp][g][o] = acc[0][o];
                red[warp][g + 8][o] = acc[1][o];
            }
        }
        __syncthreads();
        if (ks == 0 && t == 0 && rt < nrt) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r16 = g + 8 * h;
                const int64_t row = rt * 16 + r16;
                if (row < rows) {
#pragma unroll
                    for (int o = 0; o < NOUT; ++o) {
                        float v = red[warp][r16][o];
                        for (int k = 1; k < KS; ++k) v += red[warp + k][r16][o];
                        y[(int64_t)o * ldy + row] = v;
                    }
                }
            }
        }
    } else {
        if (t == 0 && rt < nrt) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int64_t row = rt * 16 + g + 8 * h;
                if (row < rows) {
#pragma unroll
                    for (int o = 0; o < NOUT; ++o) y[(int64_t)o * ldy + row] = acc[h][o];
                }
            }
        }
    }
}

// ------------------------------------------------------------------ one matrix, "batched" schedule
template <int WF, int KS, bool X2, bool ORDERED>
__global__ void __launch_bounds__(256)
qgemv_batched_kernel(const void *__restrict__ wt, const void *__restrict__ wscale, const int8_t *__restrict__ xq,
                     const float *__restrict__ xs, int64_t ldq, int64_t nbp, int ntok, float *__restrict__ y,
                     int64_t ldy, int64_t rows, int64_t nrt, const Consts k) {
    constexpr int RT = 8 / KS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rt_local = warp / KS, ks = warp % KS;
    const int64_t rt = (int64_t)blockIdx.x * RT + rt_local;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const int tok_a = X2 ? t : 2 * t, tok_b = X2 ? t : 2 * t + 1;
    if (rt < nrt) {
        const int ctok = X2 ? (g >> 1) : g;
        const int8_t *xcol = ctok < ntok ? xq + (X2 ? (int64_t)(g & 1) * ntok * ldq : 0) + (int64_t)ctok * ldq : nullptr;
        const float *xsa = tok_a < ntok ? xs + (int64_t)tok_a * nbp : nullptr;
        const float *xsb = tok_b < ntok ? xs + (int64_t)tok_b * nbp : nullptr;
        warp_tile_batched<WF, X2, ORDERED>(tile_values<WF>(wt, rt, nbp), tile_scales<WF>(wscale, rt, nbp), nbp >> 2, ks, KS, lane,
                                  xcol, xsa, xsb, k, acc);
    }
    if constexpr (KS > 1) {
        __shared__ float red[8][32][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) red[warp][lane][j] = acc[j];
        __syncthreads();
        if (ks == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float v = red[warp][lane][j];
                for (int k = 1; k < KS; ++k) v += red[warp + k][lane][j];
                acc[j] = v;
            }
        }
    }
    if (ks == 0 && rt < nrt) {
        const int64_t row_g = rt * 16 + g, row_h = row_g + 8;
        if (tok_a < ntok) {
            if (row_g < rows) y[(int64_t)tok_a * ldy + row_g] = acc[0];
            if (row_h < rows) y[(int64_t)tok_a * ldy + row_h] = acc[2];
        }
        if (!X2 && tok_b < ntok) {
            if (row_g < rows) y[(int64_t)tok_b * ldy + row_g] = acc[1];
            if (row_h < rows) y[(int64_t)tok_b * ldy + row_h] = acc[3];
        }
    }
}

// ------------------------------------------------------------------ activation quantization
// One warp per (token, block): q8::quantize_q8_into (src/q8.rs:49-69), bit-exact:
// dx = max|x| / 127 (IEEE divide), q = clamp(round-half-away(x / dx), -127, 127).
// X2: d = max|x| / 16256, q16 = round(x / d); hi = round(q16 / 128), lo = q16 - 128 hi.
template <bool X2>
__global__ void __launch_bounds__(256)
quantize_act_kernel(const float *__restrict__ x, int ntok, int64_t cols, int64_t ldx, int64_t nbp,
                    int8_t *__restrict__ xq, float *__restrict__ xs) {
    // a matvec launched behind this kernel with programmatic stream serialization may start its weight loads now
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= (int64_t)ntok * nbp) return;
    const int64_t tok = w / nbp, b = w % nbp;
    const int64_t c = b * 32 + lane;
    const float v = (c < cols) ? x[tok * ldx + c] : 0.0f;
    float mx = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    const int64_t ldq = nbp * 32;
    if constexpr (!X2) {
        const float dx = __fdiv_rn(mx, 127.0f);
        int q = 0;
        if (dx != 0.0f) q = (int)fminf(fmaxf(roundf(__fdiv_rn(v, dx)), -127.0f), 127.0f);
        uint32_t qb = (uint32_t)q & 0xFFu;
        uint32_t pk = qb | (__shfl_down_sync(0xFFFFFFFFu, qb, 1) << 8) | (__shfl_down_sync(0xFFFFFFFFu, qb, 2) << 16) |
                      (__shfl_down_sync(0xFFFFFFFFu, qb, 3) << 24);
        if ((lane & 3) == 0) ((uint32_t *)(xq + tok * ldq + b * 32))[lane >> 2] = pk;
        if (lane == 0) xs[tok * nbp + b] = dx;
    } else {
        const float d = __fdiv_rn(mx, 16256.0f);
        int q16 = 0;
        if (d != 0.0f) q16 = (int)fminf(fmaxf(roundf(__fdiv_rn(v, d)), -16256.0f), 16256.0f);
        int hi = (q16 + (q16 >= 0 ? 64 : -64)) / 128;
        int lo = q16 - 128 * hi;
        uint32_t hb = (uint32_t)hi & 0xFFu, lb = (uint32_t)lo & 0xFFu;
        uint32_t ph = hb | (__shfl_down_sync(0xFFFFFFFFu, hb, 1) << 8) | (__shfl_down_sync(0xFFFFFFFFu, hb, 2) << 16) |
                      (__shfl_down_sync(0xFFFFFFFFu, hb, 3) << 24);
        uint32_t pl = lb | (__shfl_down_sync(0xFFFFFFFFu, lb, 1) << 8) | (__shfl_down_sync(0xFFFFFFFFu, lb, 2) << 16) |
                      (__shfl_down_sync(0xFFFFFFFFu, lb, 3) << 24);
        if ((lane & 3) == 0) {
            ((uint32_t *)(xq + tok * ldq + b * 32))[lane >> 2] = ph;
            ((uint32_t *)(xq + ((int64_t)ntok + tok) * ldq + b * 32))[lane >> 2] = pl;
        }
        if (lane == 0) xs[tok * nbp + b] = d;
    }
}

// ------------------------------------------------------------------ argmax (first index of the maximum)
struct ArgPair { float v; int32_t i; };
__device__ __forceinline__ ArgPair arg_better(ArgPair a, ArgPair b) {
    // strict '>' keeps the earlier index on ties (src/model.rs:3277-3290); i < 0 marks "empty"
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ __forceinline__ ArgPair arg_block_reduce(ArgPair p) {
    __shared__ float sv[32];
    __shared__ int32_t si[32];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgPair q;
        q.v = __shfl_xor_sync(0xFFFFFFFFu, p.v, o);
        q.i = __shfl_xor_sync(0xFFFFFFFFu, p.i, o);
        p = arg_better(p, q);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = p.v; si[warp] = p.i; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        p.v = lane < nw ? sv[lane] : 0.0f;
        p.i = lane < nw ? si[lane] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgPair q;
            q.v = __shfl_xor_sync(0xFFFFFFFFu, p.v, o);
            q.i = __shfl_xor_sync(0xFFFFFFFFu, p.i, o);
            p = arg_better(p, q);
        }
    }
    return p;
}
#define ARGMAX_PARTS 128
// First index of the maximum of every row in ONE launch: ARGMAX_PARTS CTAs per row leave a partial each; the last one
// to finish (a counter per row, nobody waits) folds them.  `count` is 0 before and after.
// Measured and rejected: the same fold inside the one-token matvec kernel (a partial per matvec CTA) - the lm_head
// matvec went from 190.8 to 202.4 us, more than the launch it saves.
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ y, int64_t n, int64_t ldy, float *__restrict__ pv,
                                                    int32_t *__restrict__ pi, int32_t *__restrict__ out, unsigned *__restrict__ count) {
    __shared__ int s_last;
    // launched behind the matvec with programmatic stream serialization, this grid is resident before the logits exist
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int row = blockIdx.y;
    const float *yr = y + (int64_t)row * ldy;
    ArgPair p = {0.0f, -1};
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        ArgPair q = {yr[i], (int32_t)i};
        p = arg_better(p, q);
    }
    p = arg_block_reduce(p);
    if (threadIdx.x == 0) {
        pv[row * ARGMAX_PARTS + blockIdx.x] = p.v;
        pi[row * ARGMAX_PARTS + blockIdx.x] = p.i;
        __threadfence();
        const unsigned prev = atomicAdd(&count[row], 1u);
        s_last = prev == gridDim.x - 1 ? 1 : 0;
        if (s_last) count[row] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    p = ArgPair{0.0f, -1};
    if (threadIdx.x < ARGMAX_PARTS) p = ArgPair{__ldcg(pv + row * ARGMAX_PARTS + threadIdx.x), __ldcg(pi + row * ARGMAX_PARTS + threadIdx.x)};
    p = arg_block_reduce(p);
    if (threadIdx.x == 0) out[row] = p.i;
}

// ------------------------------------------------------------------ dispatch
template <int WF, int KS>
void launch_spread(const mk_weight *w, cudaStream_t st, const Consts &k, const int8_t *xq, const float *xs, int nslot, bool x2, float *y,
                   int64_t ldy, bool pdl) {
    constexpr int RT = 8 / KS;
    const unsigned grid = (unsigned)mk_ceil_div(w->nrt, RT);
    const int64_t ldq = w->nbp * 32;
    const void *wt = w->values;
    if (pdl && !x2 && nslot == 1) {
        // one token behind its activation quantizer: programmatic stream serialization, the kernel waits
        // (griddepcontrol.wait) between its first weight loads and its first read of the quantized activations
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, qgemv_spread_kernel<WF, KS, 1, false>, wt, (const void *)w->scales, xq, xs, ldq, (int64_t)w->nbp, y, ldy,
                           (int64_t)w->rows, (int64_t)w->nrt, k);
        return;
    }
    if (x2)
        qgemv_spread_kernel<WF, KS, 2, true><<<grid, 256, 0, st>>>(wt, w->scales, xq, xs, ldq, w->nbp, y, ldy, w->rows, w->nrt, k);
    else if (nslot == 2)
        qgemv_spread_kernel<WF, KS, 2, false><<<grid, 256, 0, st>>>(wt, w->scales, xq, xs, ldq, w->nbp, y, ldy, w->rows, w->nrt, k);
    else
        qgemv_spread_kernel<WF, KS, 1, false><<<grid, 256, 0, st>>>(wt, w->scales, xq, xs, ldq, w->nbp, y, ldy, w->rows, w->nrt, k);
}
template <int WF, int KS>
void launch_batched(const mk_weight *w, cudaStream_t st, const Consts &k, const int8_t *xq, const float *xs, int ntok, bool x2,
                    bool ordered, float *y, int64_t ldy) {
    constexpr int RT = 8 / KS;
    const unsigned grid = (unsigned)mk_ceil_div(w->nrt, RT);
    const int64_t ldq = w->nbp * 32;
    const void *wt = w->values;
    if constexpr (KS == 1) {
        if (ordered) {
            if (x2)
                qgemv_batched_kernel<WF, 1, true, true><<<grid, 256, 0, st>>>(wt, w->scales, xq, xs, ldq, w->nbp, ntok, y, ldy, w->rows, w->nrt, k);
            else
                qgemv_batched_kernel<WF, 1, false, true><<<grid, 256, 0, st>>>(wt, w->scales, xq, xs, ldq, w->nbp, ntok, y, ldy, w->rows, w->nrt, k);
            return;
        }
    }
    if (x2)
        qgemv_batched_kernel<WF, KS, true, false><<<grid, 256, 0, st>>>(wt, w->scales, xq, xs, ldq, w->nbp, ntok, y, ldy, w->rows, w->nrt, k);
    else
        qgemv_batched_kernel<WF, KS, false, false><<<grid, 256, 0, st>>>(wt, w->scales, xq, xs, ldq, w->nbp, ntok, y, ldy, w->rows, w->nrt, k);
}
template <int WF>
void launch_wf(const mk_weight *w, cudaStream_t st, const Consts &k, int ks, bool spread, bool ordered, const int8_t *xq,
               const float *xs, int ntok, bool x2, float *y, int64_t ldy, bool pdl) {
#define MK_KS_CASE(K)                                                         \
    case K:                                                                   \
        if (spread) launch_spread<WF, K>(w, st, k, xq, xs, ntok, x2, y, ldy, pdl);    \
        else launch_batched<WF, K>(w, st, k, xq, xs, ntok, x2, ordered, y, ldy);          \
        break;
    switch (ks) {
        MK_KS_CASE(1)
        MK_KS_CASE(2)
        MK_KS_CASE(4)
        MK_KS_CASE(8)
    }
#undef MK_KS_CASE
}

} // namespace

// K split: enough CTAs to fill the GPU several times over, but at least a few
// block groups per warp.
static int pick_ks(const mk_ctx *ctx, const mk_weight *w, bool strict) {
    if (strict) return 1;
    if (ctx->force_ks) return ctx->force_ks;
    const int64_t ngroups = w->nbp / 4;
    int ks = 1;
    while (ks < 8) {
        const int64_t ctas = mk_ceil_div(w->nrt, 8 / ks);
        const int64_t groups_per_warp = ngroups / (ks * 2);
        if (ctas >= (int64_t)ctx->sm_count * 16 || groups_per_warp < 3) break;
        ks *= 2;
    }
    return ks;
}

int32_t mk_launch_quantize_act(mk_ctx *ctx, const float *x, int ntok, int64_t cols, int64_t ldx, int64_t nbp, int x2,
                               int8_t *xq, float *xs) {
    const int64_t warps = (int64_t)ntok * nbp;
    const unsigned grid = (unsigned)mk_ceil_div(warps * 32, 256);
    if (x2)
        quantize_act_kernel<true><<<grid, 256, 0, ctx->stream>>>(x, ntok, cols, ldx, nbp, xq, xs);
    else
        quantize_act_kernel<false><<<grid, 256, 0, ctx->stream>>>(x, ntok, cols, ldx, nbp, xq, xs);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

int32_t mk_launch_qgemv(mk_ctx *ctx, const mk_weight *w, const int8_t *xq, const float *xs, int ntok, int x2, int strict,
                        float *y, int64_t ldy) {
    MK_CHECK_ARG(ntok >= 1 && ntok <= (x2 ? 4 : 8), "token count out of range for one pass");
    const bool spread = !strict && (x2 ? ntok == 1 : ntok <= 2);
    const int ks = pick_ks(ctx, w, strict != 0);
    const int wf = w->fmt == MK_FMT_MXFP4 ? W_MXFP4 : (w->scale_type == MK_SCALE_F16 ? W_Q8_F16 : W_Q8_F32);
    mk_prof_scope prof(ctx, w->fmt == MK_FMT_MXFP4 ? MK_PROF_MATVEC_MXFP4 : MK_PROF_LM_HEAD);
    const Consts k = {65536u, 0xFFFFFFFFu, ctx->zeros_dev};
    // the callers of this function launch the activation quantizer directly before it on the same stream
    const bool pdl = ctx->pdl != 0;
    switch (wf) {
    case W_MXFP4: launch_wf<W_MXFP4>(w, ctx->stream, k, ks, spread, strict != 0, xq, xs, ntok, x2 != 0, y, ldy, pdl); break;
    case W_Q8_F32: launch_wf<W_Q8_F32>(w, ctx->stream, k, ks, spread, strict != 0, xq, xs, ntok, x2 != 0, y, ldy, pdl); break;
    default: launch_wf<W_Q8_F16>(w, ctx->stream, k, ks, spread, strict != 0, xq, xs, ntok, x2 != 0, y, ldy, pdl); break;
    }
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

size_t mk_argmax_scratch_bytes(int batch) { return (size_t)batch * ARGMAX_PARTS * (sizeof(float) + sizeof(int32_t)); }

int32_t mk_launch_argmax(mk_ctx *ctx, const float *y, int64_t n, int64_t ldy, int batch, int32_t *out, void *scratch) {
    float *pv = (float *)scratch;
    int32_t *pi = (int32_t *)(pv + (size_t)batch * ARGMAX_PARTS);
    if (batch > 64) { mk_set_error("greedy pick: more than 64 rows"); return MK_ERR_ARG; }
    if (ctx->pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(ARGMAX_PARTS, (unsigned)batch); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = ctx->stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        cudaLaunchKernelEx(&cfg, argmax_kernel, y, n, ldy, pv, pi, out, ctx->argmax_count);
    } else {
        argmax_kernel<<<dim3(ARGMAX_PARTS, batch), 256, 0, ctx->stream>>>(y, n, ldy, pv, pi, out, ctx->argmax_count);
    }
    ctx->launches += 1;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

// ------------------------------------------------------------------ matvec that allocates nothing
// Scratch for the quantized activations of mk_matvec_mxfp4_noalloc_dev: a fixed
// array in the library's device image instead of a cudaMalloc'd workspace.  Every
// GPU that loads the library holds these 144 KiB until the process exits.
#define MK_NOALLOC_MAX_COLS 16384
#define MK_NOALLOC_MAX_TOKENS 8
#define MK_NOALLOC_XQ_BYTES (MK_NOALLOC_MAX_TOKENS * MK_NOALLOC_MAX_COLS)
#define MK_NOALLOC_XS_BYTES (MK_NOALLOC_MAX_TOKENS * (MK_NOALLOC_MAX_COLS / 32) * 4)
static __device__ __align__(256) unsigned char mk_noalloc_scratch[MK_NOALLOC_XQ_BYTES + MK_NOALLOC_XS_BYTES];

// Device address of the array above, per device ordinal.  The array's name is only
// a host-side handle; the address a kernel can use comes from cudaGetSymbolAddress
// with that device current.
// The table is written without a lock: two host threads that make their first call on the
// same device at once both look the address up and both store the SAME value (the address of
// a symbol is fixed per device), so the race is benign; a context is not re-entrant anyway.
#define MK_NOALLOC_MAX_DEVICES 64
static void *g_noalloc_addr[MK_NOALLOC_MAX_DEVICES];

extern "C" int32_t mk_matvec_mxfp4_noalloc_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch,
                                               int32_t act_mode) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && x != nullptr && y != nullptr, "NULL argument");
    MK_CHECK_ARG(w->fmt == MK_FMT_MXFP4, "weight handle is not MXFP4");
    const int x2 = (act_mode & 0xFF) == MK_ACT_Q8X2;
    const int strict = (act_mode & MK_ACT_STRICT) != 0;
    MK_CHECK_ARG((act_mode & 0xFF) == MK_ACT_Q8 || x2, "unknown act_mode");
    const int64_t ldq = w->nbp * 32;
    if (ldq > MK_NOALLOC_MAX_COLS || batch < 1 || batch * (x2 ? 2 : 1) > MK_NOALLOC_MAX_TOKENS) {
        mk_set_error("mk_matvec_mxfp4_noalloc_dev: the fixed scratch holds at most %d columns (this matrix: %lld) and %d "
                     "activation rows (asked: %d%s); use mk_matvec_mxfp4_dev for larger calls",
                     MK_NOALLOC_MAX_COLS, (long long)ldq, MK_NOALLOC_MAX_TOKENS, batch, x2 ? " x 2 limbs" : "");
        return MK_ERR_ARG;
    }
    MK_CHECK_ARG(ctx->device >= 0 && ctx->device < MK_NOALLOC_MAX_DEVICES, "device ordinal out of range");
    MK_CUDA(cudaSetDevice(ctx->device));
    if (g_noalloc_addr[ctx->device] == nullptr) {
        // set-up on the first call on this device
        void *p = nullptr;
        MK_CUDA(cudaGetSymbolAddress(&p, mk_noalloc_scratch));
        g_noalloc_addr[ctx->device] = p;
    }
    int8_t *xq = (int8_t *)g_noalloc_addr[ctx->device];
    float *xs = (float *)((unsigned char *)g_noalloc_addr[ctx->device] + MK_NOALLOC_XQ_BYTES);
    // the quantizer overwrites every byte and scale the matvec reads (padding blocks
    // included), so nothing left by an earlier call is ever consumed
    int32_t rc = mk_launch_quantize_act(ctx, x, batch, w->cols, w->cols, w->nbp, x2, xq, xs);
    if (rc != MK_OK) return rc;
    return mk_launch_qgemv(ctx, w, xq, xs, batch, x2, strict, y, w->rows);
}
