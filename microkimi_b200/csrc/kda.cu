// KDA decode step and AttnRes on the device (sm_100a).
//
// Reference: kda_conv_step, kda_norm_head, kda_gate, kda_recur_step, kda_gated_onorm and the
// part of kda_forward that strings them together (src/model.rs:1066-1228); attn_res_refs
// (src/model.rs:632-669).  One token per call; the layer's state (the conv windows of q, k, v
// and the matrix S [heads][dim][dim]) stays in device memory between calls.
//
// Arithmetic: every sum runs in the engine's order with a separate multiply and add, dot()
// with its 8 accumulators; exp is taken in double precision and rounded once, which gives
// the bits of a correctly rounded expf in all but about one case in 10^9.
//
// kda_step_kernel: one CTA per head, one thread per channel.  The columns of S are
// independent of one another (decay scales rows, delta[j] and o[j] are sums down column j),
// so thread j owns column j, reads it once into registers (dim <= 128), walks it in row
// order for delta, then again for the update and o, and writes it once: 2 * dim^2 * 4 bytes
// of traffic per head and token, coalesced across the threads of a row.
#include "f32gemv.cuh"
#include "mk_common.cuh"

#include <cmath>
#include <new>

struct mk_kda {
    int heads, dim, kconv;
    float gate_lb, rms_eps, q_scale;
    float *conv_w;   // [3][proj][kconv]  q, k, v
    float *a_log;    // [dim]
    float *dt_bias;  // [proj]
    float *o_norm;   // [dim]
    float *conv;     // [3][kconv - 1][proj]  previous raw inputs, oldest first
    float *s;        // [heads][dim][dim]
};

namespace {
__device__ __forceinline__ float exp_cr(float x) { return (float)exp((double)x); }
__device__ __forceinline__ float sigmoid_cr(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, exp_cr(-x))); }

// dot(a, a) over n values in shared memory, by one whole warp, in the engine's order; the result in every lane
__device__ __forceinline__ float warp_sumsq(const float *a, int n, int lane) {
    const int j = lane & 7, full = n & ~7;
    float acc = 0.0f;
    for (int c = 0; c < full; c += 8) acc = __fadd_rn(acc, __fmul_rn(a[c + j], a[c + j]));
    float ss = mkf::reduce8(acc, lane);
    for (int c = full; c < n; ++c) ss = __fadd_rn(ss, __fmul_rn(a[c], a[c]));
    return ss;
}

struct KdaArgs {
    const float *q_raw, *k_raw, *v_raw, *g_low, *beta_raw, *g2;
    const float *conv_w, *a_log, *dt_bias, *o_norm;
    float *conv, *s, *o;
    int heads, dim, kconv;
    float gate_lb, rms_eps, q_scale;
    // several consecutive positions in one launch (kda_step_kernel only): token t reads its q / k / v / g2 / beta rows
    // t * ld_x floats on, its low-rank gate row t * ld_g on, and writes its output row t * ld_o on
    int n_tok;
    int64_t ld_x, ld_g, ld_o;
};

// One channel's conv inputs, loaded before any arithmetic so that all global loads of a thread are in flight
// together: KC weights (weight KC - 1 on the current input) and the KC - 1 previous raw inputs, oldest first.
template <int KC>
struct ConvIn {
    float w[KC > 0 ? KC : 1], old[KC > 1 ? KC - 1 : 1], raw;
    __device__ __forceinline__ void load(const float *__restrict__ cw, const float *__restrict__ win, int64_t proj, int64_t i,
                                         const float *__restrict__ src) {
        if constexpr (KC == 4) {
            const float4 v = *reinterpret_cast<const float4 *>(cw + i * 4);
            w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
        } else {
#pragma unroll
            for (int j = 0; j < KC; ++j) w[j] = cw[i * KC + j];
        }
#pragma unroll
        for (int j = 0; j < KC - 1; ++j) old[j] = win[(int64_t)j * proj + i];
        raw = src[i];
    }
    // conv + SiLU in the engine's order; shifts the channel's window (no other thread touches it)
    __device__ __forceinline__ float apply(float *__restrict__ win, int64_t proj, int64_t i) const {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < KC - 1; ++j) {
            acc = __fadd_rn(acc, __fmul_rn(w[j], old[j]));
            win[(int64_t)j * proj + i] = j + 1 < KC - 1 ? old[j + 1] : raw;
        }
        acc = __fadd_rn(acc, __fmul_rn(w[KC - 1], raw));
        return __fmul_rn(acc, sigmoid_cr(acc));
    }
};
// any kconv: the same, with the loads inside the loop
__device__ __forceinline__ float conv_channel(const float *w, float *win, int64_t proj, int64_t i, int kconv, float raw) {
    float acc = 0.0f;
    for (int j = 0; j < kconv - 1; ++j) {
        const float old = win[(int64_t)j * proj + i];
        acc = __fadd_rn(acc, __fmul_rn(w[i * kconv + j], old));
        if (j > 0) win[(int64_t)(j - 1) * proj + i] = old;
    }
    win[(int64_t)(kconv - 2) * proj + i] = raw;
    acc = __fadd_rn(acc, __fmul_rn(w[i * kconv + kconv - 1], raw));
    return __fmul_rn(acc, sigmoid_cr(acc));
}

// DIM > 0: the column lives in registers and is fetched at kernel start, together with every other input of the
// thread; DIM == 0: any dim, the decayed column is parked in S between the passes.  KC == 4: the engine's conv
// width with its loads hoisted; KC == 0: any width.
template <int DIM, int KC>
__global__ void __launch_bounds__(DIM > 0 ? DIM : 1024) kda_step_kernel(KdaArgs a) {
    extern __shared__ float sm[];
    const int dim = DIM > 0 ? DIM : a.dim;
    float *qs = sm, *ks = sm + dim, *ds = sm + 2 * dim, *red = sm + 3 * dim;
    const int h = blockIdx.x, c = threadIdx.x, lane = c & 31, warp = c >> 5, nwarps = blockDim.x >> 5;
    const bool active = c < dim;
    const int64_t proj = (int64_t)a.heads * dim, i = (int64_t)h * dim + c;
    const int64_t wq = 0, wk = proj * a.kconv, wv = 2 * proj * a.kconv;                       // conv weights of q, k, v
    const int64_t cq = 0, ck = (int64_t)(a.kconv - 1) * proj, cv = 2 * (int64_t)(a.kconv - 1) * proj; // their windows
    float *col = a.s + (int64_t)h * dim * dim + c;
    float x[DIM > 0 ? DIM : 1];
    // n_tok consecutive positions: the column stays in registers from one position to the next (DIM > 0) and is
    // written back after the last one; each position's arithmetic is that of a launch of its own
    for (int tt = 0; tt < a.n_tok; ++tt) {
    const float *q_raw = a.q_raw + tt * a.ld_x, *k_raw = a.k_raw + tt * a.ld_x, *v_raw = a.v_raw + tt * a.ld_x;
    const float *g2_in = a.g2 + tt * a.ld_x, *beta_in = a.beta_raw + tt * a.ld_x, *glow_in = a.g_low + tt * a.ld_g;
    const bool last_tok = tt == a.n_tok - 1;
    float vv = 0.0f, g2v = 0.0f, onv = 0.0f, bh = 0.0f;
    if (active) {
        float glow, dtb, alog;
        ConvIn<KC> iq, ik, iv;
        if constexpr (KC > 0) {
            iq.load(a.conv_w + wq, a.conv + cq, proj, i, q_raw);
            ik.load(a.conv_w + wk, a.conv + ck, proj, i, k_raw);
            iv.load(a.conv_w + wv, a.conv + cv, proj, i, v_raw);
        }
        glow = glow_in[i]; dtb = a.dt_bias[i]; alog = a.a_log[c];
        g2v = g2_in[i]; onv = a.o_norm[c]; bh = beta_in[h];
        if constexpr (DIM > 0) {
            if (tt == 0) {
#pragma unroll
                for (int r = 0; r < DIM; ++r) x[r] = col[(int64_t)r * DIM];
            }
        }
        if constexpr (KC > 0) {
            qs[c] = iq.apply(a.conv + cq, proj, i);
            ks[c] = ik.apply(a.conv + ck, proj, i);
            vv = iv.apply(a.conv + cv, proj, i);
        } else {
            qs[c] = conv_channel(a.conv_w + wq, a.conv + cq, proj, i, a.kconv, q_raw[i]);
            ks[c] = conv_channel(a.conv_w + wk, a.conv + ck, proj, i, a.kconv, k_raw[i]);
            vv = conv_channel(a.conv_w + wv, a.conv + cv, proj, i, a.kconv, v_raw[i]);
        }
        const float g = __fmul_rn(a.gate_lb, sigmoid_cr(__fmul_rn(exp_cr(alog), __fadd_rn(glow, dtb))));
        ds[c] = exp_cr(g);
        bh = sigmoid_cr(bh);
        g2v = sigmoid_cr(g2v);
    }
    __syncthreads();
    // per-head L2 norms: q by warp 0, k by the last warp (the same warp when there is one)
    if (warp == 0) {
        const float n2 = warp_sumsq(qs, dim, lane);
        if (lane == 0) red[0] = __fdiv_rn(a.q_scale, fmaxf(__fsqrt_rn(n2), 1e-12f));
    }
    if (warp == nwarps - 1) {
        const float n2 = warp_sumsq(ks, dim, lane);
        if (lane == 0) red[1] = __fdiv_rn(1.0f, fmaxf(__fsqrt_rn(n2), 1e-12f));
    }
    __syncthreads();
    if (active) {
        qs[c] = __fmul_rn(qs[c], red[0]);
        ks[c] = __fmul_rn(ks[c], red[1]);
    }
    __syncthreads();
    float o = 0.0f;
    if (active) {
        float delta = vv;
        if constexpr (DIM > 0) {
#pragma unroll
            for (int r = 0; r < DIM; ++r) {
                x[r] = __fmul_rn(x[r], ds[r]);
                delta = __fsub_rn(delta, __fmul_rn(ks[r], x[r]));
            }
#pragma unroll
            for (int r = 0; r < DIM; ++r) {
                x[r] = __fadd_rn(x[r], __fmul_rn(__fmul_rn(bh, ks[r]), delta));
                o = __fadd_rn(o, __fmul_rn(qs[r], x[r]));
                if (last_tok) col[(int64_t)r * DIM] = x[r];
            }
        } else {
            for (int r = 0; r < dim; ++r) {
                const float xr = __fmul_rn(col[(int64_t)r * dim], ds[r]);
                col[(int64_t)r * dim] = xr;
                delta = __fsub_rn(delta, __fmul_rn(ks[r], xr));
            }
            for (int r = 0; r < dim; ++r) {
                const float xr = __fadd_rn(col[(int64_t)r * dim], __fmul_rn(__fmul_rn(bh, ks[r]), delta));
                o = __fadd_rn(o, __fmul_rn(qs[r], xr));
                col[(int64_t)r * dim] = xr;
            }
        }
    }
    __syncthreads();            // qs is free: it now holds o for the head's RMS
    if (active) qs[c] = o;
    __syncthreads();
    if (warp == 0) {
        const float ss = __fdiv_rn(warp_sumsq(qs, dim, lane), (float)dim);
        if (lane == 0) red[2] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ss, a.rms_eps)));
    }
    __syncthreads();
    if (active) a.o[tt * a.ld_o + i] = __fmul_rn(__fmul_rn(__fmul_rn(o, red[2]), onv), g2v);
    __syncthreads();            // qs, ks, ds and red are rewritten by the next position
    }
}

// ---------------------------------------------------------------- a run of positions as three launches
// Of a position's work only the recurrence (decay, delta, update, output) depends on the position before it.  For a run
// of n positions (prefill) the rest is done for all positions side by side:
//   kda_run_pre_kernel  (heads x n CTAs): conv + SiLU of q, k, v (position t reads the rows t-1 .. t-(kconv-1) of this call,
//       or the layer's window for what came before it), the decay exp(g), the two sigmoids, the per-head L2 norms of q, k;
//   kda_run_rec_kernel  (heads CTAs): the state column in registers from position to position, the position's q, k and
//       decay vectors double-buffered in shared memory (cp.async one position ahead), two passes per position;
//   kda_run_post_kernel (heads x n CTAs): the head's output RMS norm, o_norm and the gate; the last kconv-1 rows become
//       the layer's conv window.
// Every value is formed by the expressions of kda_step_kernel in the same order, so the bits are those of n single steps.
struct KdaRun {
    float *qn, *kn, *vv, *ds, *g2s, *oraw;   // [n][heads * dim]
    float *bhs;                              // [n][heads]
};
__device__ __forceinline__ float kda_run_conv(const float *__restrict__ w, const float *__restrict__ win, const float *__restrict__ rows, int64_t ld,
                                              int64_t proj, int64_t i, int kconv, int t) {
    float acc = 0.0f;
    for (int j = 0; j < kconv - 1; ++j) {
        const int p = t - (kconv - 1) + j;                       // the position whose raw input weight j multiplies
        const float old = p >= 0 ? rows[(int64_t)p * ld + i] : win[(int64_t)(t + j) * proj + i];
        acc = __fadd_rn(acc, __fmul_rn(w[i * kconv + j], old));
    }
    acc = __fadd_rn(acc, __fmul_rn(w[i * kconv + kconv - 1], rows[(int64_t)t * ld + i]));
    return __fmul_rn(acc, sigmoid_cr(acc));
}
__global__ void __launch_bounds__(256) kda_run_pre_kernel(KdaArgs a, KdaRun r) {
    extern __shared__ float sm[];
    const int dim = a.dim;
    float *qs = sm, *ks = sm + dim, *red = sm + 2 * dim;
    const int h = blockIdx.x, t = blockIdx.y, c = threadIdx.x, lane = c & 31, warp = c >> 5, nwarps = blockDim.x >> 5;
    const bool active = c < dim;
    const int64_t proj = (int64_t)a.heads * dim, i = (int64_t)h * dim + c, row = (int64_t)t * proj + i;
    const int64_t wq = 0, wk = proj * a.kconv, wv = 2 * proj * a.kconv;
    const int64_t cq = 0, ck = (int64_t)(a.kconv - 1) * proj, cv = 2 * (int64_t)(a.kconv - 1) * proj;
    if (active) {
        qs[c] = kda_run_conv(a.conv_w + wq, a.conv + cq, a.q_raw, a.ld_x, proj, i, a.kconv, t);
        ks[c] = kda_run_conv(a.conv_w + wk, a.conv + ck, a.k_raw, a.ld_x, proj, i, a.kconv, t);
        r.vv[row] = kda_run_conv(a.conv_w + wv, a.conv + cv, a.v_raw, a.ld_x, proj, i, a.kconv, t);
        const float glow = a.g_low[(int64_t)t * a.ld_g + i], dtb = a.dt_bias[i], alog = a.a_log[c];
        const float g = __fmul_rn(a.gate_lb, sigmoid_cr(__fmul_rn(exp_cr(alog), __fadd_rn(glow, dtb))));
        r.ds[row] = exp_cr(g);
        r.g2s[row] = sigmoid_cr(a.g2[(int64_t)t * a.ld_x + i]);
        if (c == 0) r.bhs[(int64_t)t * a.heads + h] = sigmoid_cr(a.beta_raw[(int64_t)t * a.ld_x + h]);
    }
    __syncthreads();
    if (warp == 0) {
        const float n2 = warp_sumsq(qs, dim, lane);
        if (lane == 0) red[0] = __fdiv_rn(a.q_scale, fmaxf(__fsqrt_rn(n2), 1e-12f));
    }
    if (warp == nwarps - 1) {
        const float n2 = warp_sumsq(ks, dim, lane);
        if (lane == 0) red[1] = __fdiv_rn(1.0f, fmaxf(__fsqrt_rn(n2), 1e-12f));
    }
    __syncthreads();
    if (active) {
        r.qn[row] = __fmul_rn(qs[c], red[0]);
        r.kn[row] = __fmul_rn(ks[c], red[1]);
    }
}
template <int DIM>
__global__ void __launch_bounds__(DIM) kda_run_rec_kernel(KdaRun r, float *__restrict__ s, int heads, int n_tok) {
    __shared__ float buf[2][3][DIM];                 // q, k, decay of a position, two positions
    const int h = blockIdx.x, c = threadIdx.x;
    const int64_t proj = (int64_t)heads * DIM, i = (int64_t)h * DIM + c;
    float *col = s + (int64_t)h * DIM * DIM + c;
    auto fetch = [&](int t) {
        float (*b)[DIM] = buf[t & 1];
        const int64_t row = (int64_t)t * proj + i;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&b[0][c])), "l"(r.qn + row) : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&b[1][c])), "l"(r.kn + row) : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(&b[2][c])), "l"(r.ds + row) : "memory");
    };
    fetch(0);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    float x[DIM];
#pragma unroll
    for (int q = 0; q < DIM; ++q) x[q] = col[(int64_t)q * DIM];
    float vv = r.vv[i], bh = r.bhs[h];
    for (int t = 0; t < n_tok; ++t) {
        if (t + 1 < n_tok) fetch(t + 1);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        float vv_next = 0.0f, bh_next = 0.0f;
        if (t + 1 < n_tok) { vv_next = r.vv[(int64_t)(t + 1) * proj + i]; bh_next = r.bhs[(int64_t)(t + 1) * heads + h]; }
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        __syncthreads();
        const float *qs = buf[t & 1][0], *ks = buf[t & 1][1], *ds = buf[t & 1][2];
        float delta = vv, o = 0.0f;
#pragma unroll
        for (int q = 0; q < DIM; ++q) {
            x[q] = __fmul_rn(x[q], ds[q]);
            delta = __fsub_rn(delta, __fmul_rn(ks[q], x[q]));
        }
#pragma unroll
        for (int q = 0; q < DIM; ++q) {
            x[q] = __fadd_rn(x[q], __fmul_rn(__fmul_rn(bh, ks[q]), delta));
            o = __fadd_rn(o, __fmul_rn(qs[q], x[q]));
        }
        r.oraw[(int64_t)t * proj + i] = o;
        vv = vv_next; bh = bh_next;
        __syncthreads();            // this position's vectors may be overwritten by the fetch after next
    }
#pragma unroll
    for (int q = 0; q < DIM; ++q) col[(int64_t)q * DIM] = x[q];
}
__global__ void __launch_bounds__(256) kda_run_post_kernel(KdaArgs a, KdaRun r) {
    extern __shared__ float sm[];
    const int dim = a.dim;
    float *qs = sm, *red = sm + dim;
    const int h = blockIdx.x, t = blockIdx.y, c = threadIdx.x, lane = c & 31, warp = c >> 5;
    const bool active = c < dim;
    const int64_t proj = (int64_t)a.heads * dim, i = (int64_t)h * dim + c, row = (int64_t)t * proj + i;
    float o = 0.0f;
    if (active) { o = r.oraw[row]; qs[c] = o; }
    __syncthreads();
    if (warp == 0) {
        const float ss = __fdiv_rn(warp_sumsq(qs, dim, lane), (float)dim);
        if (lane == 0) red[0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ss, a.rms_eps)));
    }
    __syncthreads();
    if (!active) return;
    a.o[(int64_t)t * a.ld_o + i] = __fmul_rn(__fmul_rn(__fmul_rn(o, red[0]), a.o_norm[c]), r.g2s[row]);
    // the layer's conv window after the run: the raw inputs of the last kconv - 1 positions, oldest first
    const int j = t - (a.n_tok - (a.kconv - 1));
    if (j >= 0) {
        const int64_t w = (int64_t)j * proj + i, cq = 0, ck = (int64_t)(a.kconv - 1) * proj, cv = 2 * (int64_t)(a.kconv - 1) * proj;
        a.conv[cq + w] = a.q_raw[(int64_t)t * a.ld_x + i];
        a.conv[ck + w] = a.k_raw[(int64_t)t * a.ld_x + i];
        a.conv[cv + w] = a.v_raw[(int64_t)t * a.ld_x + i];
    }
}

// The same step with the head's S [dim][dim] staged in shared memory by cp.async at kernel start (dim % 4 == 0,
// dim <= 224): both passes become short loops that stay in the instruction cache, the column is read from shared
// memory twice (conflict-free: consecutive threads, consecutive words) and written to global memory once.  The
// decayed value x * decay is formed twice with the same operands, so the bits equal the register form's.
template <int KC>
__global__ void __launch_bounds__(256) kda_step_smem_kernel(KdaArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int dim = a.dim;
    float *xs = sm, *qs = xs + (size_t)dim * dim, *ks = qs + dim, *ds = ks + dim, *bks = ds + dim, *red = bks + dim;
    const int h = blockIdx.x, c = threadIdx.x, lane = c & 31, warp = c >> 5, nwarps = blockDim.x >> 5;
    const bool active = c < dim;
    const int64_t proj = (int64_t)a.heads * dim, i = (int64_t)h * dim + c;
    const int64_t wq = 0, wk = proj * a.kconv, wv = 2 * proj * a.kconv;
    const int64_t cq = 0, ck = (int64_t)(a.kconv - 1) * proj, cv = 2 * (int64_t)(a.kconv - 1) * proj;
    float *S = a.s + (int64_t)h * dim * dim;
    for (int idx = c; idx < dim * dim / 4; idx += blockDim.x) mkf::cp16(xs + idx * 4, S + idx * 4);
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    float vv = 0.0f, g2v = 0.0f, onv = 0.0f, bh = 0.0f;
    if (active) {
        float glow, dtb, alog;
        ConvIn<KC> iq, ik, iv;
        if constexpr (KC > 0) {
            iq.load(a.conv_w + wq, a.conv + cq, proj, i, a.q_raw);
            ik.load(a.conv_w + wk, a.conv + ck, proj, i, a.k_raw);
            iv.load(a.conv_w + wv, a.conv + cv, proj, i, a.v_raw);
        }
        glow = a.g_low[i]; dtb = a.dt_bias[i]; alog = a.a_log[c];
        g2v = a.g2[i]; onv = a.o_norm[c]; bh = a.beta_raw[h];
        if constexpr (KC > 0) {
            qs[c] = iq.apply(a.conv + cq, proj, i);
            ks[c] = ik.apply(a.conv + ck, proj, i);
            vv = iv.apply(a.conv + cv, proj, i);
        } else {
            qs[c] = conv_channel(a.conv_w + wq, a.conv + cq, proj, i, a.kconv, a.q_raw[i]);
            ks[c] = conv_channel(a.conv_w + wk, a.conv + ck, proj, i, a.kconv, a.k_raw[i]);
            vv = conv_channel(a.conv_w + wv, a.conv + cv, proj, i, a.kconv, a.v_raw[i]);
        }
        const float g = __fmul_rn(a.gate_lb, sigmoid_cr(__fmul_rn(exp_cr(alog), __fadd_rn(glow, dtb))));
        ds[c] = exp_cr(g);
        bh = sigmoid_cr(bh);
        g2v = sigmoid_cr(g2v);
    }
    __syncthreads();
    if (warp == 0) {
        const float n2 = warp_sumsq(qs, dim, lane);
        if (lane == 0) red[0] = __fdiv_rn(a.q_scale, fmaxf(__fsqrt_rn(n2), 1e-12f));
    }
    if (warp == nwarps - 1) {
        const float n2 = warp_sumsq(ks, dim, lane);
        if (lane == 0) red[1] = __fdiv_rn(1.0f, fmaxf(__fsqrt_rn(n2), 1e-12f));
    }
    __syncthreads();
    if (active) {
        qs[c] = __fmul_rn(qs[c], red[0]);
        const float kn = __fmul_rn(ks[c], red[1]);
        ks[c] = kn;
        bks[c] = __fmul_rn(bh, kn);     // beta * k[r], the same for every column
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    float o = 0.0f;
    if (active) {
        float delta = vv;
        const float *xc = xs + c;
#pragma unroll 4
        for (int r = 0; r < dim; r += 4) {
            const float4 d4 = *reinterpret_cast<const float4 *>(ds + r), k4 = *reinterpret_cast<const float4 *>(ks + r);
            delta = __fsub_rn(delta, __fmul_rn(k4.x, __fmul_rn(xc[(r + 0) * dim], d4.x)));
            delta = __fsub_rn(delta, __fmul_rn(k4.y, __fmul_rn(xc[(r + 1) * dim], d4.y)));
            delta = __fsub_rn(delta, __fmul_rn(k4.z, __fmul_rn(xc[(r + 2) * dim], d4.z)));
            delta = __fsub_rn(delta, __fmul_rn(k4.w, __fmul_rn(xc[(r + 3) * dim], d4.w)));
        }
        float *col = S + c;
#pragma unroll 2
        for (int r = 0; r < dim; r += 4) {
            const float4 d4 = *reinterpret_cast<const float4 *>(ds + r), b4 = *reinterpret_cast<const float4 *>(bks + r);
            const float4 q4 = *reinterpret_cast<const float4 *>(qs + r);
            const float x0 = __fadd_rn(__fmul_rn(xc[(r + 0) * dim], d4.x), __fmul_rn(b4.x, delta));
            const float x1 = __fadd_rn(__fmul_rn(xc[(r + 1) * dim], d4.y), __fmul_rn(b4.y, delta));
            const float x2 = __fadd_rn(__fmul_rn(xc[(r + 2) * dim], d4.z), __fmul_rn(b4.z, delta));
            const float x3 = __fadd_rn(__fmul_rn(xc[(r + 3) * dim], d4.w), __fmul_rn(b4.w, delta));
            o = __fadd_rn(o, __fmul_rn(q4.x, x0));
            o = __fadd_rn(o, __fmul_rn(q4.y, x1));
            o = __fadd_rn(o, __fmul_rn(q4.z, x2));
            o = __fadd_rn(o, __fmul_rn(q4.w, x3));
            col[(int64_t)(r + 0) * dim] = x0;
            col[(int64_t)(r + 1) * dim] = x1;
            col[(int64_t)(r + 2) * dim] = x2;
            col[(int64_t)(r + 3) * dim] = x3;
        }
    }
    __syncthreads();
    if (active) qs[c] = o;
    __syncthreads();
    if (warp == 0) {
        const float ss = __fdiv_rn(warp_sumsq(qs, dim, lane), (float)dim);
        if (lane == 0) red[2] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ss, a.rms_eps)));
    }
    __syncthreads();
    if (active) a.o[i] = __fmul_rn(__fmul_rn(__fmul_rn(o, red[2]), onv), g2v);
}

// ---- AttnRes: scores (one warp per row: blocks 0..b-1, then the prefix), then softmax + mix
__global__ void __launch_bounds__(32) attn_res_score_kernel(const float *__restrict__ prefix, const float *__restrict__ blocks,
                                                           int64_t ld, int b, const float *__restrict__ w, int d, float eps,
                                                           float *__restrict__ scores) {
    const int row = blockIdx.x, lane = threadIdx.x, j = lane & 7, full = d & ~7;
    const float *v = row < b ? blocks + (int64_t)row * ld : prefix;
    float acc = 0.0f;
    for (int c = 0; c < full; c += 8) acc = __fadd_rn(acc, __fmul_rn(v[c + j], v[c + j]));
    float ss = mkf::reduce8(acc, lane);
    for (int c = full; c < d; ++c) ss = __fadd_rn(ss, __fmul_rn(v[c], v[c]));
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)d), eps)));
    acc = 0.0f;
    for (int c = 0; c < full; c += 8) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(v[c + j], inv), w[c + j]));
    float sc = mkf::reduce8(acc, lane);
    for (int c = full; c < d; ++c) sc = __fadd_rn(sc, __fmul_rn(__fmul_rn(v[c], inv), w[c]));
    if (lane == 0) scores[row] = sc;
}
__global__ void __launch_bounds__(256) attn_res_mix_kernel(const float *__restrict__ prefix, const float *__restrict__ blocks, int64_t ld,
                                                          int b, int d, const float *__restrict__ scores, float *__restrict__ out) {
    extern __shared__ float p[]; // b + 1 probabilities
    if (threadIdx.x == 0) {      // the engine's sequential softmax (b + 1 is a handful of values)
        float m = -INFINITY;
        for (int i = 0; i <= b; ++i) m = fmaxf(m, scores[i]);
        float z = 0.0f;
        for (int i = 0; i <= b; ++i) {
            p[i] = exp_cr(__fsub_rn(scores[i], m));
            z = __fadd_rn(z, p[i]);
        }
        for (int i = 0; i <= b; ++i) p[i] = __fdiv_rn(p[i], z);
    }
    __syncthreads();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= d) return;
    float o = 0.0f;
    for (int i = 0; i < b; ++i) o = __fadd_rn(o, __fmul_rn(p[i], blocks[(int64_t)i * ld + j]));
    out[j] = __fadd_rn(o, __fmul_rn(p[b], prefix[j]));
}
} // namespace

// ====================================================================== C ABI
extern "C" int32_t mk_kda_create(mk_ctx *ctx, const mk_kda_desc *d, mk_kda **out) {
    MK_CHECK_ARG(ctx != nullptr && d != nullptr && out != nullptr, "NULL argument");
    *out = nullptr;
    MK_CHECK_ARG(d->heads >= 1 && d->dim >= 1 && d->dim <= 1024 && d->kconv >= 2 && d->kconv <= 16,
                 "heads >= 1, dim in [1, 1024] and kconv in [2, 16] required");
    MK_CHECK_ARG(d->q_conv && d->k_conv && d->v_conv && d->a_log && d->dt_bias && d->o_norm, "NULL parameter array");
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_kda *k = new (std::nothrow) mk_kda();
    if (!k) return MK_ERR_OOM;
    memset(k, 0, sizeof(*k));
    k->heads = d->heads;
    k->dim = d->dim;
    k->kconv = d->kconv;
    k->gate_lb = d->gate_lb;
    k->rms_eps = d->rms_eps;
    k->q_scale = powf((float)d->dim, -0.5f); // (kda_dim as f32).powf(-0.5), src/model.rs:1216
    const size_t proj = (size_t)d->heads * d->dim, cw = proj * d->kconv * 4;
    const size_t win = (size_t)(d->kconv - 1) * proj * 4, sb = (size_t)d->heads * d->dim * d->dim * 4;
    cudaError_t e = cudaMalloc(&k->conv_w, 3 * cw);
    if (e == cudaSuccess) e = cudaMalloc(&k->a_log, (size_t)d->dim * 4);
    if (e == cudaSuccess) e = cudaMalloc(&k->dt_bias, proj * 4);
    if (e == cudaSuccess) e = cudaMalloc(&k->o_norm, (size_t)d->dim * 4);
    if (e == cudaSuccess) e = cudaMalloc(&k->conv, 3 * win + 16);
    if (e == cudaSuccess) e = cudaMalloc(&k->s, sb);
    const float *cws[3] = {d->q_conv, d->k_conv, d->v_conv};
    for (int t = 0; t < 3 && e == cudaSuccess; ++t)
        e = cudaMemcpyAsync((char *)k->conv_w + t * cw, cws[t], cw, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(k->a_log, d->a_log, (size_t)d->dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(k->dt_bias, d->dt_bias, proj * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(k->o_norm, d->o_norm, (size_t)d->dim * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(k->conv, 0, 3 * win + 16, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(k->s, 0, sb, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        mk_set_error("mk_kda_create: %s", cudaGetErrorString(e));
        mk_kda_free(ctx, k);
        return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    *out = k;
    return MK_OK;
}

extern "C" void mk_kda_free(mk_ctx *ctx, mk_kda *k) {
    if (!k) return;
    if (ctx) cudaSetDevice(ctx->device);
    float *bufs[6] = {k->conv_w, k->a_log, k->dt_bias, k->o_norm, k->conv, k->s};
    for (float *b : bufs)
        if (b) cudaFree(b);
    delete k;
}

extern "C" int32_t mk_kda_reset(mk_ctx *ctx, mk_kda *k) {
    MK_CHECK_ARG(ctx != nullptr && k != nullptr, "NULL argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const size_t proj = (size_t)k->heads * k->dim;
    MK_CUDA(cudaMemsetAsync(k->conv, 0, 3 * (size_t)(k->kconv - 1) * proj * 4 + 16, ctx->stream));
    MK_CUDA(cudaMemsetAsync(k->s, 0, (size_t)k->heads * k->dim * k->dim * 4, ctx->stream));
    return MK_OK;
}

// direction 0: device -> host (export), 1: host -> device (import)
static int32_t kda_state_copy(mk_ctx *ctx, mk_kda *k, float *s, float *conv, int to_device) {
    MK_CHECK_ARG(ctx != nullptr && k != nullptr && s != nullptr && conv != nullptr, "NULL argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const size_t proj = (size_t)k->heads * k->dim, win = 3 * (size_t)(k->kconv - 1) * proj * 4;
    const size_t sb = (size_t)k->heads * k->dim * k->dim * 4;
    if (to_device) {
        MK_CUDA(cudaMemcpyAsync(k->s, s, sb, cudaMemcpyHostToDevice, ctx->stream));
        if (win) MK_CUDA(cudaMemcpyAsync(k->conv, conv, win, cudaMemcpyHostToDevice, ctx->stream));
    } else {
        MK_CUDA(cudaMemcpyAsync(s, k->s, sb, cudaMemcpyDeviceToHost, ctx->stream));
        if (win) MK_CUDA(cudaMemcpyAsync(conv, k->conv, win, cudaMemcpyDeviceToHost, ctx->stream));
    }
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}
extern "C" int32_t mk_kda_export(mk_ctx *ctx, mk_kda *k, float *s, float *conv) { return kda_state_copy(ctx, k, s, conv, 0); }
extern "C" int32_t mk_kda_import(mk_ctx *ctx, mk_kda *k, const float *s, const float *conv) {
    return kda_state_copy(ctx, k, const_cast<float *>(s), const_cast<float *>(conv), 1);
}

static int32_t kda_steps(mk_ctx *ctx, mk_kda *k, int n_tok, const float *q_raw, const float *k_raw, const float *v_raw, const float *g_low,
                         const float *beta_raw, const float *g2, float *o, int64_t ld_x, int64_t ld_g, int64_t ld_o);
extern "C" int32_t mk_kda_step_dev(mk_ctx *ctx, mk_kda *k, const float *q_raw, const float *k_raw, const float *v_raw,
                                   const float *g_low, const float *beta_raw, const float *g2, float *o) {
    return kda_steps(ctx, k, 1, q_raw, k_raw, v_raw, g_low, beta_raw, g2, o, 0, 0, 0);
}
extern "C" int32_t mk_kda_steps_dev(mk_ctx *ctx, mk_kda *k, int32_t n_tok, const float *q_raw, const float *k_raw, const float *v_raw,
                                    const float *g_low, const float *beta_raw, const float *g2, float *o, int64_t ld_x, int64_t ld_g, int64_t ld_o) {
    MK_CHECK_ARG(n_tok >= 1, "n_tok >= 1 required");
    return kda_steps(ctx, k, n_tok, q_raw, k_raw, v_raw, g_low, beta_raw, g2, o, ld_x, ld_g, ld_o);
}
static int32_t kda_steps(mk_ctx *ctx, mk_kda *k, int n_tok, const float *q_raw, const float *k_raw, const float *v_raw, const float *g_low,
                         const float *beta_raw, const float *g2, float *o, int64_t ld_x, int64_t ld_g, int64_t ld_o) {
    MK_CHECK_ARG(ctx != nullptr && k != nullptr, "NULL argument");
    MK_CHECK_ARG(q_raw && k_raw && v_raw && g_low && beta_raw && g2 && o, "NULL device pointer");
    MK_CUDA(cudaSetDevice(ctx->device));
    const bool reg_form = !((ctx->kda_smem || !(k->dim == 64 || k->dim == 128)) && k->dim % 4 == 0 && k->dim >= 32 && k->dim <= 224);
    if (n_tok > 1 && !reg_form) {
        // the shared-memory form takes one position per launch
        for (int t = 0; t < n_tok; ++t) {
            const int32_t rc = kda_steps(ctx, k, 1, q_raw + t * ld_x, k_raw + t * ld_x, v_raw + t * ld_x, g_low + t * ld_g, beta_raw + t * ld_x,
                                         g2 + t * ld_x, o + t * ld_o, 0, 0, 0);
            if (rc != MK_OK) return rc;
        }
        return MK_OK;
    }
    KdaArgs a;
    a.n_tok = n_tok; a.ld_x = ld_x; a.ld_g = ld_g; a.ld_o = ld_o;
    a.q_raw = q_raw; a.k_raw = k_raw; a.v_raw = v_raw; a.g_low = g_low; a.beta_raw = beta_raw; a.g2 = g2;
    a.conv_w = k->conv_w; a.a_log = k->a_log; a.dt_bias = k->dt_bias; a.o_norm = k->o_norm;
    a.conv = k->conv; a.s = k->s; a.o = o;
    a.heads = k->heads; a.dim = k->dim; a.kconv = k->kconv;
    a.gate_lb = k->gate_lb; a.rms_eps = k->rms_eps; a.q_scale = k->q_scale;
    const size_t smem = (size_t)(3 * k->dim + 4) * sizeof(float);
    if (n_tok >= 4 && n_tok >= k->kconv - 1 && k->kconv >= 2 && (k->dim == 64 || k->dim == 128) && !ctx->kda_smem) {
        // a run of positions: everything but the recurrence for all positions side by side (three launches)
        const size_t per = (size_t)n_tok * k->heads * k->dim;
        int32_t rc = mk_ws_reserve(ctx, (6 * per + (size_t)n_tok * k->heads) * sizeof(float) + 256);
        if (rc != MK_OK) return rc;
        KdaRun r;
        float *w = (float *)ctx->ws;
        r.qn = w; r.kn = w + per; r.vv = w + 2 * per; r.ds = w + 3 * per; r.g2s = w + 4 * per; r.oraw = w + 5 * per; r.bhs = w + 6 * per;
        mk_prof_scope prof(ctx, MK_PROF_OTHER);
        const unsigned threads = (unsigned)mk_align_up(k->dim, 32);
        kda_run_pre_kernel<<<dim3((unsigned)k->heads, (unsigned)n_tok), threads, (size_t)(2 * k->dim + 4) * sizeof(float), ctx->stream>>>(a, r);
        if (k->dim == 128) kda_run_rec_kernel<128><<<k->heads, 128, 0, ctx->stream>>>(r, k->s, k->heads, n_tok);
        else kda_run_rec_kernel<64><<<k->heads, 64, 0, ctx->stream>>>(r, k->s, k->heads, n_tok);
        kda_run_post_kernel<<<dim3((unsigned)k->heads, (unsigned)n_tok), threads, (size_t)(k->dim + 4) * sizeof(float), ctx->stream>>>(a, r);
        ctx->launches += 3;
        MK_CUDA(cudaGetLastError());
        return MK_OK;
    }
    mk_prof_scope prof(ctx, MK_PROF_OTHER);
    const bool kc4 = k->kconv == 4;
    const size_t smem_s = ((size_t)k->dim * k->dim + 4 * (size_t)k->dim + 4) * sizeof(float);
    const bool reg_dim = k->dim == 64 || k->dim == 128;
    if ((ctx->kda_smem || !reg_dim) && k->dim % 4 == 0 && k->dim >= 32 && k->dim <= 224) {
        static mk_once_per_device attr;
        if (attr.pending(ctx->device)) {
            MK_CUDA(cudaFuncSetAttribute(kda_step_smem_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            MK_CUDA(cudaFuncSetAttribute(kda_step_smem_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            attr.mark(ctx->device);
        }
        const unsigned threads = (unsigned)mk_align_up(k->dim, 32);
        if (kc4) kda_step_smem_kernel<4><<<k->heads, threads, smem_s, ctx->stream>>>(a);
        else kda_step_smem_kernel<0><<<k->heads, threads, smem_s, ctx->stream>>>(a);
    } else if (k->dim == 128 && kc4)
        kda_step_kernel<128, 4><<<k->heads, 128, smem, ctx->stream>>>(a);
    else if (k->dim == 128)
        kda_step_kernel<128, 0><<<k->heads, 128, smem, ctx->stream>>>(a);
    else if (k->dim == 64 && kc4)
        kda_step_kernel<64, 4><<<k->heads, 64, smem, ctx->stream>>>(a);
    else if (k->dim == 64)
        kda_step_kernel<64, 0><<<k->heads, 64, smem, ctx->stream>>>(a);
    else if (kc4)
        kda_step_kernel<0, 4><<<k->heads, (unsigned)mk_align_up(k->dim, 32), smem, ctx->stream>>>(a);
    else
        kda_step_kernel<0, 0><<<k->heads, (unsigned)mk_align_up(k->dim, 32), smem, ctx->stream>>>(a);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

extern "C" int32_t mk_attn_res_dev(mk_ctx *ctx, const float *prefix, const float *blocks, int64_t ld, int32_t b, const float *w,
                                   int32_t d, float eps, float *out) {
    MK_CHECK_ARG(ctx != nullptr && prefix != nullptr && w != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(b >= 0 && b <= 4095 && d >= 1 && (b == 0 || (blocks != nullptr && ld >= d)), "0 <= b <= 4095, d >= 1, ld >= d required");
    MK_CUDA(cudaSetDevice(ctx->device));
    int32_t rc = mk_ws_reserve(ctx, (size_t)(b + 1) * 4);
    if (rc != MK_OK) return rc;
    float *scores = (float *)ctx->ws;
    mk_prof_scope prof(ctx, MK_PROF_OTHER);
    attn_res_score_kernel<<<b + 1, 32, 0, ctx->stream>>>(prefix, blocks, ld, b, w, d, eps, scores);
    attn_res_mix_kernel<<<(unsigned)mk_ceil_div(d, 256), 256, (size_t)(b + 1) * 4, ctx->stream>>>(prefix, blocks, ld, b, d, scores, out);
    ctx->launches += 2;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}
