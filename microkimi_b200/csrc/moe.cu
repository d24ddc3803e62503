// MoE layer on the GPU: router, top-k, expert grouping, grouped MXFP4 expert
// matvecs with fused activation, fixed-order combine (sm_100a).
//
// Reference: moe_forward (src/model.rs:2150-2380) for the router and the slot-order
// combination, ds_moe / expert_forward (src/deepseek.rs:1038-1108, 74-95) for the
// expert body (SwiGLU with clamp, routing weight folded in before w2), and
// matvec_packed_nt (src/model.rs:2412-2447) for what batching means: every
// (token, expert) result is what a single-token call would give.
//
// Launches per layer call: router logits, activation quantization, top-k (+ pair
// list), plan (group pairs by expert), gate/up (+ activation + q8 of the
// activation), down, combine.  Up to 16 tokens the first four are ONE launch
// (moe_router_fused_kernel), 4 launches per layer call in all.
#include <cuda.h>

#include "qgemv_core.cuh"
#include "f32gemv.cuh"

using namespace mkq;

struct mk_moe {
    int n_experts, top_k, d, inter, activation;   // d: width the experts work on (the latent width when there is one)
    int dx;                        // model width: router rows, layer input and output
    int router_kind;               // MK_ROUTER_*
    float route_scale;
    float limit;
    bool has_router, has_shared;
    bool tc;                       // MK_ACT_FP4X6: calls of >= 32 rows run the experts on the block-scaled tcgen05 path
    void *tmaps;                   // device [(n_experts+1)*3] tensor maps of the row-major copies below
    int32_t *tc_rows_x, *tc_rows_p; // [max_items][16] token rows / pair ids per work item of that path
    uint8_t *rm_vals, *rm_atoms;   // that path's own copy of the experts: blocked nibbles and scale atoms (moe_tc.cuh), matrix i at i * rm_vstride / rm_astride
    int64_t rm_vstride, rm_astride;
    uint8_t *xl, *xsf, *actl, *actsf;   // its activation limbs: tokens [3][rows][d] + scales, expert activations [3][pairs][inter] + scales
    bool strict;                   // MK_ACT_STRICT: expert sums in the CPU's order (one accumulator, ascending blocks, no K split)
    float *gate_w, *gate_b;        // device
    // K3 latent MoE (src/model.rs:2202-2380); the f32 matrices belong to the caller's handles
    int latent;                    // routed_hidden, 0 = none
    const float *routed_down, *routed_up; // device f32 [latent, dx], [dx, latent]
    float *routed_norm;            // device f32 [latent] (owned)
    float rms_eps;
    const float *sh_gate, *sh_down, *sh_up; // f32 shared expert [si, dx], [dx, si], [si, dx]; nullptr = none
    int shared_inter;
    bool stack3;                   // routed_down, shared gate and shared up are one contiguous [latent + 2 si, dx] matrix
    float *stk;                    // [latent + 2 si]: their products with one token (decode fast path)
    float *sh_out;                 // [cap_rows][dx] shared expert output when it is not accumulated into the layer output
    float *lat_h, *lat_y, *lat_yn; // [cap_rows][latent]: routed_down x, weighted expert sum, its rmsnorm
    float *sh_a, *sh_u;            // [cap_rows][shared_inter]
    const void **wv, **wsc;        // device tables [(n_experts+1)*3] of tiled values / scales (nullptr = not resident)
    int64_t nbp_d, nbp_i;          // padded block counts of d and inter
    // workspace, sized for cap_rows activation rows and cap_pairs pairs
    int cap_rows, cap_pairs;
    float *logits;                 // [3][cap_rows][n_experts]: logits, scores, selection keys
    int32_t *ids;                  // [rows][top_k]
    float *wts;                    // [rows][top_k]
    int8_t *xq; float *xs;         // q8 activations of the rows
    int32_t *pair_row, *pair_expert; float *pair_weight;   // forward path pair list
    int32_t *sorted;               // pair ids grouped by expert
    int32_t *items;                // [max_items][3] = expert, offset into sorted, count (<= 8)
    int32_t *n_items;              // device scalar
    int32_t *counter;              // device scalar, 0 between calls (fused router kernel)
    int8_t *actq; float *acts;     // q8 of the expert activations, per pair
    float *outs;                   // [pairs][d]
    int max_items;
};

// Expert parallelism over the GPUs of one node for decode (token rows replicated on every rank, <= 16 rows):
// every rank routes all rows (bit-identical ids), runs the pairs whose expert it holds, pushes their
// output rows into the (token, slot) table of every other rank (peer memory), and combines the full table.
// Buffer per rank (cudaMalloc, shared by CUDA IPC): [flags: 2 parities x 8 ranks u32, 256 B]
// [outs: 2 parities x max_tokens * slots x d f32].
struct mk_moe_ep {
    int rank, world, max_tokens, slots, d;
    size_t par_bytes, blob_bytes;
    void *blob;
    void *peer[8];
    void *absent;       // stand-in target for ranks that have not joined (all-zero handle): local scratch
    bool is_absent[8];
    bool connected;
    uint32_t step;      // host mirror of the device step count (counter[1]): picks the table parity of a call
    int32_t *n_local;   // device: pairs computed by this rank in the current call
    uint32_t *counter;  // device: [0] exchange kernel's finished CTAs, 0 between calls; [1] steps finished
};

// a recorded token replays `n` exchange steps that the host did not issue one by one: keep the mirror in step
uint32_t mk_moe_ep_steps(const mk_moe_ep *ep) { return ep->step; }
void mk_moe_ep_note_replay(mk_moe_ep *ep, uint32_t n) { ep->step += n; }

namespace {

// ------------------------------------------------------------------ router logits
// logits[t][e] = dot(gate_w[e], x[t]) in the engine's order (src/model.rs:63-82):
// 8 accumulators, element j of each 8-chunk into accumulator j with a separate
// multiply and add, then ((a0+a1)+(a2+a3))+(a4+a5))+(a6+a7), tail sequential.
// Every logits kernel also stores the score - MK_ROUTER_SIGMOID: 1/(1+exp(-l))
// (src/model.rs:2152-2156); MK_ROUTER_SQRT_SOFTPLUS: sqrt(softplus(l)), softplus = l above 20,
// else ln(1 + exp(l)) (src/deepseek.rs:29-32, 60-68) - and key = score + bias.  exp() and
// log() run in double and are rounded once, which agrees with a correctly rounded libm.
__device__ __forceinline__ void router_store(float *__restrict__ logits, float *__restrict__ score, float *__restrict__ key,
                                             const float *__restrict__ gate_b, int64_t at, int e, float l, int kind) {
    float sg;
    if (kind == MK_ROUTER_SQRT_SOFTPLUS) {
        const float sp = l > 20.0f ? l : (float)log((double)__fadd_rn(1.0f, (float)exp((double)l)));
        sg = __fsqrt_rn(sp);
    } else {
        const float ex = (float)exp((double)(-l));
        sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, ex));
    }
    logits[at] = l;
    score[at] = sg;
    key[at] = __fadd_rn(sg, gate_b ? gate_b[e] : 0.0f);
}

// Generic form (any d, any alignment): a warp = 4 experts (mkf::rows_dot).
template <int T>
__global__ void __launch_bounds__(256)
moe_router_logits_kernel(const float *__restrict__ gate_w, const float *__restrict__ gate_b, const float *__restrict__ x,
                         float *__restrict__ logits, float *__restrict__ score, float *__restrict__ key, int n_experts, int d,
                         int n_tokens, int kind) {
    const int warp_g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31, sub = lane >> 3, j = lane & 7;
    const int ewarps = (n_experts + 3) / 4;
    const int tile = warp_g / ewarps;
    const int e = (warp_g % ewarps) * 4 + sub;
    const int tok0 = tile * T;
    if (tok0 >= n_tokens) return;
    const bool ev = e < n_experts;
    float out[T];
    mkf::rows_dot<T>(gate_w + (size_t)(ev ? e : 0) * d, x, d, n_tokens, tok0, ev, lane, out);
#pragma unroll
    for (int t = 0; t < T; ++t)
        if (j == 0 && ev && tok0 + t < n_tokens) router_store(logits, score, key, gate_b, (int64_t)(tok0 + t) * n_experts + e, e, out[t], kind);
}

// Tiled form (mkf::tile_dot; d a multiple of 4, rows 16-byte aligned).  Two shapes: RtBig
// for throughput, RtSmall (<= 4 tokens) keeps a deeper queue of the router rows in flight
// because at small batches those come cold from HBM.
using RtBig = mkf::TileShape<2, 16, 256, 3>;
using RtSmall = mkf::TileShape<1, 4, 512, 6>;

template <class S>
__global__ void __launch_bounds__(256)
moe_router_tile_kernel(const float *__restrict__ gate_w, const float *__restrict__ gate_b, const float *__restrict__ x,
                       float *__restrict__ logits, float *__restrict__ score, float *__restrict__ key, int n_experts, int d,
                       int n_tokens, int kind) {
    extern __shared__ __align__(16) float rsm[];
    int e, tok;
    bool valid;
    const float l = mkf::tile_dot<S>(gate_w, x, n_experts, d, n_tokens, blockIdx.x * S::NE, blockIdx.y * S::NT, rsm, &e, &tok, &valid);
    if (valid) router_store(logits, score, key, gate_b, (int64_t)tok * n_experts + e, e, l, kind);
}


// The router's logits for many tokens: mkf::reg_tile_product (16 experts x 16 tokens per CTA of 128 threads, every pair the
// engine's dot()) with the router's epilogue.
using mkf::RG_TE;
using mkf::RG_TT;
using mkf::RG_THREADS;
using mkf::RG_SMEM;
__global__ void __launch_bounds__(RG_THREADS)
moe_router_gemm_kernel(const float *__restrict__ gate_w, const float *__restrict__ gate_b, const float *__restrict__ x,
                       float *__restrict__ logits, float *__restrict__ score, float *__restrict__ key, int n_experts, int d,
                       int n_tokens, int kind) {
    extern __shared__ __align__(16) float gsm[];
    mkf::reg_tile_product(gate_w, x, n_experts, d, n_tokens, blockIdx.x * RG_TE, blockIdx.y * RG_TT, gsm, [&](int e, int tok, float v) {
        router_store(logits, score, key, gate_b, (int64_t)tok * n_experts + e, e, v, kind);
    });
}

// ------------------------------------------------------------------ top-k
// One warp per token.  The top_k by (key descending, index ascending) in that order is
// what the engine's running selection ends with (src/model.rs:2157-2171); weights =
// score / (sum + 1e-20) with the sum taken in slot order (src/model.rs:2172-2173), or for
// MK_ROUTER_SQRT_SOFTPLUS score / sum * route_scale (src/deepseek.rs:51-56).
// kb: n_experts floats of shared memory owned by this warp.
__device__ __forceinline__ uint32_t float_order(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
// weights and pair list of a token from its picks (lane r holds the r-th pick)
__device__ __forceinline__ void topk_finish(const float *score, int n_experts, int top_k, int tok, int lane, int my_id, int32_t *__restrict__ ids,
                                            float *__restrict__ wts, int32_t *__restrict__ pair_row, int32_t *__restrict__ pair_expert,
                                            float *__restrict__ pair_weight, int shared_slot, int kind, float route_scale) {
    const float my_sc = lane < top_k ? __ldcg(score + (size_t)tok * n_experts + my_id) : 0.0f;
    float sumw = 0.0f;
    for (int r = 0; r < top_k; ++r) sumw = __fadd_rn(sumw, __shfl_sync(0xFFFFFFFFu, my_sc, r));
    if (kind != MK_ROUTER_SQRT_SOFTPLUS) sumw = __fadd_rn(sumw, 1e-20f);
    const int slots = top_k + (shared_slot ? 1 : 0);
    if (lane < top_k) {
        float w = __fdiv_rn(my_sc, sumw);
        if (kind == MK_ROUTER_SQRT_SOFTPLUS) w = __fmul_rn(w, route_scale);
        ids[(size_t)tok * top_k + lane] = my_id;
        wts[(size_t)tok * top_k + lane] = w;
        if (pair_row) {
            const int p = tok * slots + lane;
            pair_row[p] = tok;
            pair_expert[p] = my_id;
            pair_weight[p] = w;
        }
    }
    if (pair_row && shared_slot && lane == 31) {
        const int p = tok * slots + top_k;
        pair_row[p] = tok;
        pair_expert[p] = n_experts; // the shared expert, unweighted
        pair_weight[p] = 1.0f;
    }
}
__device__ __forceinline__ int topk_token(const float *score, const float *key, int n_experts, int top_k, int tok, int lane, float *kb,
                                           int32_t *__restrict__ ids, float *__restrict__ wts, int32_t *__restrict__ pair_row,
                                           int32_t *__restrict__ pair_expert, float *__restrict__ pair_weight, int shared_slot,
                                           int kind, float route_scale) {
    int my_id = 0;
    if (n_experts <= 32 * 32) {
        // Up to 1024 experts: lane l keeps keys l, l + 32, ... in registers and its own running maximum; a round is two
        // redux over the lanes' maxima, after which only the winner's registers change (every lane runs the same
        // predicated code).  Same order as below: larger key first, equal keys by ascending index.
        float kv[32];
#pragma unroll
        for (int s = 0; s < 32; ++s) {
            const int e = lane + 32 * s;
            kv[s] = e < n_experts ? __fadd_rn(__ldcg(key + (size_t)tok * n_experts + e), 0.0f) : -INFINITY; // -0 -> +0
        }
        for (int r = 0; r < top_k; ++r) {
            // tournament over the 32 slots (depth 5 instead of a chain of 31): the higher slot wins only with a larger key,
            // so the lowest index of the lane's maximum survives
            float tv[16];
            int ts[16];
#pragma unroll
            for (int s = 0; s < 16; ++s) {
                const bool hi = kv[2 * s + 1] > kv[2 * s];
                tv[s] = hi ? kv[2 * s + 1] : kv[2 * s];
                ts[s] = hi ? 2 * s + 1 : 2 * s;
            }
#pragma unroll
            for (int w = 8; w >= 1; w >>= 1) {
#pragma unroll
                for (int s = 0; s < w; ++s) {
                    const bool hi = tv[2 * s + 1] > tv[2 * s];
                    tv[s] = hi ? tv[2 * s + 1] : tv[2 * s];
                    ts[s] = hi ? ts[2 * s + 1] : ts[2 * s];
                }
            }
            const float bk = tv[0];
            const int bs = ts[0];
            const int bi = lane + 32 * bs;
            const uint32_t u = bi < n_experts ? float_order(bk) : 0u;
            const uint32_t gmax = __reduce_max_sync(0xFFFFFFFFu, u);
            int gi = __reduce_min_sync(0xFFFFFFFFu, (u == gmax) ? bi : 0x7FFFFFFF);
            if (gi == 0x7FFFFFFF) gi = 0;
            if (lane == r) my_id = gi;
            const int ws = (gi & 31) == lane ? (gi >> 5) : -1;  // taken; real keys are finite, so they always come first
#pragma unroll
            for (int s = 0; s < 32; ++s)
                if (s == ws) kv[s] = -INFINITY;
        }
    } else {
    for (int e = lane; e < n_experts; e += 32) kb[e] = __fadd_rn(__ldcg(key + (size_t)tok * n_experts + e), 0.0f); // -0 -> +0
    __syncwarp();
    for (int r = 0; r < top_k; ++r) {
        float bk = -INFINITY;
        int bi = 0x7FFFFFFF;
        for (int e = lane; e < n_experts; e += 32) {
            const float kv = kb[e];
            if (kv > bk || bi == 0x7FFFFFFF) { bk = kv; bi = e; } // ascending e: the lowest index of the lane's maximum
        }
        const uint32_t u = bi == 0x7FFFFFFF ? 0u : float_order(bk);
        const uint32_t gmax = __reduce_max_sync(0xFFFFFFFFu, u);
        int gi = __reduce_min_sync(0xFFFFFFFFu, (u == gmax) ? bi : 0x7FFFFFFF);
        if (gi == 0x7FFFFFFF) gi = 0;
        if (lane == r) my_id = gi;
        if (lane == 0) kb[gi] = -INFINITY; // taken; real keys are finite, so they always come first
        __syncwarp();
    }
    }
    topk_finish(score, n_experts, top_k, tok, lane, my_id, ids, wts, pair_row, pair_expert, pair_weight, shared_slot, kind, route_scale);
    return my_id;   // lane r: the r-th pick
}

__global__ void __launch_bounds__(128)
moe_topk_kernel(const float *__restrict__ score, const float *__restrict__ key, int n_experts, int top_k, int n_tokens,
                int32_t *__restrict__ ids, float *__restrict__ wts, int32_t *__restrict__ pair_row,
                int32_t *__restrict__ pair_expert, float *__restrict__ pair_weight, int shared_slot, int kind,
                float route_scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tok = blockIdx.x * (blockDim.x >> 5) + warp;
    if (tok >= n_tokens) return;
    topk_token(score, key, n_experts, top_k, tok, lane, sm + (size_t)warp * n_experts, ids, wts, pair_row, pair_expert, pair_weight,
               shared_slot, kind, route_scale);
}

// Grouping of a SMALL pair list by one CTA without per-expert arrays: the place of a pair
// in the expert-sorted list is the number of pairs that come before it in (expert, pair id)
// order; one work item starts at every 8th pair of an expert.  sh: 3 * n_pairs ints.
// ep_world > 0 (expert parallel over replicated tokens): pairs of experts that live on another rank are
// left to that rank without complaint, and the shared expert (resident everywhere) of token t is taken
// by rank t % ep_world; n_local receives the number of pairs this rank computes (= entries of `sorted`).
__device__ __forceinline__ void plan_small(const int32_t *pair_expert, int n_pairs, int n_slots, const void *const *__restrict__ wv,
                                           int32_t *__restrict__ sorted, int32_t *__restrict__ items, int32_t *__restrict__ n_items,
                                           int max_items, int32_t *__restrict__ status, int *sh, int pairs_per_tok, int ep_rank,
                                           int ep_world, int32_t *__restrict__ n_local) {
    int *sh_e = sh, *sh_rank = sh + n_pairs, *sh_start = sh + 2 * n_pairs;
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = pair_expert[p];
        bool ok = e >= 0 && e < n_slots && wv[e * 3] != nullptr;
        if (ep_world > 0) {
            if (ok && e == n_slots - 1 && (p / pairs_per_tok) % ep_world != ep_rank) ok = false;
        } else if (!ok) {
            atomicCAS(status, 0, MK_ERR_ARG);
        }
        sh_e[p] = ok ? e : -1; // pairs naming an expert that is not resident are dropped
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = sh_e[p];
        int rank = 0, before = 0;
        if (e >= 0) {
            for (int q = 0; q < n_pairs; ++q) {
                const int eq = sh_e[q];
                if (eq < 0) continue;
                if (eq < e || (eq == e && q < p)) ++rank;
                if (eq == e && q < p) ++before;
            }
            sorted[rank] = p;
        }
        sh_rank[p] = e >= 0 ? rank : -1;
        sh_start[p] = (e >= 0 && (before & 7) == 0) ? 1 : 0;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        if (!sh_start[p]) continue;
        const int e = sh_e[p];
        int idx = 0, after = 0;
        for (int q = 0; q < n_pairs; ++q) {
            if (sh_start[q] && sh_rank[q] < sh_rank[p]) ++idx;
            if (sh_e[q] == e && q >= p) ++after; // pairs of this expert from p on
        }
        if (idx < max_items) {
            items[idx * 3 + 0] = e;
            items[idx * 3 + 1] = sh_rank[p];
            items[idx * 3 + 2] = after < 8 ? after : 8;
        }
    }
    if (threadIdx.x == 0) {
        int total = 0, mine = 0;
        for (int q = 0; q < n_pairs; ++q) { total += sh_start[q]; mine += sh_e[q] >= 0 ? 1 : 0; }
        if (n_local) *n_local = mine;
        *n_items = total < max_items ? total : max_items;
        if (total > max_items) atomicCAS(status, 0, MK_ERR_STATE);
    }
}

// ------------------------------------------------------------------ whole router side in ONE launch (<= 16 tokens)
// grid.x = ceil(n_experts / S::NE) logits CTAs (as moe_router_tile_kernel) + CTAs that quantize
// the token rows to q8_0 (src/q8.rs:49-69) for the expert kernels.  The LAST logits CTA to
// finish (a counter; nobody waits) runs top-k, one warp per token, and then groups the
// (token, slot) pairs by expert.
struct RouterFusedArgs {
    const float *gate_w, *gate_b, *x;
    float *logits, *score, *key;
    int n_experts, d, n_tokens, top_k, shared_slot, router_kind;
    float route_scale;
    int32_t *ids; float *wts;
    int32_t *pair_row, *pair_expert; float *pair_weight;
    const void *const *wv;
    int32_t *sorted, *items, *n_items; int max_items;
    int32_t *status, *counter;
    int8_t *xq; float *xs; int64_t nbp;
    int ep_rank, ep_world; int32_t *n_local;   // expert parallel over replicated tokens (ep_world 0 = off)
};
template <class S>
__global__ void __launch_bounds__(256) moe_router_fused_kernel(const RouterFusedArgs a) {
    extern __shared__ __align__(16) float rsm[];
    mk_dep_trigger();       // the expert kernel launched behind this one may become resident; it waits for the routing itself
    const int d = a.d, n_tokens = a.n_tokens, n_experts = a.n_experts;
    const int logit_ctas = (n_experts + S::NE - 1) / S::NE;
    if ((int)blockIdx.x >= logit_ctas) {
        // ---- quantize role: one warp per (token, block of 32)
        const int64_t unit = ((int64_t)(blockIdx.x - logit_ctas) * blockDim.x + threadIdx.x) >> 5;
        const int lane = threadIdx.x & 31;
        if (unit >= (int64_t)n_tokens * a.nbp) return;
        const int64_t tok = unit / a.nbp, b = unit % a.nbp;
        const int64_t c = b * 32 + lane;
        const float v = (c < d) ? a.x[tok * d + c] : 0.0f;
        float mx = fabsf(v);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        const float dx = __fdiv_rn(mx, 127.0f);
        int q = 0;
        if (dx != 0.0f) q = (int)fminf(fmaxf(roundf(__fdiv_rn(v, dx)), -127.0f), 127.0f);
        const uint32_t qb = (uint32_t)q & 0xFFu;
        const uint32_t pk = qb | (__shfl_down_sync(0xFFFFFFFFu, qb, 1) << 8) | (__shfl_down_sync(0xFFFFFFFFu, qb, 2) << 16) |
                            (__shfl_down_sync(0xFFFFFFFFu, qb, 3) << 24);
        if ((lane & 3) == 0) ((uint32_t *)(a.xq + tok * a.nbp * 32 + b * 32))[lane >> 2] = pk;
        if (lane == 0) a.xs[tok * a.nbp + b] = dx;
        return;
    }
    {
        int e, tok;
        bool valid;
        const float l = mkf::tile_dot<S>(a.gate_w, a.x, n_experts, d, n_tokens, blockIdx.x * S::NE, 0, rsm, &e, &tok, &valid);
        if (valid) router_store(a.logits, a.score, a.key, a.gate_b, (int64_t)tok * n_experts + e, e, l, a.router_kind);
    }
    // ---- the last logits CTA to get here does the rest
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(a.counter, 1);
        s_last = (prev == logit_ctas - 1) ? 1 : 0;
        if (s_last) *a.counter = 0; // ready for the next call
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    __shared__ int s_planned;
    if (threadIdx.x == 0) s_planned = 0;
    if (n_tokens == 1) {
        // one token: warp 0 picks, writes weights and pairs and, when every pick is resident here and no shared slot or
        // expert parallelism is involved, the grouping as well: one work item per pick, ordered by expert (the picks
        // are distinct)
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (warp == 0) {
            const int my_id = topk_token(a.score, a.key, n_experts, a.top_k, 0, lane, rsm, a.ids, a.wts, a.pair_row, a.pair_expert,
                                         a.pair_weight, a.shared_slot, a.router_kind, a.route_scale);
            // the shared expert, when the layer has one, is pair top_k with the largest expert number: the last work item
            const int n_it = a.top_k + (a.shared_slot ? 1 : 0);
            const int my_e = lane < a.top_k ? my_id : n_experts;
            const bool res = lane < n_it ? a.wv[(size_t)my_e * 3] != nullptr : true;
            const bool fast = __all_sync(0xFFFFFFFFu, res) && a.ep_world == 0 && n_it <= a.max_items;
            if (fast) {
                int rank = 0;
                for (int j = 0; j < a.top_k; ++j) rank += __shfl_sync(0xFFFFFFFFu, my_id, j) < my_e ? 1 : 0;
                if (lane < n_it) {
                    a.sorted[rank] = lane;
                    a.items[rank * 3 + 0] = my_e;
                    a.items[rank * 3 + 1] = rank;
                    a.items[rank * 3 + 2] = 1;
                }
                if (lane == 0) {
                    *a.n_items = n_it;
                    if (a.n_local) *a.n_local = n_it;
                    s_planned = 1;
                }
            }
        }
    } else {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        for (int tok = warp; tok < n_tokens; tok += nw)
            topk_token(a.score, a.key, n_experts, a.top_k, tok, lane, rsm + (size_t)warp * n_experts, a.ids, a.wts, a.pair_row,
                       a.pair_expert, a.pair_weight, a.shared_slot, a.router_kind, a.route_scale);
    }
    __threadfence_block();
    __syncthreads();
    if (s_planned) return;
    const int slots = a.top_k + (a.shared_slot ? 1 : 0);
    plan_small(a.pair_expert, n_tokens * slots, n_experts + 1, a.wv, a.sorted, a.items, a.n_items, a.max_items, a.status, (int *)rsm, slots,
               a.ep_rank, a.ep_world, a.n_local);
    __syncthreads();
}

// ------------------------------------------------------------------ plan
// Single block: counting sort of the pairs by expert, then one work item per
// (expert, chunk of <= 8 pairs).  Pairs naming an expert that is not resident are
// dropped and flagged in the status word.
__device__ __forceinline__ void
plan_body(const int32_t *__restrict__ pair_expert, int n_pairs, int n_slots /* n_experts + 1 */,
          const void *const *__restrict__ wv, int32_t *__restrict__ sorted, int32_t *__restrict__ items,
          int32_t *__restrict__ n_items, int max_items, int32_t *__restrict__ status, int chunk /* pairs per work item: 8, or 16 */, int *sh) {
    int *cnt = sh, *off = sh + n_slots, *ioff = off + n_slots, *cur = ioff + n_slots;
    for (int e = threadIdx.x; e < n_slots; e += blockDim.x) { cnt[e] = 0; cur[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = pair_expert[p];
        if (e < 0 || e >= n_slots || wv[e * 3] == nullptr) { atomicCAS(status, 0, MK_ERR_ARG); continue; }
        atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    {
        // exclusive prefix sums over the slots of the pair counts (off) and of the work items (ioff): every thread sums a
        // run of consecutive slots, the runs are scanned across the block (a single thread walking 897 slots took 50 us)
        __shared__ int wsum[2][32];
        const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = (blockDim.x + 31) >> 5;
        const int per = (n_slots + (int)blockDim.x - 1) / (int)blockDim.x;
        const int e0 = min(tid * per, n_slots), e1 = min(e0 + per, n_slots);
        int so = 0, si = 0;
        for (int e = e0; e < e1; ++e) { so += cnt[e]; si += (cnt[e] + chunk - 1) / chunk; }
        int xo = so, xi = si;                                   // inclusive scan inside the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int yo = __shfl_up_sync(0xFFFFFFFFu, xo, d), yi = __shfl_up_sync(0xFFFFFFFFu, xi, d);
            if (lane >= d) { xo += yo; xi += yi; }
        }
        if (lane == 31) { wsum[0][warp] = xo; wsum[1][warp] = xi; }
        __syncthreads();
        if (warp == 0) {
            int to = lane < nwarp ? wsum[0][lane] : 0, ti = lane < nwarp ? wsum[1][lane] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int yo = __shfl_up_sync(0xFFFFFFFFu, to, d), yi = __shfl_up_sync(0xFFFFFFFFu, ti, d);
                if (lane >= d) { to += yo; ti += yi; }
            }
            wsum[0][lane] = to; wsum[1][lane] = ti;             // inclusive over the warps
        }
        __syncthreads();
        int o = xo - so + (warp > 0 ? wsum[0][warp - 1] : 0), io = xi - si + (warp > 0 ? wsum[1][warp - 1] : 0);
        for (int e = e0; e < e1; ++e) {
            off[e] = o;
            ioff[e] = io;
            o += cnt[e];
            io += (cnt[e] + chunk - 1) / chunk;
        }
        if (tid == 0) {
            const int total = wsum[1][nwarp - 1];
            *n_items = total < max_items ? total : max_items;
            if (total > max_items) atomicCAS(status, 0, MK_ERR_STATE);
        }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = pair_expert[p];
        if (e < 0 || e >= n_slots || wv[e * 3] == nullptr) continue;
        sorted[off[e] + atomicAdd(&cur[e], 1)] = p;
    }
    for (int e = threadIdx.x; e < n_slots; e += blockDim.x) {
        const int nch = (cnt[e] + chunk - 1) / chunk;
        for (int c = 0; c < nch; ++c) {
            const int it = ioff[e] + c;
            if (it < max_items) {
                items[it * 3 + 0] = e;
                items[it * 3 + 1] = off[e] + c * chunk;
                items[it * 3 + 2] = min(chunk, cnt[e] - c * chunk);
            }
        }
    }
}
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int32_t *__restrict__ pair_expert, int n_pairs, int n_slots, const void *const *__restrict__ wv, int32_t *__restrict__ sorted,
                int32_t *__restrict__ items, int32_t *__restrict__ n_items, int max_items, int32_t *__restrict__ status, int chunk) {
    extern __shared__ int sh[];
    plan_body(pair_expert, n_pairs, n_slots, wv, sorted, items, n_items, max_items, status, chunk, sh);
}

} // namespace

namespace {

struct MoeArgs {
    const void *const *wv;       // [(E+1)*3] tiled values
    const void *const *wsc;      // [(E+1)*3] tiled scales
    const int32_t *items;        // [n][3]
    const int32_t *n_items;
    const int32_t *sorted;       // pair ids
    const int32_t *pair_row;
    const float *pair_weight;
    const int8_t *xq;            // [rows][ldq_d]
    const float *xs;             // [rows][nbp_d]
    int8_t *actq;                // [pairs][ldq_i]
    float *acts;                 // [pairs][nbp_i]
    float *outs;                 // [pairs][d]
    int64_t nbp_d, nbp_i;
    int d, inter;
    int activation;              // MK_MOE_*
    float limit;
    Consts k;
};

} // namespace
#include "moe_tc.cuh"
namespace {

// Everything the tensor-core expert kernels need, one launch: block 0 groups the pairs by expert (plan_body) and writes
// the per-item row tables; the other blocks turn the token rows into their E2M1 limbs.  Neither half needs the other.
__global__ void __launch_bounds__(1024)
moe_tc_prepare_kernel(const int32_t *__restrict__ pair_expert, int n_pairs, int n_slots, const void *const *__restrict__ wv, int32_t *__restrict__ sorted,
                      int32_t *__restrict__ items, int32_t *__restrict__ n_items, int max_items, int32_t *__restrict__ status,
                      const int32_t *__restrict__ pair_row, int32_t *__restrict__ rows_x, int32_t *__restrict__ rows_p, const float *__restrict__ x,
                      int n_rows, int cols, int64_t ldx, uint8_t *__restrict__ xl, uint8_t *__restrict__ xsf) {
    extern __shared__ int sh[];
    if (blockIdx.x == 0) {
        plan_body(pair_expert, n_pairs, n_slots, wv, sorted, items, n_items, max_items, status, mtc::NT, sh);
        __syncthreads();        // this block's own writes of items / sorted / n_items, read back below
        const int ni = *n_items;
        for (int idx = threadIdx.x; idx < max_items * mtc::NT; idx += blockDim.x) {
            const int item = idx / mtc::NT, t = idx % mtc::NT;
            int p = 0;
            if (item < ni && t < min(items[item * 3 + 2], mtc::NT)) p = sorted[items[item * 3 + 1] + t];
            rows_p[idx] = p;
            rows_x[idx] = pair_row[p];
        }
        return;
    }
    mtc::act_limbs_body(x, n_rows, cols, ldx, xl, xsf, (int64_t)(blockIdx.x - 1) * blockDim.x + threadIdx.x, (int64_t)(gridDim.x - 1) * blockDim.x);
}

// Partial sums of one warp for a 16-row tile and up to 8 columns, into smem part[16][8].
// SPREAD: items of <= 2 columns (or, without BATCHED, any item by repeated passes) take the
// spread schedule, 2 columns per pass.  BATCHED: items of more than 2 columns take the
// batched schedule.  Both give the same bits for a column.
template <int WF, bool SPREAD, bool BATCHED, bool ORDERED = false>
__device__ __forceinline__ void warp_tile_any(const uint4 *tile, const void *sc, int64_t ngroups, int ks, int KS, int lane,
                                              int n, const int8_t *const *xrow /* [n] */, const float *const *xsrow /* [n] */,
                                              const Consts &k, float (*part)[8]) {
    const int g = lane >> 2, t = lane & 3;
    if (SPREAD && n == 1) {
        float o[2][1];
        warp_tile_spread<WF, 1, false>(tile, sc, ngroups, ks, KS, lane, (g & 1) == 0 ? xrow[0] : nullptr, xsrow[0], xsrow[0], k, o);
        if (t == 0) { part[g][0] = o[0][0]; part[g + 8][0] = o[1][0]; }
    } else if (SPREAD && (n == 2 || !BATCHED)) {
        const int slot = g & 1;
#pragma unroll 1
        for (int c0 = 0; c0 < n; c0 += 2) {
            const bool two = c0 + 1 < n; // an odd last column runs with an empty second slot
            const int8_t *xr = (slot == 0 || two) ? xrow[c0 + slot] : nullptr;
            float o[2][2];
            warp_tile_spread<WF, 2, false>(tile, sc, ngroups, ks, KS, lane, xr, xsrow[c0], xsrow[two ? c0 + 1 : c0], k, o);
            if (t == 0) {
                part[g][c0] = o[0][0]; part[g + 8][c0] = o[1][0];
                if (two) { part[g][c0 + 1] = o[0][1]; part[g + 8][c0 + 1] = o[1][1]; }
            }
        }
    } else if constexpr (BATCHED) {
        float acc[4];
        const int ca = 2 * t, cb = 2 * t + 1;
        warp_tile_batched<WF, false, ORDERED>(tile, sc, ngroups, ks, KS, lane, g < n ? xrow[g] : nullptr, ca < n ? xsrow[ca] : nullptr,
                                     cb < n ? xsrow[cb] : nullptr, k, acc);
        part[g][ca] = acc[0]; part[g][cb] = acc[1];
        part[g + 8][ca] = acc[2]; part[g + 8][cb] = acc[3];
    }
}

// ------------------------------------------------------------------ gate / up + activation + q8 of the activation
// grid = (inter/32, max_items).  CTA = 16 warps: 32 rows of w1 and the same 32 rows of w3
// of one expert for <= 8 pairs: warp = (matrix, 16-row half, K quarter).  Then warp c
// turns column c into the activation (src/deepseek.rs:1083-1087) and quantizes
// its 32 values as one q8_0 block (src/q8.rs:49-69): the input of the w2 matvec.
#ifndef MK_G1_KS
#define MK_G1_KS 2   // K slices per 16-row tile in the gate/up kernel: CTA = 4 * MK_G1_KS warps
#endif
// MODE: which work items a launch takes and how.  MOE_ALL_SPREAD: all of them by spread
// passes (calls of <= 2 token rows; fewest registers, 4 CTAs per SM = one wave at batch 1).
// MOE_MIXED: all of them, each by the schedule its size asks for, still 4 CTAs per SM
// (calls of a few tokens, where most items are small and the shared expert's big items
// overlap them).  Large calls launch MOE_BIG_ITEMS (batched schedule with all the registers
// it wants, 2 CTAs per SM) and MOE_SMALL_ITEMS (items of <= 2 pairs) one after the other.
// MOE_STRICT: every item by the batched schedule with ONE accumulator per output, the block terms added in ascending
// order with a separate multiply and add, and no K split (the other K-slice warps contribute an exact zero): the bits of
// the CPU's matvec_packed_q8 (src/mxfp4.rs:409-418), so the q8 rounding of the activations cannot flip.
enum { MOE_ALL_SPREAD = 0, MOE_SMALL_ITEMS = 1, MOE_BIG_ITEMS = 2, MOE_MIXED = 3, MOE_STRICT = 4 };
#ifndef MK_MOE_BIG_CTAS
#define MK_MOE_BIG_CTAS 2
#endif
#ifndef MK_MOE_MIXED_MAX
#define MK_MOE_MIXED_MAX 32   // calls of up to this many token rows use MOE_MIXED
#endif
template <int MODE>
__global__ void __launch_bounds__(MK_G1_KS * 128, (MODE == MOE_BIG_ITEMS || MODE == MOE_STRICT) ? MK_MOE_BIG_CTAS : 8 / MK_G1_KS) moe_gate_up_kernel(const MoeArgs a) {
    constexpr bool STRICT = MODE == MOE_STRICT;
    constexpr bool BATCHED = MODE == MOE_BIG_ITEMS || MODE == MOE_MIXED || STRICT, SPREAD = MODE != MOE_BIG_ITEMS && !STRICT;
    // behind the router by programmatic stream serialization: resident early, waits for the routing; the trigger comes after
    // the wait, so that a kernel launched behind this one finds the routing complete whenever it starts
    mk_dep_wait();
    mk_dep_trigger();
    const int item = blockIdx.y;
    if (item >= *a.n_items) return;
    const int e = a.items[item * 3], off = a.items[item * 3 + 1], n = a.items[item * 3 + 2];
    if ((MODE == MOE_SMALL_ITEMS && n > 2) || (MODE == MOE_BIG_ITEMS && n <= 2)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ float part[4 * MK_G1_KS][16][8];
    __shared__ const int8_t *xrow[8];
    __shared__ const float *xsrow[8];
    __shared__ int pair_s[8];
    __shared__ float wgt_s[8];
    if (threadIdx.x < 8) {
        const int c = threadIdx.x;
        const int p = c < n ? a.sorted[off + c] : -1;
        pair_s[c] = p;
        const int row = p >= 0 ? a.pair_row[p] : 0;
        xrow[c] = a.xq + (int64_t)row * a.nbp_d * 32;
        xsrow[c] = a.xs + (int64_t)row * a.nbp_d;
        wgt_s[c] = p >= 0 ? a.pair_weight[p] : 0.0f;
    }
    __syncthreads();
    {
        const int job = warp / MK_G1_KS, ks = warp % MK_G1_KS;
        const int mat = (job >> 1) ? 2 : 0, half = job & 1;
        const int64_t rt = (int64_t)blockIdx.x * 2 + half;
        const void *wv = a.wv[e * 3 + mat], *ws = a.wsc[e * 3 + mat];
        if (!STRICT)
            warp_tile_any<W_MXFP4, SPREAD, BATCHED>(tile_values<W_MXFP4>(wv, rt, a.nbp_d), tile_scales<W_MXFP4>(ws, rt, a.nbp_d), a.nbp_d >> 2, ks, MK_G1_KS,
                                   lane, n, xrow, xsrow, a.k, part[warp]);
        else if (ks == 0)   // the whole K range in one warp, in order; the slices ks > 0 are not read below
            warp_tile_any<W_MXFP4, false, true, true>(tile_values<W_MXFP4>(wv, rt, a.nbp_d), tile_scales<W_MXFP4>(ws, rt, a.nbp_d), a.nbp_d >> 2, 0, 1,
                                   lane, n, xrow, xsrow, a.k, part[warp]);
    }
    __syncthreads();
    const int c = warp; // column
    if (c < n) {
        const int half = lane >> 4, r16 = lane & 15;
        const int jg = (0 + half) * MK_G1_KS, ju = (2 + half) * MK_G1_KS;
        float gate = part[jg][r16][c], up = part[ju][r16][c];
        if (!STRICT) {
#pragma unroll
            for (int q = 1; q < MK_G1_KS; ++q) { gate += part[jg + q][r16][c]; up += part[ju + q][r16][c]; }
        }
        float act;
        if (a.activation == MK_MOE_SITU) {
            act = mk_situ(gate, up); // the routing weight is applied after w2 (src/model.rs:2346-2351)
        } else {
            const float gl = fminf(gate, a.limit);
            const float ul = fminf(fmaxf(up, -a.limit), a.limit);
            const float ex = (float)exp((double)(-gl));
            const float silu = __fdiv_rn(gl, __fadd_rn(1.0f, ex));
            act = __fmul_rn(__fmul_rn(wgt_s[c], silu), ul);
        }
        float mx = fabsf(act);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        const float dx = __fdiv_rn(mx, 127.0f);
        int q = 0;
        if (dx != 0.0f) q = (int)fminf(fmaxf(roundf(__fdiv_rn(act, dx)), -127.0f), 127.0f);
        const int p = pair_s[c];
        a.actq[(int64_t)p * a.nbp_i * 32 + (int64_t)blockIdx.x * 32 + lane] = (int8_t)q;
        if (lane == 0) a.acts[(int64_t)p * a.nbp_i + blockIdx.x] = dx;
    }
}

// ------------------------------------------------------------------ down projection
// grid = (ceil(d/32), max_items).  CTA: 2 row tiles of w2 x 4 K slices.
template <int MODE>
__global__ void __launch_bounds__(256, (MODE == MOE_BIG_ITEMS || MODE == MOE_STRICT) ? MK_MOE_BIG_CTAS : 4) moe_down_kernel(const MoeArgs a) {
    constexpr bool STRICT = MODE == MOE_STRICT;
    constexpr bool BATCHED = MODE == MOE_BIG_ITEMS || MODE == MOE_MIXED || STRICT, SPREAD = MODE != MOE_BIG_ITEMS && !STRICT;
    const int item = blockIdx.y;
    // Behind the gate / up kernel by programmatic stream serialization, this CTA may be resident while that kernel's last
    // CTAs still run.  The routing is complete by then (the gate / up kernel triggers after its own wait), so the work
    // item is known: the CTA asks L2 for its two weight tiles (32 KB + 2 KB of scales), which do not depend on the
    // activations, and only then waits for them.
    if (item < *a.n_items) {
        const int e0 = a.items[item * 3];
        const int64_t nrt0 = (a.d + 15) >> 4, rt0 = (int64_t)blockIdx.x * 2;
        if (rt0 < nrt0) {
            const char *wv0 = (const char *)tile_values<W_MXFP4>(a.wv[e0 * 3 + 1], rt0, a.nbp_i);
            const char *ws0 = (const char *)tile_scales<W_MXFP4>(a.wsc[e0 * 3 + 1], rt0, a.nbp_i);
            const int64_t tile_bytes = a.nbp_i * 256, scale_bytes = a.nbp_i * 16, ntile = rt0 + 1 < nrt0 ? 2 : 1;
            for (int64_t o = (int64_t)threadIdx.x * 128; o < ntile * tile_bytes; o += 256 * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(wv0 + o));
            if ((int64_t)threadIdx.x * 128 < ntile * scale_bytes) asm volatile("prefetch.global.L2 [%0];" ::"l"(ws0 + (int64_t)threadIdx.x * 128));
        }
    }
    mk_dep_wait();
    mk_dep_trigger();
    if (item >= *a.n_items) return;
    const int e = a.items[item * 3], off = a.items[item * 3 + 1], n = a.items[item * 3 + 2];
    if ((MODE == MOE_SMALL_ITEMS && n > 2) || (MODE == MOE_BIG_ITEMS && n <= 2)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ float part[8][16][8];
    __shared__ const int8_t *xrow[8];
    __shared__ const float *xsrow[8];
    __shared__ int pair_s[8];
    if (threadIdx.x < 8) {
        const int c = threadIdx.x;
        const int p = c < n ? a.sorted[off + c] : -1;
        pair_s[c] = p;
        const int pp = p >= 0 ? p : 0;
        xrow[c] = a.actq + (int64_t)pp * a.nbp_i * 32;
        xsrow[c] = a.acts + (int64_t)pp * a.nbp_i;
    }
    __syncthreads();
    const int64_t nrt = (a.d + 15) >> 4;
    const int rt_local = warp >> 2, ks = warp & 3;
    const int64_t rt = (int64_t)blockIdx.x * 2 + rt_local;
    if (rt < nrt) {
        const void *wv = a.wv[e * 3 + 1], *ws = a.wsc[e * 3 + 1];
        if (!STRICT)
            warp_tile_any<W_MXFP4, SPREAD, BATCHED>(tile_values<W_MXFP4>(wv, rt, a.nbp_i), tile_scales<W_MXFP4>(ws, rt, a.nbp_i), a.nbp_i >> 2, ks, 4,
                                   lane, n, xrow, xsrow, a.k, part[warp]);
        else if (ks == 0)
            warp_tile_any<W_MXFP4, false, true, true>(tile_values<W_MXFP4>(wv, rt, a.nbp_i), tile_scales<W_MXFP4>(ws, rt, a.nbp_i), a.nbp_i >> 2, 0, 1,
                                   lane, n, xrow, xsrow, a.k, part[warp]);
    }
    __syncthreads();
    // 2 tiles x 16 rows x 8 columns = 256 outputs, one per thread
    const int tl = threadIdx.x >> 7, r16 = (threadIdx.x >> 3) & 15, c = threadIdx.x & 7;
    const int64_t row = ((int64_t)blockIdx.x * 2 + tl) * 16 + r16;
    if (c < n && row < a.d) {
        float v = part[tl * 4 + 0][r16][c];
        if (!STRICT) v = ((v + part[tl * 4 + 1][r16][c]) + part[tl * 4 + 2][r16][c]) + part[tl * 4 + 3][r16][c];
        // K3 body: the routing weight multiplies the expert output, y += w_i * o_i (src/model.rs:2346-2351);
        // the product is formed here and the combine step adds the terms in slot order
        if (a.activation == MK_MOE_SITU) v = __fmul_rn(a.pair_weight[pair_s[c]], v);
        a.outs[(int64_t)pair_s[c] * a.d + row] = v;
    }
}

// out[t][j] = ((0 + outs[t,0][j]) + outs[t,1][j]) + ... in slot order (src/deepseek.rs:1095-1106)
__global__ void __launch_bounds__(256) moe_combine_kernel(const float *__restrict__ outs, int n_tokens, int slots, int d,
                                                         float *__restrict__ out) {
    mk_dep_wait();      // behind the down kernel by programmatic stream serialization
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)n_tokens * d) return;
    const int64_t t = idx / d, j = idx % d;
    float v = 0.0f;
    for (int s = 0; s < slots; ++s) v = __fadd_rn(v, outs[(t * slots + s) * d + j]);
    out[idx] = v;
}

// ------------------------------------------------------------------ expert-parallel exchange
// CTA c copies the output row of the c-th pair this rank computed into the same table slot of every other
// rank (16-byte peer stores).  The last CTA to finish publishes this rank's step number in every rank's flag
// word and waits - bounded - for all ranks' flags: when the kernel ends, the local table is complete.
constexpr uint32_t EP_WAIT_LIMIT = 1u << 22; // polls of >= 100 ns: about half a second
struct EpPeers { float *outs[8]; uint32_t *flag[8]; };
__global__ void __launch_bounds__(256) moe_ep_exchange_kernel(const EpPeers pe, const float *__restrict__ local_outs,
                                                             const int32_t *__restrict__ sorted, const int32_t *__restrict__ n_local, int d,
                                                             int rank, int world, const uint32_t *__restrict__ flags, uint32_t *__restrict__ counter,
                                                             int32_t *__restrict__ status) {
    __shared__ int s_last;
    // the step number lives on the device (counter[1] = steps finished so far), not in the launch arguments: a recorded
    // launch (CUDA graph) must publish a new number at every replay.  Every thread reads it here; the last CTA, which
    // writes the new value at its end, is by construction the one that saw all other CTAs count in after this read.
    const uint32_t step = *(volatile const uint32_t *)(counter + 1) + 1u;
    if ((int)blockIdx.x < *n_local) {
        const int64_t p = sorted[blockIdx.x];
        const float4 *src = (const float4 *)(local_outs + p * d);
        for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
            const float4 v = __ldcg(src + i);
            for (int q = 0; q < world; ++q)
                if (q != rank) ((float4 *)(pe.outs[q] + p * d))[i] = v;
        }
    }
    // Release by one thread for the CTA: the barrier orders every thread's peer stores before thread 0's system-wide
    // fence (fences are cumulative), the fence before the count; the last CTA's thread 0 fences again after it saw the
    // full count and the second barrier hands that to the flag writers, whose release stores carry it to the peers.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned prev = atomicAdd(counter, 1u);
        s_last = prev == gridDim.x - 1 ? 1 : 0;
        if (s_last) {
            *counter = 0u;
            __threadfence_system();
        }
    }
    __syncthreads();
    if (!s_last) return;
    if ((int)threadIdx.x < world) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pe.flag[threadIdx.x]), "r"(step) : "memory");
        bool ok = false;
        uint64_t t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (uint32_t it = 0; it < EP_WAIT_LIMIT; ++it) {   // bounded twice: by polls and by one second of wall time
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
            if ((int32_t)(v - step) >= 0) { ok = true; break; }
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 1000000000ull) break;
            __nanosleep(100);
        }
        if (!ok) atomicCAS(status, 0, MK_ERR_TIMEOUT);
    }
    if (threadIdx.x == 0) counter[1] = step;
    __threadfence_system();
}

} // namespace

// ====================================================================== host side
#include <new>
#include <vector>

static void moe_free_ws(mk_moe *m) {
    void *ptrs[] = {m->logits, m->ids, m->wts, m->xq, m->xs, m->pair_row, m->pair_expert, m->pair_weight,
                    m->sorted, m->items, m->n_items, m->actq, m->acts, m->outs, m->lat_h, m->lat_y, m->lat_yn, m->sh_a, m->sh_u,
                    m->stk, m->sh_out, m->xl, m->xsf, m->actl, m->actsf, m->tc_rows_x, m->tc_rows_p};
    for (void *p : ptrs) if (p) cudaFree(p);
    m->xl = m->xsf = m->actl = m->actsf = nullptr;
    m->tc_rows_x = m->tc_rows_p = nullptr;
    m->lat_h = m->lat_y = m->lat_yn = m->sh_a = m->sh_u = m->stk = m->sh_out = nullptr;
    m->logits = nullptr; m->ids = nullptr; m->wts = nullptr; m->xq = nullptr; m->xs = nullptr;
    m->pair_row = m->pair_expert = nullptr; m->pair_weight = nullptr; m->sorted = m->items = m->n_items = nullptr;
    m->actq = nullptr; m->acts = nullptr; m->outs = nullptr;
    m->cap_rows = m->cap_pairs = 0;
}

// (Re)allocates the per-call buffers for `rows` activation rows and `pairs` pairs.
// Grows geometrically; steady-state calls allocate nothing.
static int32_t moe_reserve(mk_ctx *ctx, mk_moe *m, int rows, int pairs) {
    if (rows <= m->cap_rows && pairs <= m->cap_pairs) return MK_OK;
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    int nr = m->cap_rows > 0 ? m->cap_rows : 1, np = m->cap_pairs > 0 ? m->cap_pairs : 1;
    while (nr < rows) nr *= 2;
    while (np < pairs) np *= 2;
    moe_free_ws(m);
    ctx->alloc_epoch++;         // recorded launches that point into the old buffers are stale
    const int E = m->n_experts, k = m->top_k;
    m->max_items = np / 8 + (np < E + 1 ? np : E + 1) + 1;
    const size_t ldq_d = (size_t)m->nbp_d * 32, ldq_i = (size_t)m->nbp_i * 32;
    MK_CUDA(cudaMalloc(&m->logits, (size_t)nr * E * 4 * 3));
    MK_CUDA(cudaMalloc(&m->ids, (size_t)nr * k * 4));
    MK_CUDA(cudaMalloc(&m->wts, (size_t)nr * k * 4));
    MK_CUDA(cudaMalloc(&m->xq, (size_t)nr * ldq_d));
    MK_CUDA(cudaMalloc(&m->xs, (size_t)nr * m->nbp_d * 4));
    MK_CUDA(cudaMalloc(&m->pair_row, (size_t)np * 4));
    MK_CUDA(cudaMalloc(&m->pair_expert, (size_t)np * 4));
    MK_CUDA(cudaMalloc(&m->pair_weight, (size_t)np * 4));
    MK_CUDA(cudaMalloc(&m->sorted, (size_t)np * 4));
    MK_CUDA(cudaMalloc(&m->items, (size_t)m->max_items * 3 * 4));
    MK_CUDA(cudaMalloc(&m->n_items, 4));
    MK_CUDA(cudaMalloc(&m->actq, (size_t)np * ldq_i));
    MK_CUDA(cudaMalloc(&m->acts, (size_t)np * m->nbp_i * 4));
    MK_CUDA(cudaMalloc(&m->outs, (size_t)np * m->d * 4));
    if (m->latent > 0) {
        MK_CUDA(cudaMalloc(&m->lat_h, (size_t)nr * m->latent * 4));
        MK_CUDA(cudaMalloc(&m->lat_y, (size_t)nr * m->latent * 4));
        MK_CUDA(cudaMalloc(&m->lat_yn, (size_t)nr * m->latent * 4));
    }
    if (m->sh_gate) {
        MK_CUDA(cudaMalloc(&m->sh_a, (size_t)nr * m->shared_inter * 4));
        MK_CUDA(cudaMalloc(&m->sh_u, (size_t)nr * m->shared_inter * 4));
        MK_CUDA(cudaMalloc(&m->sh_out, (size_t)nr * m->dx * 4));
        if (m->latent > 0) MK_CUDA(cudaMalloc(&m->stk, (size_t)(m->latent + 2 * m->shared_inter) * 4));
    }
    if (m->tc) {
        MK_CUDA(cudaMalloc(&m->xl, (size_t)mtc::NL * nr * (m->d / 2)));
        MK_CUDA(cudaMalloc(&m->xsf, (size_t)mtc::NL * nr * (m->d / 32)));
        MK_CUDA(cudaMalloc(&m->actl, (size_t)mtc::NL * np * (m->inter / 2)));
        MK_CUDA(cudaMalloc(&m->actsf, (size_t)mtc::NL * np * (m->inter / 32)));
        MK_CUDA(cudaMalloc(&m->tc_rows_x, (size_t)m->max_items * mtc::NT * 4));
        MK_CUDA(cudaMalloc(&m->tc_rows_p, (size_t)m->max_items * mtc::NT * 4));
    }
    // padded tails of the q8 rows must read as zero
    MK_CUDA(cudaMemsetAsync(m->actq, 0, (size_t)np * ldq_i, ctx->stream));
    MK_CUDA(cudaMemsetAsync(m->acts, 0, (size_t)np * m->nbp_i * 4, ctx->stream));
    m->cap_rows = nr;
    m->cap_pairs = np;
    return MK_OK;
}

// A 2-D tensor map over bytes: rows of 128 bytes (256 E2M1 codes), `rows` of them, box = 128 bytes x 128 rows, 128-byte
// swizzle: what a box lands in shared memory is the K-major FP4 operand tile of a kind::mxf4 MMA.  Rows past the end read
// as zero.  The driver entry point is looked up at run time (no link against libcuda).
static bool moe_encode_fp4(CUtensorMap *map, const void *base, uint64_t rows) {
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess || !fn) return false;
        encode = (encode_fn)fn;
    }
    const cuuint64_t dims[2] = {128, rows}, strides[1] = {128};
    const cuuint32_t box[2] = {128, 128}, estr[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

extern "C" int32_t mk_moe_create(mk_ctx *ctx, const mk_moe_desc *desc, mk_moe **out) {
    MK_CHECK_ARG(ctx != nullptr && desc != nullptr && out != nullptr, "NULL argument");
    *out = nullptr;
    const int E = desc->n_experts, k = desc->top_k, dx = desc->d, I = desc->inter, latent = desc->latent;
    const int d = latent > 0 ? latent : dx; // the width the experts work on
    MK_CHECK_ARG(E >= 1 && E <= 4095 && k >= 1 && k <= 31 && k <= E, "need 1 <= top_k <= min(31, n_experts) and n_experts <= 4095");
    MK_CHECK_ARG(dx > 0 && dx % 32 == 0 && I > 0 && I % 32 == 0, "d and inter must be positive multiples of 32");
    MK_CHECK_ARG(desc->activation == MK_MOE_SWIGLU_CLAMP || desc->activation == MK_MOE_SITU, "unknown activation");
    MK_CHECK_ARG(desc->router == MK_ROUTER_SIGMOID || desc->router == MK_ROUTER_SQRT_SOFTPLUS, "unknown router kind");
    MK_CHECK_ARG(desc->experts != nullptr, "experts table is NULL");
    MK_CHECK_ARG((desc->act_mode & ~MK_ACT_STRICT) == MK_ACT_Q8 || desc->act_mode == MK_ACT_FP4X6,
                 "the MoE layer takes MK_ACT_Q8 (optionally with MK_ACT_STRICT) or MK_ACT_FP4X6");
    MK_CHECK_ARG(desc->act_mode != MK_ACT_FP4X6 || ((latent > 0 ? latent : dx) % 256 == 0 && I % 256 == 0),
                 "MK_ACT_FP4X6 needs the experts' input width and inter to be multiples of 256");
    const bool situ = desc->activation == MK_MOE_SITU;
    auto f32ok = [](const mk_weight *w, int rows, int cols) { return w && w->fmt == MK_FMT_F32 && w->rows == rows && w->cols == cols; };
    if (latent != 0) {
        MK_CHECK_ARG(situ, "a latent width needs MK_MOE_SITU (the K3 body)");
        MK_CHECK_ARG(latent > 0 && latent % 32 == 0, "latent must be a positive multiple of 32");
        MK_CHECK_ARG(f32ok(desc->routed_down, latent, dx) && f32ok(desc->routed_up, dx, latent) && desc->routed_norm != nullptr,
                     "latent MoE needs f32 routed_down [latent, d], routed_up [d, latent] and routed_norm [latent]");
    }
    const bool sh32 = desc->shared_f32[0] || desc->shared_f32[1] || desc->shared_f32[2];
    int si = 0;
    if (sh32) {
        MK_CHECK_ARG(situ, "the f32 shared expert belongs to MK_MOE_SITU (the K3 body)");
        MK_CHECK_ARG(desc->shared_f32[0] && desc->shared_f32[0]->fmt == MK_FMT_F32, "shared_f32[0] must be an f32 weight");
        si = (int)desc->shared_f32[0]->rows;
        MK_CHECK_ARG(f32ok(desc->shared_f32[0], si, dx) && f32ok(desc->shared_f32[1], dx, si) && f32ok(desc->shared_f32[2], si, dx),
                     "f32 shared expert needs gate [si, d], down [d, si], up [si, d]");
    }
    if (situ) MK_CHECK_ARG(!desc->shared[0] && !desc->shared[1] && !desc->shared[2], "MK_MOE_SITU takes its shared expert in shared_f32");
    MK_CUDA(cudaSetDevice(ctx->device));
    std::vector<const void *> hv((size_t)(E + 1) * 3, nullptr), hs((size_t)(E + 1) * 3, nullptr);
    auto check = [&](const mk_weight *w, int rows, int cols) {
        return w && w->fmt == MK_FMT_MXFP4 && w->rows == rows && w->cols == cols;
    };
    for (int e = 0; e <= E; ++e) {
        const mk_weight *t[3];
        for (int j = 0; j < 3; ++j) t[j] = e < E ? desc->experts[(size_t)e * 3 + j] : desc->shared[j];
        if (!t[0] && !t[1] && !t[2]) continue;
        if (!check(t[0], I, d) || !check(t[1], d, I) || !check(t[2], I, d)) {
            mk_set_error("mk_moe_create: expert %d needs MXFP4 w1 [inter,d], w2 [d,inter], w3 [inter,d]", e);
            return MK_ERR_ARG;
        }
        for (int j = 0; j < 3; ++j) {
            hv[(size_t)e * 3 + j] = t[j]->values;
            hs[(size_t)e * 3 + j] = t[j]->scales;
        }
    }
    mk_moe *m = new (std::nothrow) mk_moe();
    if (!m) return MK_ERR_OOM;
    memset(m, 0, sizeof(*m));
    m->n_experts = E; m->top_k = k; m->d = d; m->dx = dx; m->inter = I; m->activation = desc->activation;
    m->router_kind = desc->router;
    m->route_scale = desc->route_scale == 0.0f ? 1.0f : desc->route_scale;
    m->limit = desc->swiglu_limit;
    m->latent = latent > 0 ? latent : 0;
    m->rms_eps = desc->rms_eps;
    m->strict = (desc->act_mode & MK_ACT_STRICT) != 0;
    m->tc = desc->act_mode == MK_ACT_FP4X6;
    if (latent > 0) { m->routed_down = (const float *)desc->routed_down->values; m->routed_up = (const float *)desc->routed_up->values; }
    if (sh32) {
        m->sh_gate = (const float *)desc->shared_f32[0]->values;
        m->sh_down = (const float *)desc->shared_f32[1]->values;
        m->sh_up = (const float *)desc->shared_f32[2]->values;
        m->shared_inter = si;
        m->stack3 = latent > 0 && m->sh_gate == m->routed_down + (size_t)latent * dx && m->sh_up == m->sh_gate + (size_t)si * dx;
    }
    m->has_router = desc->gate_w != nullptr;
    m->has_shared = hv[(size_t)E * 3] != nullptr;
    m->nbp_d = mk_ceil_div(d / 32, 4) * 4;
    m->nbp_i = mk_ceil_div(I / 32, 4) * 4;
    cudaError_t e_ = cudaSuccess;
    const size_t tb = hv.size() * sizeof(void *);
    e_ = cudaMalloc((void **)&m->wv, tb);
    if (e_ == cudaSuccess) e_ = cudaMalloc((void **)&m->wsc, tb);
    if (e_ == cudaSuccess) e_ = cudaMemcpyAsync((void *)m->wv, hv.data(), tb, cudaMemcpyHostToDevice, ctx->stream);
    if (e_ == cudaSuccess) e_ = cudaMemcpyAsync((void *)m->wsc, hs.data(), tb, cudaMemcpyHostToDevice, ctx->stream);
    if (e_ == cudaSuccess && m->has_router) {
        e_ = cudaMalloc(&m->gate_w, (size_t)E * dx * 4);
        if (e_ == cudaSuccess) e_ = cudaMalloc(&m->gate_b, (size_t)E * 4);
        if (e_ == cudaSuccess) e_ = cudaMemcpyAsync(m->gate_w, desc->gate_w, (size_t)E * dx * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e_ == cudaSuccess) {
            if (desc->gate_b) e_ = cudaMemcpyAsync(m->gate_b, desc->gate_b, (size_t)E * 4, cudaMemcpyHostToDevice, ctx->stream);
            else e_ = cudaMemsetAsync(m->gate_b, 0, (size_t)E * 4, ctx->stream);
        }
    }
    if (e_ == cudaSuccess && latent > 0) {
        e_ = cudaMalloc(&m->routed_norm, (size_t)latent * 4);
        if (e_ == cudaSuccess) e_ = cudaMemcpyAsync(m->routed_norm, desc->routed_norm, (size_t)latent * 4, cudaMemcpyHostToDevice, ctx->stream);
    }
    if (e_ == cudaSuccess && m->tc && d % 256 == 0 && I % 256 == 0) {
        // The tensor-core path reads the nibbles blocked by (128 rows, 256 columns) - a TMA box each - and scale atoms: a
        // second copy of every resident expert, made here on the device from the registered (tiled) one.
        m->rm_vstride = (int64_t)d * I / 2;
        m->rm_astride = (int64_t)d * I / 32;
        const size_t nmat = hv.size();
        e_ = cudaMalloc(&m->rm_vals, nmat * (size_t)m->rm_vstride);
        if (e_ == cudaSuccess) e_ = cudaMalloc(&m->rm_atoms, nmat * (size_t)m->rm_astride);
        std::vector<CUtensorMap> maps(nmat);
        memset(maps.data(), 0, maps.size() * sizeof(CUtensorMap));
        for (size_t i = 0; i < nmat && e_ == cudaSuccess; ++i) {
            if (!hv[i]) continue;
            const int e = (int)(i / 3), j = (int)(i % 3);
            const mk_weight *w = e < E ? desc->experts[(size_t)e * 3 + j] : desc->shared[j];
            uint8_t *vals = m->rm_vals + i * m->rm_vstride, *atoms = m->rm_atoms + i * m->rm_astride;
            const int64_t nthreads = std::max<int64_t>(w->nrt * (w->nbp / 2) * 128, w->rows * w->nb);
            mtc::tc_weight_copy_kernel<<<(unsigned)mk_ceil_div(nthreads, 256), 256, 0, ctx->stream>>>((const uint32_t *)w->values, (const uint8_t *)w->scales, w->rows,
                                                                                                     w->nb, w->nbp, (uint32_t *)vals, atoms);
            ctx->launches++;
            // as a tensor: rows of 256 codes (128 bytes), rows * cols / 256 of them; a step's box is 128 consecutive rows
            if (!moe_encode_fp4(&maps[i], vals, (uint64_t)(w->rows * (w->cols / 256)))) {
                mk_set_error("mk_moe_create: cuTensorMapEncodeTiled failed");
                mk_moe_free(ctx, m);
                return MK_ERR_CUDA;
            }
        }
        if (e_ == cudaSuccess) e_ = cudaStreamSynchronize(ctx->stream);
        if (e_ == cudaSuccess) e_ = cudaMalloc(&m->tmaps, maps.size() * sizeof(CUtensorMap));
        if (e_ == cudaSuccess) e_ = cudaMemcpy(m->tmaps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
    }
    if (e_ == cudaSuccess) e_ = cudaMalloc(&m->counter, 4);
    if (e_ == cudaSuccess) e_ = cudaMemsetAsync(m->counter, 0, 4, ctx->stream);
    if (e_ == cudaSuccess) e_ = cudaStreamSynchronize(ctx->stream);
    if (e_ != cudaSuccess) {
        mk_set_error("mk_moe_create: %s", cudaGetErrorString(e_));
        mk_moe_free(ctx, m);
        return e_ == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    *out = m;
    return MK_OK;
}

extern "C" int32_t mk_moe_free(mk_ctx *ctx, mk_moe *m) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr, "NULL argument");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    moe_free_ws(m);
    if (m->wv) cudaFree((void *)m->wv);
    if (m->wsc) cudaFree((void *)m->wsc);
    if (m->tmaps) cudaFree(m->tmaps);
    if (m->rm_vals) cudaFree(m->rm_vals);
    if (m->rm_atoms) cudaFree(m->rm_atoms);
    if (m->gate_w) cudaFree(m->gate_w);
    if (m->gate_b) cudaFree(m->gate_b);
    if (m->counter) cudaFree(m->counter);
    if (m->routed_norm) cudaFree(m->routed_norm);
    delete m;
    return MK_OK;
}

// router logits + top-k on device rows x [n][d]; fills m->ids / m->wts (and the
// forward pair list when with_pairs).
static int32_t moe_route_launch(mk_ctx *ctx, mk_moe *m, const float *x, int n, bool with_pairs) {
    const int E = m->n_experts;
    float *score = m->logits + (size_t)m->cap_rows * E, *key = score + (size_t)m->cap_rows * E;
    {
        mk_prof_scope prof(ctx, MK_PROF_ROUTER);
        const int ewarps = (E + 3) / 4;
        if (m->dx % 4 == 0 && ((uintptr_t)x & 15) == 0) {
            static mk_once_per_device attr;
            if (attr.pending(ctx->device)) {
                MK_CUDA(cudaFuncSetAttribute(moe_router_tile_kernel<RtBig>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RtBig::SMEM));
                MK_CUDA(cudaFuncSetAttribute(moe_router_tile_kernel<RtSmall>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RtSmall::SMEM));
                attr.mark(ctx->device);
            }
            if (n <= RtSmall::NT) {
                moe_router_tile_kernel<RtSmall><<<dim3((unsigned)mk_ceil_div(E, RtSmall::NE), 1), 256, RtSmall::SMEM, ctx->stream>>>(
                    m->gate_w, m->gate_b, x, m->logits, score, key, E, m->dx, n, m->router_kind);
            } else if (n >= 64) {   // fewer tokens leave too few CTAs (a lone CTA of 4 warps takes ~60 us): the 2 x 16 shape is faster there
                static mk_once_per_device attr_g;
                if (attr_g.pending(ctx->device)) {
                    MK_CUDA(cudaFuncSetAttribute(moe_router_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RG_SMEM));
                    attr_g.mark(ctx->device);
                }
                moe_router_gemm_kernel<<<dim3((unsigned)mk_ceil_div(E, RG_TE), (unsigned)mk_ceil_div(n, RG_TT)), RG_THREADS, RG_SMEM, ctx->stream>>>(
                    m->gate_w, m->gate_b, x, m->logits, score, key, E, m->dx, n, m->router_kind);
            } else
                moe_router_tile_kernel<RtBig><<<dim3((unsigned)mk_ceil_div(E, RtBig::NE), (unsigned)mk_ceil_div(n, RtBig::NT)), 256,
                                                RtBig::SMEM, ctx->stream>>>(m->gate_w, m->gate_b, x, m->logits, score, key, E, m->dx, n, m->router_kind);
        } else if (n >= 4) {
            const int64_t warps = (int64_t)ewarps * mk_ceil_div(n, 4);
            moe_router_logits_kernel<4><<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(m->gate_w, m->gate_b, x, m->logits,
                                                                                                       score, key, E, m->dx, n, m->router_kind);
        } else {
            const int64_t warps = (int64_t)ewarps * n;
            moe_router_logits_kernel<1><<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(m->gate_w, m->gate_b, x, m->logits,
                                                                                                       score, key, E, m->dx, n, m->router_kind);
        }
        const size_t smem = (size_t)4 * E * sizeof(float);
        moe_topk_kernel<<<(unsigned)mk_ceil_div(n, 4), 128, smem, ctx->stream>>>(
            score, key, E, m->top_k, n, m->ids, m->wts, with_pairs ? m->pair_row : nullptr, m->pair_expert, m->pair_weight,
            m->has_shared ? 1 : 0, m->router_kind, m->route_scale);
        ctx->launches += 2;
    }
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

constexpr int MOE_TC_MIN_ROWS = 4;
// grouped experts over an explicit pair list (device arrays); x rows already on device
static int32_t moe_experts_launch(mk_ctx *ctx, mk_moe *m, const float *x, int n_rows, const int32_t *pair_row,
                                  const int32_t *pair_expert, const float *pair_weight, int n_pairs, float *outs,
                                  bool prepared = false, bool quantized = false, bool expert_parallel = false) {
    // prepared: the fused router kernel has already grouped the pairs; quantized: and quantized x
    // MK_ACT_FP4X6: from MOE_TC_MIN_ROWS rows up the experts run on the tensor cores (measured at 384 + 1 experts of 7168 x 2048:
    // 4 rows 0.223 -> 0.206 ms, 16 rows 0.657 -> 0.556 ms, 1 row 0.085 -> 0.098 ms, hence not below 4).  The expert-parallel
    // step keeps the q8 kernels (its pair lists and counters are theirs).
    const bool use_tc = m->tc && m->tmaps && !expert_parallel && n_rows >= MOE_TC_MIN_ROWS && m->d % 256 == 0 && m->inter % 256 == 0;
    if (use_tc) {
        // the experts as block-scaled tensor-core products (moe_tc.cuh); work items of up to 16 pairs
        mk_prof_scope prof(ctx, MK_PROF_EXPERTS);
        const int slots = m->n_experts + 1;
        MK_CHECK_ARG(((uintptr_t)x & 15) == 0, "MK_ACT_FP4X6: the token rows must be 16-byte aligned");
        const int64_t limb_threads = (int64_t)n_rows * (m->d / 8);     // 8 columns per thread
        moe_tc_prepare_kernel<<<1 + (unsigned)std::min<int64_t>(mk_ceil_div(limb_threads, 1024), 4 * ctx->sm_count), 1024, (size_t)slots * 4 * sizeof(int),
                                ctx->stream>>>(pair_expert, n_pairs, slots, m->wv, m->sorted, m->items, m->n_items, m->max_items, ctx->status_dev, pair_row,
                                               m->tc_rows_x, m->tc_rows_p, x, n_rows, m->d, m->d, m->xl, m->xsf);
        mtc::TcArgs t;
        t.maps = (const unsigned char *)m->tmaps; t.atoms = m->rm_atoms; t.atom_stride = m->rm_astride; t.rows_x = m->tc_rows_x; t.rows_p = m->tc_rows_p; t.items = m->items; t.n_items = m->n_items; t.sorted = m->sorted; t.pair_row = pair_row;
        t.pair_weight = pair_weight; t.xl = m->xl; t.xsf = m->xsf; t.actl = m->actl; t.actsf = m->actsf; t.outs = outs;
        t.rows = n_rows; t.pairs = m->cap_pairs; t.d = m->d; t.inter = m->inter;
        t.activation = m->activation; t.limit = m->limit; t.status = ctx->status_dev;
        static mk_once_per_device attr;
        if (attr.pending(ctx->device)) {
            MK_CUDA(cudaFuncSetAttribute(mtc::moe_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, mtc::SM_TOTAL));
            MK_CUDA(cudaFuncSetAttribute(mtc::moe_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, mtc::SM_TOTAL));
            attr.mark(ctx->device);
        }
        // persistent CTAs, one per SM; the work units are dealt round-robin inside the kernels
        mtc::moe_tc_kernel<false><<<(unsigned)ctx->sm_count, mtc::THREADS, mtc::SM_TOTAL, ctx->stream>>>(t);
        mtc::moe_tc_kernel<true><<<(unsigned)ctx->sm_count, mtc::THREADS, mtc::SM_TOTAL, ctx->stream>>>(t);
        ctx->launches += 3;
        MK_CUDA(cudaGetLastError());
        return MK_OK;
    }
    if (!quantized) {
        int32_t rc = mk_launch_quantize_act(ctx, x, n_rows, m->d, m->d, m->nbp_d, 0, m->xq, m->xs);
        if (rc != MK_OK) return rc;
    }
    mk_prof_scope prof(ctx, MK_PROF_EXPERTS);
    const int slots = m->n_experts + 1;
    if (!prepared) {
        moe_plan_kernel<<<1, 1024, (size_t)slots * 4 * sizeof(int), ctx->stream>>>(pair_expert, n_pairs, slots, m->wv, m->sorted,
                                                                                  m->items, m->n_items, m->max_items, ctx->status_dev, 8);
        ctx->launches++;
    }
    MoeArgs a;
    a.wv = m->wv; a.wsc = m->wsc; a.items = m->items; a.n_items = m->n_items; a.sorted = m->sorted;
    a.pair_row = pair_row; a.pair_weight = pair_weight; a.xq = m->xq; a.xs = m->xs; a.actq = m->actq; a.acts = m->acts;
    a.outs = outs; a.nbp_d = m->nbp_d; a.nbp_i = m->nbp_i; a.d = m->d; a.inter = m->inter; a.activation = m->activation; a.limit = m->limit;
    a.k = Consts{65536u, 0xFFFFFFFFu, ctx->zeros_dev};
    // an upper bound on the work items of this call (the kernels exit early past *n_items)
    int items_ub = n_pairs / 8 + (n_pairs < slots ? n_pairs : slots);
    if (items_ub > m->max_items) items_ub = m->max_items;
    if (items_ub < 1) items_ub = 1;
    // calls of <= 2 rows have at most 2 pairs per expert: the build without the batched schedule
    // needs fewer registers and keeps 4 CTAs per SM, one wave at batch 1
    const dim3 g1((unsigned)(m->inter / 32), (unsigned)items_ub), g2((unsigned)mk_ceil_div(m->d, 32), (unsigned)items_ub);
    // the kernels of a small call are chained by programmatic stream serialization (each waits for its predecessor itself)
    const bool dep = ctx->pdl != 0;
    if (m->strict) {
        moe_gate_up_kernel<MOE_STRICT><<<g1, MK_G1_KS * 128, 0, ctx->stream>>>(a);
        moe_down_kernel<MOE_STRICT><<<g2, 256, 0, ctx->stream>>>(a);
    } else if (n_rows <= 2) {
        mk_launch_dep(dep, moe_gate_up_kernel<MOE_ALL_SPREAD>, g1, dim3(MK_G1_KS * 128), 0, ctx->stream, a);
        mk_launch_dep(dep, moe_down_kernel<MOE_ALL_SPREAD>, g2, dim3(256), 0, ctx->stream, a);
    } else if (n_rows <= MK_MOE_MIXED_MAX) {
        mk_launch_dep(dep, moe_gate_up_kernel<MOE_MIXED>, g1, dim3(MK_G1_KS * 128), 0, ctx->stream, a);
        mk_launch_dep(dep, moe_down_kernel<MOE_MIXED>, g2, dim3(256), 0, ctx->stream, a);
    } else {
        moe_gate_up_kernel<MOE_BIG_ITEMS><<<g1, MK_G1_KS * 128, 0, ctx->stream>>>(a);
        moe_gate_up_kernel<MOE_SMALL_ITEMS><<<g1, MK_G1_KS * 128, 0, ctx->stream>>>(a);
        moe_down_kernel<MOE_BIG_ITEMS><<<g2, 256, 0, ctx->stream>>>(a);
        moe_down_kernel<MOE_SMALL_ITEMS><<<g2, 256, 0, ctx->stream>>>(a);
        ctx->launches += 2;
    }
    ctx->launches += 2;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

extern "C" int32_t mk_moe_combine_dev(mk_ctx *ctx, const float *outs, int32_t n_tokens, int32_t slots, int32_t d, float *out) {
    MK_CHECK_ARG(ctx != nullptr && outs != nullptr && out != nullptr && n_tokens > 0 && slots > 0 && d > 0, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_prof_scope prof(ctx, MK_PROF_EXPERTS);
    mk_launch_dep(ctx->pdl != 0, moe_combine_kernel, dim3((unsigned)mk_ceil_div((int64_t)n_tokens * d, 256)), dim3(256), 0, ctx->stream, outs, n_tokens, slots, d, out);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

extern "C" int32_t mk_moe_route_dev(mk_ctx *ctx, mk_moe *m, const float *x, int32_t n, int32_t *ids, float *weights, float *logits) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && x != nullptr && n > 0, "bad argument");
    MK_CHECK_ARG(m->has_router, "this MoE object was created without a router");
    MK_CUDA(cudaSetDevice(ctx->device));
    int32_t rc = moe_reserve(ctx, m, n, n * (m->top_k + 1));
    if (rc != MK_OK) return rc;
    rc = moe_route_launch(ctx, m, x, n, false);
    if (rc != MK_OK) return rc;
    if (ids) MK_CUDA(cudaMemcpyAsync(ids, m->ids, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (weights) MK_CUDA(cudaMemcpyAsync(weights, m->wts, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (logits) MK_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)n * m->n_experts * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_moe_experts_dev(mk_ctx *ctx, mk_moe *m, const float *x, int32_t n_rows, const int32_t *pair_row,
                                      const int32_t *pair_expert, const float *pair_weight, int32_t n_pairs, float *outs) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && x != nullptr && pair_row != nullptr && pair_expert != nullptr &&
                     pair_weight != nullptr && outs != nullptr, "NULL argument");
    MK_CHECK_ARG(n_rows > 0 && n_pairs > 0, "n_rows and n_pairs must be positive");
    MK_CUDA(cudaSetDevice(ctx->device));
    int32_t rc = moe_reserve(ctx, m, n_rows, n_pairs);
    if (rc != MK_OK) return rc;
    return moe_experts_launch(ctx, m, x, n_rows, pair_row, pair_expert, pair_weight, n_pairs, outs);
}

// out[t][j] = slot-order sum of the pair rows (as moe_combine_kernel), then rmsnorm over the row (src/model.rs:2346-2356):
// one CTA per token, the row in shared memory, dot(y, y) in the engine's 8-accumulator order by warp 0.
__global__ void __launch_bounds__(256) moe_combine_norm_kernel(const float *__restrict__ outs, int slots, int d, const float *__restrict__ nw,
                                                              float eps, float *__restrict__ y_out, float *__restrict__ yn_out) {
    extern __shared__ float ysm[];
    __shared__ float s_inv;
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < d; j += blockDim.x) {
        float v = 0.0f;
        for (int s = 0; s < slots; ++s) v = __fadd_rn(v, outs[((int64_t)t * slots + s) * d + j]);
        ysm[j] = v;
        if (y_out) y_out[(int64_t)t * d + j] = v;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x, j8 = lane & 7, full = d & ~7;
        float acc = 0.0f;
        for (int c = 0; c < full; c += 8) acc = __fadd_rn(acc, __fmul_rn(ysm[c + j8], ysm[c + j8]));
        float ss = mkf::reduce8(acc, lane);
        for (int c = full; c < d; ++c) ss = __fadd_rn(ss, __fmul_rn(ysm[c], ysm[c]));
        if (lane == 0) s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)d), eps)));
    }
    __syncthreads();
    for (int j = threadIdx.x; j < d; j += blockDim.x) yn_out[(int64_t)t * d + j] = __fmul_rn(__fmul_rn(ysm[j], s_inv), nw[j]);
}
__global__ void __launch_bounds__(256) moe_add_rows_kernel(float *__restrict__ out, const float *__restrict__ b, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(out[i], b[i]);
}

// One token through a narrow router (d <= 2048): 32 experts per CTA, each row's dot by one lane octet.
using RtOne = mkf::TileShape<32, 1, 256, 3>;   // one token: few, long slices - the router rows come cold from HBM and every slice wait is a round trip

// The K3 latent layer for one token, as independent chains (see mk_moe_forward_k3_split in mk_common.cuh):
//   main : [routed_down; shared gate; shared up] x  (one stacked matvec) -> q8 of h -> (router done) gate/up -> down ->
//          slot-order sum + rmsnorm -> routed_up
//   side0: router logits, top-k and grouping (needs only x)
//   side1: SiTU of the shared pair -> shared down (needs the stacked matvec)
static int32_t moe_k3_decode(mk_ctx *ctx, mk_moe *m, const float *x, float *out_routed, float *out_shared) {
    const int n = 1, slots = m->top_k;
    int32_t rc = moe_reserve(ctx, m, n, n * slots);
    if (rc != MK_OK) return rc;
    const int si = m->shared_inter, lat = m->latent;
    float *h = m->stk, *sa = m->stk + lat, *su = sa + si;
    rc = mk_fork(ctx, 0);
    if (rc != MK_OK) return rc;
    {   // side 0: the router
        mk_on_side on(ctx, 0);
        RouterFusedArgs ra;
        ra.gate_w = m->gate_w; ra.gate_b = m->gate_b; ra.x = x; ra.logits = m->logits;
        ra.score = m->logits + (size_t)m->cap_rows * m->n_experts; ra.key = ra.score + (size_t)m->cap_rows * m->n_experts;
        ra.n_experts = m->n_experts; ra.d = m->dx; ra.n_tokens = n; ra.top_k = m->top_k; ra.shared_slot = 0;
        ra.router_kind = m->router_kind; ra.route_scale = m->route_scale;
        ra.ids = m->ids; ra.wts = m->wts; ra.pair_row = m->pair_row; ra.pair_expert = m->pair_expert; ra.pair_weight = m->pair_weight;
        ra.wv = m->wv; ra.sorted = m->sorted; ra.items = m->items; ra.n_items = m->n_items; ra.max_items = m->max_items;
        ra.status = ctx->status_dev; ra.counter = m->counter; ra.xq = m->xq; ra.xs = m->xs; ra.nbp = m->nbp_d;
        ra.ep_rank = 0; ra.ep_world = 0; ra.n_local = nullptr;
        size_t smem_f = RtOne::SMEM;
        if ((size_t)8 * m->n_experts * 4 > smem_f) smem_f = (size_t)8 * m->n_experts * 4;
        mk_prof_scope prof(ctx, MK_PROF_ROUTER);
        static mk_once_per_device attr;
        if (attr.pending(ctx->device)) {
            MK_CUDA(cudaFuncSetAttribute(moe_router_fused_kernel<RtOne>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr.mark(ctx->device);
        }
        moe_router_fused_kernel<RtOne><<<(unsigned)mk_ceil_div(m->n_experts, RtOne::NE), 256, smem_f, ctx->stream>>>(ra);
        ctx->launches++;
        MK_CUDA(cudaGetLastError());
    }
    rc = mk_launch_f32_gemv(ctx, m->routed_down, lat + 2 * si, m->dx, x, 1, h, lat + 2 * si, 0);
    if (rc != MK_OK) return rc;
    rc = mk_fork(ctx, 1);
    if (rc != MK_OK) return rc;
    {   // side 1: the f32 shared expert (src/model.rs:2357-2378)
        mk_on_side on(ctx, 1);
        rc = mk_launch_situ(ctx, sa, su, si, sa);
        if (rc == MK_OK) rc = mk_launch_f32_gemv(ctx, m->sh_down, m->dx, si, sa, 1, out_shared, m->dx, 0);
        if (rc != MK_OK) return rc;
    }
    rc = mk_launch_quantize_act(ctx, h, 1, lat, lat, m->nbp_d, 0, m->xq, m->xs);
    if (rc != MK_OK) return rc;
    rc = mk_join(ctx, 0);
    if (rc != MK_OK) return rc;
    rc = moe_experts_launch(ctx, m, h, 1, m->pair_row, m->pair_expert, m->pair_weight, slots, m->outs, true, true);
    if (rc != MK_OK) return rc;
    {
        mk_prof_scope prof(ctx, MK_PROF_EXPERTS);
        moe_combine_norm_kernel<<<1, 256, (size_t)lat * 4, ctx->stream>>>(m->outs, slots, lat, m->routed_norm, m->rms_eps, m->lat_y, m->lat_yn);
        ctx->launches++;
        MK_CUDA(cudaGetLastError());
    }
    rc = mk_launch_f32_gemv(ctx, m->routed_up, m->dx, lat, m->lat_yn, 1, out_routed, m->dx, 0);
    if (rc != MK_OK) return rc;
    return mk_join(ctx, 1);
}
static bool moe_k3_decode_ok(const mk_ctx *ctx, const mk_moe *m, const float *x, int n) {
    return n == 1 && m->has_router && m->latent > 0 && m->stack3 && m->sh_gate && !m->has_shared && m->dx % 4 == 0 && m->dx <= 2048 &&
           m->latent % 4 == 0 && m->shared_inter % 4 == 0 && ((uintptr_t)x & 15) == 0 && (size_t)8 * m->n_experts * 4 <= 200 * 1024 &&
           !ctx->moe_no_fuse;
}
int32_t mk_moe_forward_k3_split(mk_ctx *ctx, mk_moe *m, const float *x, float *out_routed, float *out_shared) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && x != nullptr && out_routed != nullptr && out_shared != nullptr, "NULL argument");
    if (!moe_k3_decode_ok(ctx, m, x, 1)) return MK_ERR_UNSUPPORTED;
    MK_CUDA(cudaSetDevice(ctx->device));
    return moe_k3_decode(ctx, m, x, out_routed, out_shared);
}

static int32_t moe_forward_impl(mk_ctx *ctx, mk_moe *m, mk_moe_ep *ep, const float *x, int32_t n, float *out, int32_t *ids, float *weights) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && x != nullptr && out != nullptr && n > 0, "bad argument");
    MK_CHECK_ARG(m->has_router, "this MoE object was created without a router");
    MK_CUDA(cudaSetDevice(ctx->device));
    const int slots = m->top_k + (m->has_shared ? 1 : 0);
    int32_t rc = moe_reserve(ctx, m, n, n * slots);
    if (rc != MK_OK) return rc;
    if (ep == nullptr && moe_k3_decode_ok(ctx, m, x, n)) {
        // one token of the K3 layer: independent chains on side streams, then out = routed + shared (src/model.rs:2375-2377)
        rc = moe_k3_decode(ctx, m, x, out, m->sh_out);
        if (rc != MK_OK) return rc;
        moe_add_rows_kernel<<<(unsigned)mk_ceil_div(m->dx, 256), 256, 0, ctx->stream>>>(out, m->sh_out, m->dx);
        ctx->launches++;
        MK_CUDA(cudaGetLastError());
        if (ids) MK_CUDA(cudaMemcpyAsync(ids, m->ids, (size_t)m->top_k * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        if (weights) MK_CUDA(cudaMemcpyAsync(weights, m->wts, (size_t)m->top_k * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        return MK_OK;
    }
    // K3 latent MoE: the experts work on h = routed_down x (src/model.rs:2202-2204)
    const float *xe = x;
    if (m->latent > 0) {
        rc = mk_launch_f32_gemv(ctx, m->routed_down, m->latent, m->dx, x, n, m->lat_h, m->latent, 0);
        if (rc != MK_OK) return rc;
        xe = m->lat_h;
    }
    // small batches: router logits, activation quantization, top-k and pair grouping in ONE launch
    const bool small = n <= RtSmall::NT;
    size_t smem_f = small ? RtSmall::SMEM : RtBig::SMEM;
    if ((size_t)8 * m->n_experts * 4 > smem_f) smem_f = (size_t)8 * m->n_experts * 4;
    if ((size_t)3 * n * slots * 4 > smem_f) smem_f = (size_t)3 * n * slots * 4;
    const bool fused = n <= 16 && m->dx % 4 == 0 && ((uintptr_t)x & 15) == 0 && smem_f <= 200 * 1024 && (!ctx->moe_no_fuse || ep);
    MK_CHECK_ARG(ep == nullptr || (fused && n <= ep->max_tokens && slots == ep->slots && m->d == ep->d && (ep->connected || ep->world == 1)),
                 "expert-parallel call: needs <= max_tokens (<= 16) aligned rows and a connected exchange object made for this layer");
    const bool tc_call = m->tc && m->tmaps && ep == nullptr && n >= MOE_TC_MIN_ROWS;   // the tensor-core experts make their own limbs
    const bool fused_q = fused && m->latent == 0 && !tc_call; // the router's rows are the experts' rows: quantize them in the same launch
    if (fused) {
        RouterFusedArgs ra;
        ra.gate_w = m->gate_w; ra.gate_b = m->gate_b; ra.x = x; ra.logits = m->logits;
        ra.score = m->logits + (size_t)m->cap_rows * m->n_experts; ra.key = ra.score + (size_t)m->cap_rows * m->n_experts;
        ra.n_experts = m->n_experts; ra.d = m->dx; ra.n_tokens = n; ra.top_k = m->top_k; ra.shared_slot = m->has_shared ? 1 : 0;
        ra.router_kind = m->router_kind; ra.route_scale = m->route_scale;
        ra.ids = m->ids; ra.wts = m->wts; ra.pair_row = m->pair_row; ra.pair_expert = m->pair_expert; ra.pair_weight = m->pair_weight;
        ra.wv = m->wv; ra.sorted = m->sorted; ra.items = m->items; ra.n_items = m->n_items; ra.max_items = m->max_items;
        ra.status = ctx->status_dev; ra.counter = m->counter; ra.xq = m->xq; ra.xs = m->xs; ra.nbp = m->nbp_d;
        ra.ep_rank = ep ? ep->rank : 0; ra.ep_world = ep ? ep->world : 0; ra.n_local = ep ? ep->n_local : nullptr;
        const unsigned qctas = fused_q ? (unsigned)mk_ceil_div((int64_t)n * m->nbp_d, 8) : 0u;
        {
            mk_prof_scope prof(ctx, MK_PROF_ROUTER);
            static mk_once_per_device attr;
            if (attr.pending(ctx->device)) {
                MK_CUDA(cudaFuncSetAttribute(moe_router_fused_kernel<RtBig>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                MK_CUDA(cudaFuncSetAttribute(moe_router_fused_kernel<RtSmall>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                attr.mark(ctx->device);
            }
            if (small)
                moe_router_fused_kernel<RtSmall><<<(unsigned)mk_ceil_div(m->n_experts, RtSmall::NE) + qctas, 256, smem_f, ctx->stream>>>(ra);
            else
                moe_router_fused_kernel<RtBig><<<(unsigned)mk_ceil_div(m->n_experts, RtBig::NE) + qctas, 256, smem_f, ctx->stream>>>(ra);
            ctx->launches++;
        }
        MK_CUDA(cudaGetLastError());
    } else {
        rc = moe_route_launch(ctx, m, x, n, true);
        if (rc != MK_OK) return rc;
    }
    float *outs = m->outs;
    if (ep) {
        // the (token, slot) table of this step lives in the exchange buffer: local pairs are written by the
        // expert kernels, the others arrive from their ranks
        ep->step++;
        const uint32_t par = ep->step & 1u;
        outs = (float *)((char *)ep->blob + 256 + (size_t)par * ep->par_bytes);
        rc = moe_experts_launch(ctx, m, xe, n, m->pair_row, m->pair_expert, m->pair_weight, n * slots, outs, true, fused_q, true);
        if (rc != MK_OK) return rc;
        EpPeers pe;
        memset(&pe, 0, sizeof(pe));
        for (int r = 0; r < ep->world; ++r) {
            pe.outs[r] = (float *)((char *)ep->peer[r] + 256 + (size_t)par * ep->par_bytes);
            pe.flag[r] = (uint32_t *)ep->peer[r] + par * 8 + ep->rank;
        }
        mk_prof_scope prof(ctx, MK_PROF_EXPERTS);
        moe_ep_exchange_kernel<<<(unsigned)(n * slots), 256, 0, ctx->stream>>>(pe, outs, m->sorted, ep->n_local, m->d, ep->rank, ep->world,
                                                                             (const uint32_t *)ep->blob + par * 8, ep->counter, ctx->status_dev);
        ctx->launches++;
        MK_CUDA(cudaGetLastError());
    } else {
        rc = moe_experts_launch(ctx, m, xe, n, m->pair_row, m->pair_expert, m->pair_weight, n * slots, outs, fused, fused_q);
        if (rc != MK_OK) return rc;
    }
    // slot-order sum (for MK_MOE_SITU the terms already carry their routing weights)
    rc = mk_moe_combine_dev(ctx, outs, n, slots, m->d, m->latent > 0 ? m->lat_y : out);
    if (rc != MK_OK) return rc;
    if (m->latent > 0) {
        // norm BEFORE the up projection (src/model.rs:2352-2356)
        rc = mk_launch_rmsnorm(ctx, m->lat_y, m->routed_norm, n, m->latent, m->rms_eps, m->lat_yn);
        if (rc != MK_OK) return rc;
        rc = mk_launch_f32_gemv(ctx, m->routed_up, m->dx, m->latent, m->lat_yn, n, out, m->dx, 0);
        if (rc != MK_OK) return rc;
    }
    if (m->sh_gate) {
        // f32 shared expert on the layer input, added to the routed output (src/model.rs:2357-2378)
        const int si = m->shared_inter;
        rc = mk_launch_f32_gemv(ctx, m->sh_gate, si, m->dx, x, n, m->sh_a, si, 0);
        if (rc == MK_OK) rc = mk_launch_f32_gemv(ctx, m->sh_up, si, m->dx, x, n, m->sh_u, si, 0);
        if (rc == MK_OK) rc = mk_launch_situ(ctx, m->sh_a, m->sh_u, (int64_t)n * si, m->sh_a);
        if (rc == MK_OK) rc = mk_launch_f32_gemv(ctx, m->sh_down, m->dx, si, m->sh_a, n, out, m->dx, 1);
        if (rc != MK_OK) return rc;
    }
    if (ids) MK_CUDA(cudaMemcpyAsync(ids, m->ids, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    if (weights) MK_CUDA(cudaMemcpyAsync(weights, m->wts, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToDevice, ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_moe_forward_dev(mk_ctx *ctx, mk_moe *m, const float *x, int32_t n, float *out, int32_t *ids, float *weights) {
    return moe_forward_impl(ctx, m, nullptr, x, n, out, ids, weights);
}

extern "C" int32_t mk_moe_forward_ep_dev(mk_ctx *ctx, mk_moe *m, mk_moe_ep *ep, const float *x, int32_t n, float *out, int32_t *ids,
                                         float *weights) {
    MK_CHECK_ARG(ep != nullptr, "NULL exchange object");
    return moe_forward_impl(ctx, m, ep, x, n, out, ids, weights);
}

extern "C" int32_t mk_moe_ep_create(mk_ctx *ctx, const mk_moe *m, int32_t rank, int32_t world, int32_t max_tokens, mk_moe_ep **out,
                                    uint8_t *handle /* 64 bytes */) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && out != nullptr && handle != nullptr, "NULL argument");
    MK_CHECK_ARG(world >= 1 && world <= 8 && rank >= 0 && rank < world, "need 0 <= rank < world <= 8");
    MK_CHECK_ARG(max_tokens >= 1 && max_tokens <= 16, "max_tokens must be in [1, 16]");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    *out = nullptr;
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_moe_ep *ep = new (std::nothrow) mk_moe_ep();
    if (!ep) return MK_ERR_OOM;
    memset(ep, 0, sizeof(*ep));
    ep->rank = rank; ep->world = world; ep->max_tokens = max_tokens;
    ep->slots = m->top_k + (m->has_shared ? 1 : 0);
    ep->d = m->d;
    ep->par_bytes = (size_t)max_tokens * ep->slots * ep->d * 4;
    ep->blob_bytes = 256 + 2 * ep->par_bytes;
    cudaError_t e = cudaMalloc(&ep->blob, ep->blob_bytes);
    if (e == cudaSuccess) e = cudaMemset(ep->blob, 0, ep->blob_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&ep->n_local, 4);
    if (e == cudaSuccess) e = cudaMalloc(&ep->counter, 8);      // [0] finished CTAs of the running exchange, [1] steps finished
    if (e == cudaSuccess) e = cudaMemset(ep->n_local, 0, 4);
    if (e == cudaSuccess) e = cudaMemset(ep->counter, 0, 8);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ep->blob);
    if (e != cudaSuccess) {
        mk_set_error("mk_moe_ep_create: %s", cudaGetErrorString(e));
        if (ep->blob) cudaFree(ep->blob);
        if (ep->n_local) cudaFree(ep->n_local);
        if (ep->counter) cudaFree(ep->counter);
        delete ep;
        return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    memcpy(handle, &h, 64);
    ep->peer[rank] = ep->blob;
    *out = ep;
    return MK_OK;
}

extern "C" int32_t mk_moe_ep_connect(mk_ctx *ctx, mk_moe_ep *ep, const uint8_t *handles /* [world][64], by rank */) {
    MK_CHECK_ARG(ctx != nullptr && ep != nullptr && handles != nullptr, "NULL argument");
    MK_CHECK_ARG(!ep->connected, "already connected");
    MK_CUDA(cudaSetDevice(ctx->device));
    for (int r = 0; r < ep->world; ++r) {
        if (r == ep->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        bool zero = true;
        for (int b = 0; b < 64; ++b) zero = zero && handles[(size_t)r * 64 + b] == 0;
        cudaError_t e = cudaSuccess;
        if (zero) { // the rank never joined: its table rows go to local scratch, its flag never arrives, the wait runs out
            if (!ep->absent) e = cudaMalloc(&ep->absent, ep->blob_bytes);
            if (e == cudaSuccess) e = cudaMemset(ep->absent, 0, ep->blob_bytes);
            ep->peer[r] = ep->absent;
            ep->is_absent[r] = true;
        } else {
            e = cudaIpcOpenMemHandle(&ep->peer[r], h, cudaIpcMemLazyEnablePeerAccess);
        }
        if (e != cudaSuccess) {
            mk_set_error("mk_moe_ep_connect: rank %d cannot open rank %d's buffer: %s", ep->rank, r, cudaGetErrorString(e));
            for (int q = 0; q < r; ++q)
                if (q != ep->rank && ep->peer[q] && !ep->is_absent[q]) { cudaIpcCloseMemHandle(ep->peer[q]); ep->peer[q] = nullptr; }
            return MK_ERR_CUDA;
        }
    }
    ep->connected = true;
    return MK_OK;
}

extern "C" int32_t mk_moe_ep_free(mk_ctx *ctx, mk_moe_ep *ep) {
    MK_CHECK_ARG(ctx != nullptr && ep != nullptr, "NULL argument");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < ep->world; ++r)
        if (r != ep->rank && ep->peer[r] && !ep->is_absent[r]) cudaIpcCloseMemHandle(ep->peer[r]);
    if (ep->absent) cudaFree(ep->absent);
    if (ep->blob) cudaFree(ep->blob);
    if (ep->n_local) cudaFree(ep->n_local);
    if (ep->counter) cudaFree(ep->counter);
    delete ep;
    return MK_OK;
}

// host-pointer variants: stage through the context's device buffer
extern "C" int32_t mk_moe_route(mk_ctx *ctx, mk_moe *m, const float *x, int32_t n, int32_t *ids, float *weights, float *logits) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && x != nullptr && n > 0, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const size_t xb = (size_t)n * m->dx * 4;
    int32_t rc = mk_io_reserve(ctx, mk_align_up(xb, 256));
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(ctx->io_dev, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = mk_moe_route_dev(ctx, m, (const float *)ctx->io_dev, n, nullptr, nullptr, nullptr);
    if (rc != MK_OK) return rc;
    if (ids) MK_CUDA(cudaMemcpyAsync(ids, m->ids, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (weights) MK_CUDA(cudaMemcpyAsync(weights, m->wts, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (logits) MK_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)n * m->n_experts * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_moe_forward(mk_ctx *ctx, mk_moe *m, const float *x, int32_t n, float *out, int32_t *ids, float *weights) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && x != nullptr && out != nullptr && n > 0, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const size_t xb = mk_align_up((size_t)n * m->dx * 4, 256);
    int32_t rc = mk_io_reserve(ctx, 2 * xb);
    if (rc != MK_OK) return rc;
    float *dx = (float *)ctx->io_dev, *dout = (float *)((char *)ctx->io_dev + xb);
    MK_CUDA(cudaMemcpyAsync(dx, x, (size_t)n * m->dx * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = mk_moe_forward_dev(ctx, m, dx, n, dout, nullptr, nullptr);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(out, dout, (size_t)n * m->dx * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (ids) MK_CUDA(cudaMemcpyAsync(ids, m->ids, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (weights) MK_CUDA(cudaMemcpyAsync(weights, m->wts, (size_t)n * m->top_k * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

