// Vocabulary-sharded lm_head across the GPUs of one node without a collective library
// call on the decode path.  The matvec kernel of rank r writes its logits rows into rank
// r's own gather buffer; ONE exchange kernel (a few CTAs) then pushes that slice into the
// gather buffers of all other ranks (peer memory over NVLink, 16-byte stores); each CTA ends
// with a barrier and one system-wide fence and counts itself in, the last one to arrive
// publishes this rank's step number in every rank's flag word (st.release.sys) and waits,
// bounded, until all ranks have published the current step (ld.acquire.sys).
// Phases of the exchange kernel, stamped with %globaltimer on 4 GPUs (40960 rows per rank): copy 3.8 us, fence + count
// 4-6.5 us, flag store 2.3 us, wait for the slowest rank 0.4-7 us.  Measured alternative, rejected: no counter, every
// CTA releasing its own flag to every rank (16 x world st.release.sys) - 28 us against 22 us per step at 4 GPUs.
// Measured alternative, rejected: storing the rows to the peers from the matvec kernel's own
// epilogue (4-byte peer stores from every CTA) made the matvec 12 % slower at 2 GPUs (105 vs
// 94 us) - with or without a system-wide fence per CTA - which costs more than this push.
//
// The reference engine is single-process (no rank concept), so there is no reference code
// for this file; what it preserves is the single-GPU result: the gathered logits are the
// bits one GPU computes for the whole matrix (rows are independent), and the greedy pick is
// the first index of the maximum (src/model.rs:3277-3290).
// Token-only step (mk_matvec_q8_gather_token_dev: greedy decode needs the token, not the logits of the other shards):
// the rows stay where the matvec wrote them, only the 16-byte (maximum, index) pair of every rank crosses NVLink;
// same kernel, same flags, no row copy and no system-wide fence per CTA.
//
// Buffers: one cudaMalloc blob per rank, exported with cudaIpcGetMemHandle and opened by the
// other ranks: [flags: 2 parities x 8 ranks u32][pad to 256 B][(maximum, index) pairs: 2 parities x 8 ranks x 2 tokens x 16 B]
// [logits: 2 x max_batch x vocab f32].
// Two parities: a rank may run one step ahead of a peer that still reads the previous logits.
// A rank cannot get two steps ahead: its wait for step s+1 needs the peer's flag of s+1, which
// the peer publishes after (stream order) it has consumed step s.
#include "mk_common.cuh"

#include <new>

struct mk_gather {
    int rank, world, max_batch;
    int64_t vocab;
    size_t logits_off, blob_bytes;
    void *blob;        // local
    void *peer[8];     // blobs of all ranks (peer[rank] == blob)
    void *scratch;     // device: per-CTA (maximum, index) partials [32][2], then the CTA counter
    void *absent;      // stand-in target for ranks that have not joined (all-zero handle): local scratch
    bool is_absent[8];
    bool connected;
    uint32_t step;     // host mirror of the device step count: picks the buffer parity of a call
};

// a recorded token replays exchange steps that the host did not issue one by one: keep the mirror in step
uint32_t mk_gather_steps(const mk_gather *g) { return g->step; }
void mk_gather_note_replay(mk_gather *g, uint32_t n) { g->step += n; }

namespace {
constexpr uint32_t GATHER_WAIT_LIMIT = 1u << 22; // polls of >= 100 ns each: about half a second

struct Best { float v; int64_t i; };
// first index of the maximum (src/model.rs:3277-3290): a larger value wins, an equal value only with a lower index
__device__ __forceinline__ Best better(Best a, Best b) { return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a; }

// gridDim.x CTAs share this rank's slice [batch][n] (row stride ld), each a contiguous range of 16-byte pieces, read
// once: every piece goes to the same place in every other rank's buffer and into the CTA's running (maximum,
// index), which lands in `partials`.  Every CTA fences system-wide and counts itself in; the last one to arrive
// folds the partials, sends this rank's (maximum, index) pairs to every rank, fences, lane r publishes this rank's
// step in rank r's flag word and waits for rank r's flag here to reach `step`; finally thread b picks token b's
// winner among the ranks' pairs.  Without 16-byte alignment the host launches one CTA and it copies by floats.
constexpr int GATHER_MAX_CTAS = 32, GATHER_PIECES_PER_CTA = 2048;
struct GatherPeers { float *dst[8]; uint32_t *flag[8]; Best *pairs[8]; };
__global__ void __launch_bounds__(1024) gather_exchange_kernel(const GatherPeers pe, const float *__restrict__ src, int batch, int64_t n,
                                                              int64_t ld, int64_t row0, int rank, int world,
                                                              const uint32_t *__restrict__ flags, const Best *__restrict__ my_pairs,
                                                              int32_t *__restrict__ argmax, int32_t *__restrict__ status,
                                                              Best *__restrict__ partials, unsigned *__restrict__ counter, bool push) {
    __shared__ Best red[32];
    __shared__ int s_last;
    // the step number lives on the device (counter[1] = steps finished so far), not in the launch arguments: a recorded
    // launch (CUDA graph) must publish a new number at every replay.  Every thread reads it here; the last CTA, which
    // writes the new value at its end, is the one that saw all other CTAs count in after this read.
    asm volatile("griddepcontrol.wait;" ::: "memory");   // launched behind the matvec with programmatic stream serialization
    const uint32_t step = *(volatile const unsigned *)(counter + 1) + 1u;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, ncta = gridDim.x, cta = blockIdx.x;
    const bool vec = (n % 4 == 0) && (ld % 4 == 0) && (row0 % 4 == 0) && (((uintptr_t)src & 15) == 0);
    for (int b = 0; b < batch; ++b) {
        const float *s = src + (int64_t)b * ld;
        Best best = {-INFINITY, INT64_MAX};
        if (vec) {
            // up to 4 independent 16-byte loads in flight per thread
            const int64_t n4 = n / 4, per = (n4 + ncta - 1) / ncta, lo = cta * per, hi = min(n4, lo + per), stride = blockDim.x;
            for (int64_t i0 = lo + tid; i0 < hi; i0 += 4 * stride) {
                float4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t i = i0 + u * stride;
                    v[u] = i < hi ? __ldcg((const float4 *)s + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int64_t i = i0 + u * stride;
                    if (i >= hi) continue;
                    if (push)
                        for (int p = 0; p < world; ++p)
                            if (p != rank) ((float4 *)(pe.dst[p] + (int64_t)b * ld))[i] = v[u];
                    best = better(best, Best{v[u].x, 4 * i});
                    best = better(best, Best{v[u].y, 4 * i + 1});
                    best = better(best, Best{v[u].z, 4 * i + 2});
                    best = better(best, Best{v[u].w, 4 * i + 3});
                }
            }
        } else if (cta == 0) {
            for (int64_t i = tid; i < n; i += blockDim.x) {
                const float v = s[i];
                if (push)
                    for (int p = 0; p < world; ++p)
                        if (p != rank) pe.dst[p][(int64_t)b * ld + i] = v;
                best = better(best, Best{v, i});
            }
        }
        for (int o = 16; o > 0; o >>= 1) {
            Best other = {__shfl_xor_sync(0xFFFFFFFFu, best.v, o), __shfl_xor_sync(0xFFFFFFFFu, best.i, o)};
            best = better(best, other);
        }
        if (lane == 0) red[warp] = best;
        __syncthreads();
        if (warp == 0) {
            best = lane < (int)(blockDim.x >> 5) ? red[lane] : Best{-INFINITY, INT64_MAX};
            for (int o = 16; o > 0; o >>= 1) {
                Best other = {__shfl_xor_sync(0xFFFFFFFFu, best.v, o), __shfl_xor_sync(0xFFFFFFFFu, best.i, o)};
                best = better(best, other);
            }
            if (lane == 0) partials[cta * 2 + b] = best;
        }
        __syncthreads();
    }
    // Release by one thread for the CTA: the barrier orders every thread's peer stores and the partials before
    // thread 0's system-wide fence (fences are cumulative), the fence before the count; the last CTA's thread 0
    // fences again after it saw the full count (acquire side) and the second barrier hands that to its flag writers.
    __syncthreads();
    if (tid == 0) {
        if (push) __threadfence_system();
        else __threadfence();          // token-only step: nothing of this CTA left the GPU, the partials are for the last CTA here
        const unsigned prev = atomicAdd(counter, 1u);
        s_last = prev == (unsigned)ncta - 1 ? 1 : 0;
        if (s_last) {
            *counter = 0u;
            __threadfence();   // acquire side towards the other CTAs of this GPU; the flag's st.release.sys below is the system-wide release
        }
    }
    __syncthreads();
    if (!s_last) return;
    if (warp == 0) {
        for (int b = 0; b < batch; ++b) {
            Best best = {-INFINITY, INT64_MAX};
            if (lane < ncta) {
                best.v = __ldcg(&partials[lane * 2 + b].v);
                best.i = __ldcg(&partials[lane * 2 + b].i);
            }
            for (int o = 16; o > 0; o >>= 1) {
                Best other = {__shfl_xor_sync(0xFFFFFFFFu, best.v, o), __shfl_xor_sync(0xFFFFFFFFu, best.i, o)};
                best = better(best, other);
            }
            if (lane < world) pe.pairs[lane][b] = Best{best.v, best.i == INT64_MAX ? row0 : row0 + best.i}; // this rank's pair, to rank `lane`
        }
    }
    // thread r (a lane of warp 0) wrote rank r's pairs itself: its release store below orders them, and everything
    // the barriers above made visible to it, before the flag
    if (tid < world) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pe.flag[tid]), "r"(step) : "memory");
        bool ok = false;
        uint64_t t0, t1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        for (uint32_t it = 0; it < GATHER_WAIT_LIMIT; ++it) {   // bounded twice: by polls and by one second of wall time
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + tid) : "memory");
            if ((int32_t)(v - step) >= 0) { ok = true; break; }
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > 1000000000ull) break;
            __nanosleep(100);
        }
        if (!ok) atomicCAS(status, 0, MK_ERR_TIMEOUT);
    }
    // thread r acquired rank r's flag (ld.acquire.sys); the barrier hands what that made visible to the threads that read the pairs
    __syncthreads();
    if (argmax != nullptr && tid < batch) {
        Best best = {-INFINITY, INT64_MAX};
        for (int r = 0; r < world; ++r) {
            Best q;
            q.v = __ldcv(&my_pairs[(int64_t)r * 2 + tid].v);
            q.i = __ldcv(&my_pairs[(int64_t)r * 2 + tid].i);
            best = better(best, q);
        }
        argmax[tid] = (int32_t)best.i;
    }
    if (tid == 0) counter[1] = step;
}
} // namespace

extern "C" int32_t mk_gather_create(mk_ctx *ctx, int32_t rank, int32_t world, int64_t vocab, int32_t max_batch, mk_gather **out,
                                    uint8_t *handle /* 64 bytes */) {
    MK_CHECK_ARG(ctx != nullptr && out != nullptr && handle != nullptr, "NULL argument");
    MK_CHECK_ARG(world >= 1 && world <= 8 && rank >= 0 && rank < world, "need 0 <= rank < world <= 8");
    MK_CHECK_ARG(vocab > 0 && max_batch >= 1 && max_batch <= 2, "vocab > 0 and max_batch in [1, 2] required");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    *out = nullptr;
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_gather *g = new (std::nothrow) mk_gather();
    if (!g) return MK_ERR_OOM;
    memset(g, 0, sizeof(*g));
    g->rank = rank; g->world = world; g->max_batch = max_batch; g->vocab = vocab;
    g->logits_off = 256 + 2 * 8 * 2 * sizeof(Best); // flags, pairs, then the logits (768 B in: 16-byte aligned)
    g->blob_bytes = g->logits_off + (size_t)2 * max_batch * vocab * 4;
    cudaError_t e = cudaMalloc(&g->blob, g->blob_bytes);
    if (e == cudaSuccess) e = cudaMemset(g->blob, 0, g->blob_bytes);
    const size_t scratch_bytes = (size_t)GATHER_MAX_CTAS * 2 * sizeof(Best) + 256;
    if (e == cudaSuccess) e = cudaMalloc(&g->scratch, scratch_bytes);
    if (e == cudaSuccess) e = cudaMemset(g->scratch, 0, scratch_bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, g->blob);
    if (e != cudaSuccess) {
        mk_set_error("mk_gather_create: %s", cudaGetErrorString(e));
        if (g->blob) cudaFree(g->blob);
        if (g->scratch) cudaFree(g->scratch);
        delete g;
        return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    memcpy(handle, &h, 64);
    g->peer[rank] = g->blob;
    *out = g;
    return MK_OK;
}

extern "C" int32_t mk_gather_connect(mk_ctx *ctx, mk_gather *g, const uint8_t *handles /* [world][64], by rank */) {
    MK_CHECK_ARG(ctx != nullptr && g != nullptr && handles != nullptr, "NULL argument");
    MK_CHECK_ARG(!g->connected, "already connected");
    MK_CUDA(cudaSetDevice(ctx->device));
    for (int r = 0; r < g->world; ++r) {
        if (r == g->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        bool zero = true;
        for (int b = 0; b < 64; ++b) zero = zero && handles[(size_t)r * 64 + b] == 0;
        cudaError_t e = cudaSuccess;
        if (zero) { // the rank never joined: its rows go to local scratch, its flag never arrives, the wait runs out
            if (!g->absent) e = cudaMalloc(&g->absent, g->blob_bytes);
            if (e == cudaSuccess) e = cudaMemset(g->absent, 0, g->blob_bytes);
            g->peer[r] = g->absent;
            g->is_absent[r] = true;
        } else {
            e = cudaIpcOpenMemHandle(&g->peer[r], h, cudaIpcMemLazyEnablePeerAccess);
        }
        if (e != cudaSuccess) {
            mk_set_error("mk_gather_connect: rank %d cannot open rank %d's buffer: %s", g->rank, r, cudaGetErrorString(e));
            for (int q = 0; q < r; ++q)
                if (q != g->rank && g->peer[q] && !g->is_absent[q]) { cudaIpcCloseMemHandle(g->peer[q]); g->peer[q] = nullptr; }
            return MK_ERR_CUDA;
        }
    }
    g->connected = true;
    return MK_OK;
}

extern "C" int32_t mk_gather_free(mk_ctx *ctx, mk_gather *g) {
    MK_CHECK_ARG(ctx != nullptr && g != nullptr, "NULL argument");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (int r = 0; r < g->world; ++r)
        if (r != g->rank && g->peer[r] && !g->is_absent[r]) cudaIpcCloseMemHandle(g->peer[r]);
    if (g->absent) cudaFree(g->absent);
    if (g->scratch) cudaFree(g->scratch);
    if (g->blob) cudaFree(g->blob);
    delete g;
    return MK_OK;
}

// push: the rows of this rank go to every rank (complete logits everywhere); otherwise only the (maximum, index) pairs do
static int32_t gather_step(mk_ctx *ctx, const mk_weight *w, mk_gather *g, const float *x, int32_t batch, int64_t row0, bool push,
                           const float **logits /* out: device pointer to [batch][vocab] (push) or to this rank's rows of it */, int32_t *argmax) {
    MK_CHECK_ARG(ctx != nullptr && w != nullptr && g != nullptr && x != nullptr, "NULL argument");
    MK_CHECK_ARG(w->fmt == MK_FMT_Q8, "weight handle has the wrong format for this call");
    MK_CHECK_ARG(g->connected || g->world == 1, "mk_gather_connect has not run");
    MK_CHECK_ARG(batch >= 1 && batch <= g->max_batch, "batch exceeds the gather buffers");
    MK_CHECK_ARG(row0 >= 0 && row0 + w->rows <= g->vocab, "shard rows outside the vocabulary");
    MK_CUDA(cudaSetDevice(ctx->device));
    const int64_t ldq = w->nbp * 32;
    const size_t xq_bytes = mk_align_up((size_t)batch * ldq, 256), xs_bytes = mk_align_up((size_t)batch * w->nbp * 4, 256);
    int32_t rc = mk_ws_reserve(ctx, xq_bytes + xs_bytes);
    if (rc != MK_OK) return rc;
    int8_t *xq = (int8_t *)ctx->ws;
    float *xs = (float *)((char *)ctx->ws + xq_bytes);
    rc = mk_launch_quantize_act(ctx, x, batch, w->cols, w->cols, w->nbp, 0, xq, xs);
    if (rc != MK_OK) return rc;

    g->step++;
    const uint32_t par = g->step & 1u;
    const size_t step_off = g->logits_off + (size_t)par * g->max_batch * g->vocab * 4;
    // this rank's rows go straight into its own gather buffer ...
    float *full = (float *)((char *)g->blob + step_off);
    rc = mk_launch_qgemv(ctx, w, xq, xs, batch, 0, 0, full + row0, g->vocab);
    if (rc != MK_OK) return rc;
    // ... and one kernel pushes them to the other ranks, signals and waits
    GatherPeers pe;
    memset(&pe, 0, sizeof(pe));
    const size_t pairs_off = 256 + (size_t)par * 8 * 2 * sizeof(Best);
    for (int r = 0; r < g->world; ++r) {
        pe.dst[r] = (float *)((char *)g->peer[r] + step_off) + row0;
        pe.flag[r] = (uint32_t *)g->peer[r] + par * 8 + g->rank;
        pe.pairs[r] = (Best *)((char *)g->peer[r] + pairs_off) + (size_t)g->rank * 2;
    }
    {
        mk_prof_scope prof(ctx, MK_PROF_OTHER);
        // several CTAs when the slice can move in 16-byte pieces (the kernel's own test, repeated here)
        const bool vec = w->rows % 4 == 0 && g->vocab % 4 == 0 && row0 % 4 == 0 && (((uintptr_t)(full + row0)) & 15) == 0;
        int64_t ncta = vec ? mk_ceil_div(w->rows / 4, GATHER_PIECES_PER_CTA) : 1;
        if (ncta > GATHER_MAX_CTAS) ncta = GATHER_MAX_CTAS;
        if (ncta < 1) ncta = 1;
        Best *partials = (Best *)g->scratch;
        unsigned *counter = (unsigned *)((char *)g->scratch + (size_t)GATHER_MAX_CTAS * 2 * sizeof(Best));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)ncta); cfg.blockDim = dim3(1024); cfg.dynamicSmemBytes = 0; cfg.stream = ctx->stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = ctx->pdl ? 1 : 0;
        cudaLaunchKernelEx(&cfg, gather_exchange_kernel, pe, (const float *)(full + row0), (int)batch, (int64_t)w->rows, (int64_t)g->vocab, (int64_t)row0,
                           (int)g->rank, (int)g->world, (const uint32_t *)g->blob + par * 8, (const Best *)((char *)g->blob + pairs_off), argmax,
                           ctx->status_dev, partials, counter, push);
        ctx->launches++;
    }
    MK_CUDA(cudaGetLastError());
    if (logits) *logits = push ? full : full + row0;
    return MK_OK;
}

extern "C" int32_t mk_matvec_q8_gather_dev(mk_ctx *ctx, const mk_weight *w, mk_gather *g, const float *x, int32_t batch, int64_t row0,
                                           const float **logits, int32_t *argmax) {
    return gather_step(ctx, w, g, x, batch, row0, true, logits, argmax);
}

extern "C" int32_t mk_matvec_q8_gather_token_dev(mk_ctx *ctx, const mk_weight *w, mk_gather *g, const float *x, int32_t batch, int64_t row0,
                                                 const float **local_rows, int32_t *argmax) {
    MK_CHECK_ARG(argmax != nullptr, "the token-only step returns the token: argmax must not be NULL");
    return gather_step(ctx, w, g, x, batch, row0, false, local_rows, argmax);
}
