// Shared declarations for libmk_b200: context, weight records, error plumbing
// and the small device helpers every kernel file uses (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/mk_cuda.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "libmk_b200 is written for sm_100a only"
#endif

// ---------------------------------------------------------------- errors
void mk_set_error(const char *fmt, ...);

#define MK_CHECK_ARG(cond, msg)                                   \
    do {                                                          \
        if (!(cond)) {                                            \
            mk_set_error("%s: %s", __func__, msg);                \
            return MK_ERR_ARG;                                    \
        }                                                         \
    } while (0)

#define MK_CUDA(call)                                                                  \
    do {                                                                               \
        cudaError_t e_ = (call);                                                       \
        if (e_ != cudaSuccess) {                                                       \
            mk_set_error("%s: %s failed: %s", __func__, #call, cudaGetErrorString(e_)); \
            return (e_ == cudaErrorMemoryAllocation) ? MK_ERR_OOM : MK_ERR_CUDA;       \
        }                                                                              \
    } while (0)

// A function attribute (cudaFuncSetAttribute) belongs to one device: one flag per call site AND device
// ordinal, so that a second context on another GPU of the same process opts in as well.
#define MK_MAX_DEVICES 64
struct mk_once_per_device {
    bool done[MK_MAX_DEVICES];
    bool pending(int dev) const { return dev < 0 || dev >= MK_MAX_DEVICES || !done[dev]; }
    void mark(int dev) { if (dev >= 0 && dev < MK_MAX_DEVICES) done[dev] = true; }
};

// ---------------------------------------------------------------- records
enum { MK_FMT_MXFP4 = 0, MK_FMT_Q8 = 1, MK_FMT_F32 = 2, MK_FMT_VQ1 = 3 };

// A registered weight matrix in the fragment-major ("tiled") device layout.
//
// Rows are cut into tiles of 16, columns into q8/mxfp4 blocks of 32.  The block
// count is padded to a multiple of 4 (nbp) and the row count to a multiple of 16
// (padding holds zero codes / zero scales, which contribute exactly 0).
//
// One 512-byte CHUNK is what a warp loads with one 16-byte load per lane; lane
// L = 4*g + t (g = L>>2, t = L&3) holds the A fragment of mma.m16n8k32 for
// rows {g, g+8} of the tile and the real columns [8t, 8t+8) of a block:
//   q8   : chunk (rt, b)      = [row g: cols 8t..8t+3][row g+8: same][row g: cols 8t+4..8t+7][row g+8: same]
//   mxfp4: chunk (rt, bp)     = [row g, block 2bp: 8 codes of cols 8t..8t+7][row g+8, block 2bp]
//                               [row g, block 2bp+1][row g+8, block 2bp+1]   (natural nibble order in each word)
// Scales are tiled as [rt][block][16 rows] so a warp's scales are contiguous.
struct mk_weight {
    int fmt;            // MK_FMT_*
    int scale_type;     // MK_SCALE_* (q8 only)
    int64_t rows, cols;
    int64_t nrt;        // row tiles = ceil(rows/16)
    int64_t nb;         // blocks per row = cols/32
    int64_t nbp;        // padded to a multiple of 4
    void *values;       // tiled values
    void *scales;       // tiled scales (u8 for mxfp4, f32/f16 for q8)
    size_t values_bytes, scales_bytes;
};

struct mk_ctx {
    int device;
    int sm_count;
    int cc_major, cc_minor;
    size_t mem_bytes;
    cudaStream_t own_stream;
    cudaStream_t stream;
    int64_t launches;
    uint64_t alloc_epoch;   // counts the re-allocations of buffers that recorded launches (CUDA graphs) may point into: an
                            // object that grows its per-call buffers bumps it, a holder of a recording compares and re-records
    int32_t *status_dev;    // device status word
    int8_t *zeros_dev;      // 256 zero bytes (B operand of unused MMA columns)
    unsigned *argmax_count; // 64 counters, 0 between calls: CTAs of the greedy-pick kernel that have finished, per row
    // activation workspace (grown on demand, never per call once warm)
    void *ws;
    size_t ws_bytes;
    // host-call staging
    void *io_dev;
    size_t io_bytes;
    void *io_pinned;
    size_t io_pinned_bytes;
    int force_ks;           // 0 = choose per shape
    int pdl;                // 1 = the one-token matvec starts behind its activation quantizer by programmatic stream serialization
    int mla_max_split;      // > 0: upper bound on the KV splits of an attention call (study / test knob)
    int moe_no_fuse;        // 1 = separate router / top-k / plan / quantize launches also for small batches (study knob)
    int mla_no_tc;
    int mla_strict;         // 1 = per-head attention by the one-warp-per-head kernel that keeps the CPU's summation order (parity mode)
    int mla_no_t5;          // 1 = absorbed MLA on the mma.sync kernel instead of the tcgen05 one (study knob)
    int kda_smem;           // 1 = KDA step with S staged in shared memory also for dim 64 / 128, where the register form is the default (study knob)
    // side streams for launches that do not depend on each other (forked from and joined to `stream` with events,
    // which also works while `stream` is being recorded into a CUDA graph); created on first use
    cudaStream_t side[2];
    cudaEvent_t side_ev[4];
    int side_ready;
    // optional per-category event timing (mk_prof_*)
    int prof_on;
    struct mk_prof_pair *prof_pairs; // pool of event pairs
    int prof_cap, prof_used;
    int64_t prof_count[MK_PROF_NCAT];
    double prof_ms[MK_PROF_NCAT];
};
struct mk_prof_pair { cudaEvent_t a, b; int cat; };
// Brackets one kernel launch with an event pair when profiling is on.
struct mk_prof_scope {
    mk_ctx *ctx;
    mk_prof_pair *p;
    mk_prof_scope(mk_ctx *c, int cat);
    ~mk_prof_scope();
};
int32_t mk_prof_drain(mk_ctx *ctx); // folds finished pairs into the accumulators (synchronizes)

int32_t mk_fork(mk_ctx *ctx, int i);   // side stream i continues from everything enqueued on ctx->stream so far
int32_t mk_join(mk_ctx *ctx, int i);   // ctx->stream waits for everything enqueued on side stream i
// launches made while one of these lives go to side stream i
struct mk_on_side {
    mk_ctx *ctx; cudaStream_t saved;
    mk_on_side(mk_ctx *c, int i) : ctx(c), saved(c->stream) { c->stream = c->side[i]; }
    ~mk_on_side() { ctx->stream = saved; }
};
int32_t mk_ws_reserve(mk_ctx *ctx, size_t bytes);      // activation workspace
int32_t mk_io_reserve(mk_ctx *ctx, size_t bytes);      // device staging for host-pointer calls
int32_t mk_pinned_reserve(mk_ctx *ctx, size_t bytes);  // pinned host staging

static inline int64_t mk_ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t mk_align_up(size_t a, size_t b) { return (a + b - 1) / b * b; }

// ---------------------------------------------------------------- kernel launchers (defined in the .cu files)
// activation quantization: x f32 [ntok, cols] -> xq i8 [limbs][ntok][ldq], xs f32 [ntok][nbp]
int32_t mk_launch_quantize_act(mk_ctx *ctx, const float *x, int ntok, int64_t cols, int64_t ldx, int64_t nbp,
                               int x2, int8_t *xq, float *xs);
// the fused dequant + GEMV
int32_t mk_launch_qgemv(mk_ctx *ctx, const mk_weight *w, const int8_t *xq, const float *xs, int ntok,
                        int x2, int strict, float *y, int64_t ldy);
// spine.cu: y[tok * ldy + row] (+)= dot(w[row], x[tok]) in the engine's dot() order; rmsnorm; SiTU
int32_t mk_launch_f32_gemv(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols, const float *x, int n, float *y, int64_t ldy,
                           int accumulate);
int32_t mk_launch_rmsnorm(mk_ctx *ctx, const float *x, const float *w, int n, int len, float eps, float *out);
int32_t mk_launch_situ(mk_ctx *ctx, const float *a, const float *u, int64_t count, float *out);
int32_t mk_launch_argmax(mk_ctx *ctx, const float *y, int64_t n, int64_t ldy, int batch, int32_t *out, void *scratch);
size_t mk_argmax_scratch_bytes(int batch);
// moe.cu: the K3 latent MoE layer for ONE token with the shared expert on a side stream: out_routed = routed_up(...),
// out_shared = the f32 shared expert's output, NOT added (the caller adds routed + shared, in that order).
// MK_ERR_UNSUPPORTED when the layer is not of that kind (the caller then uses mk_moe_forward_dev).
int32_t mk_moe_forward_k3_split(mk_ctx *ctx, mk_moe *m, const float *x, float *out_routed, float *out_shared);
void mk_mla_note_replay(mk_mla *m, int seq);   // mla.cu: host-side position count after a graph replay of a decode step
struct mk_moe_ep;
struct mk_gather;
uint32_t mk_moe_ep_steps(const mk_moe_ep *ep);            // moe.cu: exchange steps issued so far (host mirror of the device count)
void mk_moe_ep_note_replay(mk_moe_ep *ep, uint32_t n);    //         n more steps ran from a recorded token
uint32_t mk_gather_steps(const mk_gather *g);             // gather.cu: the same for the sharded lm_head
void mk_gather_note_replay(mk_gather *g, uint32_t n);
// weight (re)tiling
int32_t mk_launch_retile_mxfp4(mk_ctx *ctx, const uint8_t *packed, const uint8_t *scales, mk_weight *w);
int32_t mk_launch_untile_mxfp4(mk_ctx *ctx, const mk_weight *w, uint8_t *packed, uint8_t *scales);
int32_t mk_launch_dequant_mxfp4(mk_ctx *ctx, const mk_weight *w, float *out);
int32_t mk_launch_quantize_weight_q8(mk_ctx *ctx, const float *wf32, int64_t row0, int64_t nrows, mk_weight *w);
int32_t mk_launch_retile_q8(mk_ctx *ctx, const int8_t *q, const void *scales, mk_weight *w);
int32_t mk_launch_untile_q8(mk_ctx *ctx, const mk_weight *w, int8_t *q, void *scales);

// SiTU (src/model.rs:617-621): 4 tanh(g/4) sigmoid(g) * 25 tanh(u/25), multiplied left to
// right as the engine writes it; tanh and exp in double precision, rounded once.
__device__ __forceinline__ float mk_situ(float g, float u) {
    const float tg = (float)tanh((double)__fdiv_rn(g, 4.0f));
    const float sg = __fdiv_rn(1.0f, __fadd_rn(1.0f, (float)exp((double)(-g))));
    const float tu = (float)tanh((double)__fdiv_rn(u, 25.0f));
    return __fmul_rn(__fmul_rn(__fmul_rn(4.0f, tg), sg), __fmul_rn(25.0f, tu));
}

// Element offset of the scale of (row tile rt, block b, row r16 of the tile).  Scales are
// tiled [row tile][group of 4 blocks][16 rows][4 blocks]: the four scales one row needs for
// a group of blocks are adjacent (one 32-bit / 64-bit / 128-bit load by scale type).
__host__ __device__ __forceinline__ int64_t mk_scale_off(int64_t rt, int64_t nbp, int64_t b, int r16) {
    return (rt * nbp + (b & ~(int64_t)3)) * 16 + r16 * 4 + (b & 3);
}
#ifdef __CUDACC__
// ---------------------------------------------------------------- device helpers
// 2^(sb-127) from a ue8m0 byte as an exact bit pattern; sb == 0 is the subnormal 2^-127.
__device__ __forceinline__ float mk_e8m0(uint32_t sb) {
    return __uint_as_float(sb == 0 ? 0x00400000u : (sb << 23));
}
// 2^(sb-128): the scale of the integer LUT (E2M1 x 2) convention.
__device__ __forceinline__ float mk_e8m0_half(uint32_t sb) {
    // 2^(sb-127) * 0.5: exact for every byte (sb == 1 gives the subnormal 2^-127)
    return mk_e8m0(sb) * 0.5f;
}
// prmt.b32 in its generic form: selector nibble n picks byte (n & 7) of {b,a};
// a selector nibble with bit 3 set yields 0x00/0xFF from that byte's sign bit.
__device__ __forceinline__ uint32_t mk_prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// D += A(16x32, s8, row) * B(32x8, s8, col), int32 accumulate.
__device__ __forceinline__ void mk_mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16-byte streaming load that does not allocate in L1 (weights are read once).
__device__ __forceinline__ uint4 mk_ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// E2M1 x 2 magnitudes as two prmt pool registers: bytes {0,1,2,3} and {4,6,8,12}.
#define MK_LUT2_LO 0x03020100u
#define MK_LUT2_HI 0x0C080604u
#endif

// A launch that may start behind the previous launch of the stream by programmatic stream serialization (`dep`): the
// kernel itself waits (griddepcontrol.wait) before it touches what that launch produces.  Otherwise an ordinary launch.
template <typename... KArgs, typename... Args>
inline cudaError_t mk_launch_dep(bool dep, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = dep ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
__device__ __forceinline__ void mk_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void mk_dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
