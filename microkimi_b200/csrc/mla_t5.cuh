// Absorbed-layout MLA decode attention on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), sm_100a.
//
// Same arithmetic as mla_tc.cuh (the q8_0 latent tile dequantized once to f16 and used
// twice, f16 x f16 -> f32, online softmax, split-KV + merge), restructured for tcgen05:
//
//   * positions are the M dimension.  For a tile of 128 positions
//         S^T [128 pos x 64 heads] = K_tile [128 x 576] . Q^T          (36 MMAs, K = 16 each)
//         O^T [512 x 64 heads]    += V_tile^T [512 x 128] . P^T         (4 x 8 MMAs)
//     so S^T takes 64 columns of tensor memory and O^T 4 x 64, with all 128 lanes in use
//     (heads as M would leave half the lanes idle and need 512 columns for O alone).
//   * the dequantized tile is written ONCE in the canonical 128-byte-swizzled layout
//     (9 atoms of [128 positions][64 columns]).  Read as a K-major A operand it is K;
//     read as an MN-major A operand (same bytes, other strides) it is V^T = its first
//     8 atoms.  Q is the K-major B operand of the first product; P^T, written into the
//     9th atom (the rope columns, dead once S is done), the K-major B operand of the second.
//   * softmax runs over LANES (positions).  Each thread owns one position and 16 heads and keeps,
//     in registers, the maximum in use m_use of those heads (log2 domain; all threads of a column
//     group hold identical copies).  Fast path: P = 2^(s - m_use) straight away, and a CTA-wide
//     vote (barrier with OR) whether any score lies more than a margin (2^11) above m_use.  Only
//     then - always on the first tile, rarely later - the slow path computes the true column maxima
//     (redux.sync on order-preserving integer keys + shared-memory atomicMax), moves m_use,
//     rescales O^T (tcgen05.ld / st) and l, and writes P^T again.  l takes the column sums of the
//     f16 P^T from shared memory, the very terms the second product uses.
//   * the next tile's bytes are requested right after the first product is issued and consumed
//     after the second one: HBM latency hides behind the softmax and the second product.
//   * one thread issues the MMAs; completion comes back through tcgen05.commit on an
//     mbarrier.  Every wait is bounded: a wait that runs out sets MK_ERR_TIMEOUT in the
//     status word and the kernel carries on to its end (tensor memory is always freed).
//
// Measured and set aside: a 17th warp that only issues the MMAs, the second product committed per 128-row group, the next
// tile converted pair of atoms by pair as the groups finish, the first product's K steps issued per pair (named barriers,
// workers never wait for the issuer).  Correct, but 17 warps are allocated registers as 20, which caps a thread at 96: at
// that cap this kernel, unchanged, goes from 0.191 to 0.260 ms (ctx 65536, batch 8) and the overlapped form reaches
// 0.256 ms.  With the issuing thread inside one of the 16 warps that warp's share of the conversion waits for its issue
// loop (an issue blocks for about as long as the MMA runs) and the whole CTA waits for that warp.  Quantizing the query
// rows in this kernel's prologue instead of a launch of its own was also no faster (28.8 -> 30.8 us at ctx 4096).
//
// Reference recipe: mla_attn_flash_q8_mqa (src/model.rs:1804-1908) applied to one shared
// q8_0 row per position; operands carry one f16 rounding each.
#pragma once
#include <cuda_fp16.h>

#include "mk_common.cuh"
#include "mla_tc.cuh" // dequant8

namespace mla_t5 {

constexpr int H = 64, LAT = 576, VD = 512, NBLK = 18, TJ = 128, THREADS = 512;
constexpr int NATOM = LAT / 64;            // 9 column atoms of 64 f16 (128 bytes)
constexpr int K_ATOM = TJ * 128;           // 16384 bytes: [128 positions][128 B]
constexpr int Q_ATOM = H * 128;            // 8192 bytes:  [64 heads][128 B]
constexpr int SM_K = 0, SM_Q = SM_K + NATOM * K_ATOM, SM_P = SM_K + 8 * K_ATOM;
constexpr int SM_MUSED = SM_Q + NATOM * Q_ATOM, SM_L = SM_MUSED + H * 4, SM_ALPHA = SM_L + H * 4;
constexpr int SM_TMAX = SM_ALPHA + H * 4;              // uint32 tmax[64] (+64 spare): tile maxima as ordered keys, 0 between uses
constexpr int SM_BAR = SM_TMAX + 2 * H * 4;            // 2 mbarriers, tmem slot
constexpr int SM_USED = SM_BAR + 32;
constexpr int SM_TOTAL = SM_USED + 1024;               // slack to align the base to 1024 bytes
constexpr int UNITS = TJ * (LAT / 16) / THREADS;       // 16-byte units (half a scale block) of a tile per thread = 9
constexpr int TMEM_COLS = 512, COL_S = 0, COL_O = 64;
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr float RESCALE_MARGIN2 = 11.0f;                // in log2 units: P <= 2^11, far inside f16

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor: 128-byte swizzle, version 1 (sm_100)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor: f16 x f16 -> f32, M = 128, N = 64; a_mn: A is MN-major
__device__ __forceinline__ uint32_t instr_desc(bool a_mn) {
    return (1u << 4) | (a_mn ? (1u << 15) : 0u) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// bounded wait for a phase of an mbarrier; false = gave up
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    uint32_t done = 0;
    for (uint32_t it = 0; it < WAIT_LIMIT && !done; ++it)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t addr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                   "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t addr, const uint32_t (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n" ::"r"(addr),
                 "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
                 "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                 : "memory");
}
// 8 int8 values (two words) times one f32 scale -> 8 f16.  The scale is split into two f16 terms,
// s = s_hi + s_lo, and the product formed as fma(v, s_hi, v * s_lo): v is an exact small integer, so the
// result is the correctly rounded v * s up to a second rounding of relative size 2^-22.  f16 arithmetic
// only: no conversions in the inner loop.
__device__ __forceinline__ uint4 dequant8_h(uint2 w, float s) {
    const uint32_t x0 = w.x ^ 0x80808080u, x1 = w.y ^ 0x80808080u; // bytes + 128
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);       // 0x64uu as f16 is 1024 + uu
    const __half sh = __float2half_rn(s);
    const __half2 s_hi = __half2half2(sh), s_lo = __half2half2(__float2half_rn(s - __half2float(sh)));
    uint32_t m[4] = {__byte_perm(x0, 0x64646464u, 0x4140), __byte_perm(x0, 0x64646464u, 0x4342),
                     __byte_perm(x1, 0x64646464u, 0x4140), __byte_perm(x1, 0x64646464u, 0x4342)};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 v = __hsub2(*(__half2 *)&m[i], off);
        const __half2 r = __hfma2(v, s_hi, __hmul2(v, s_lo));
        o[i] = *(const uint32_t *)&r;
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
// 2^x, one MUFU instruction; 2^(-inf) = 0
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t f_order(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float f_unorder(uint32_t u) { return __uint_as_float((u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u); }

__global__ void __launch_bounds__(THREADS, 1)
mla_absorbed_t5_kernel(const int8_t *__restrict__ vq, const float *__restrict__ vs, int cap, const int8_t *__restrict__ qq,
                       const float *__restrict__ qs, int64_t ldq, int64_t q_nbp, const int *__restrict__ npos_arr,
                       int npos_fixed, int seq0, float scale, int nsplit, float *__restrict__ part_m,
                       float *__restrict__ part_l, float *__restrict__ part_o, float *__restrict__ out, int32_t *__restrict__ status) {
    extern __shared__ unsigned char sm_raw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)sm_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, cg = warp >> 2; // tensor-memory lane quadrant of this warp; its column group
    const int bi = blockIdx.y, seq = seq0 + bi, split = blockIdx.x;
    float *m_used = (float *)(sm + SM_MUSED), *l_run = (float *)(sm + SM_L), *alpha = (float *)(sm + SM_ALPHA);
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    uint32_t *tmem_slot = (uint32_t *)(sm + SM_BAR + 16);
    uint32_t *tmax = (uint32_t *)(sm + SM_TMAX);
    const uint32_t bar_s = s32(&bars[0]), bar_o = s32(&bars[1]);
    const uint32_t k_base = s32(sm + SM_K), q_base = s32(sm + SM_Q), p_base = s32(sm + SM_P);

    const int n = npos_arr ? npos_arr[seq] : npos_fixed;
    const int ntiles = (n + TJ - 1) / TJ;
    const int tps = (ntiles + nsplit - 1) / nsplit;
    const int t0 = split * tps, t1 = min(t0 + tps, ntiles);

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_s));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_o));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid < H) { m_used[tid] = -INFINITY; l_run[tid] = 0.0f; alpha[tid] = 1.0f; tmax[tid] = 0u; tmax[H + tid] = 0u; }
    // ---- Q: q8 rows (quantized by the activation quantizer) -> f16, K-major swizzled atoms [64 heads][64 columns]
    for (int u = tid; u < H * (LAT / 8); u += THREADS) {
        const int h = u / (LAT / 8), c8 = u % (LAT / 8);
        const int64_t row = (int64_t)bi * H + h;
        const uint2 w = *(const uint2 *)(qq + row * ldq + c8 * 8);
        const float s = qs[row * q_nbp + (c8 >> 2)];
        *(uint4 *)(sm + SM_Q + (c8 >> 3) * Q_ATOM + h * 128 + (((c8 & 7) ^ (h & 7)) << 4)) = mla_tc::dequant8(w, s);
    }

    const int8_t *vbase = vq + (int64_t)seq * cap * LAT;
    const float *sbase = vs + (int64_t)seq * cap * NBLK;
    uint4 raw[UNITS];
    float rsc[UNITS];
    auto load_raw = [&](int tile) {
#pragma unroll
        for (int i = 0; i < UNITS; ++i) {
            const int u = tid + i * THREADS;
            const int p = u / (LAT / 16), c16 = u % (LAT / 16);
            const int j = tile * TJ + p;
            if (j < n) {
                raw[i] = __ldg((const uint4 *)(vbase + (int64_t)j * LAT + c16 * 16));
                rsc[i] = __ldg(sbase + (int64_t)j * NBLK + (c16 >> 1));
            } else {
                raw[i] = make_uint4(0u, 0u, 0u, 0u);
                rsc[i] = 0.0f;
            }
        }
    };
    if (t0 < t1) load_raw(t0);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = *tmem_slot;
    const uint32_t idesc_s = instr_desc(false), idesc_o = instr_desc(true);
    // base descriptors: K tile as K-major A (S^T) and as MN-major A (V^T: 64-row blocks 16 KB apart), Q and P^T as K-major B
    const uint64_t desc_k = smem_desc(k_base, 16, 1024), desc_v = smem_desc(k_base, K_ATOM, 1024), desc_q = smem_desc(q_base, 16, 1024),
                   desc_p = smem_desc(p_base, 16, 1024);
    bool timed_out = false;

    // softmax state of this thread: its position lane, heads 16 cg .. +15.  Threads of one column group
    // hold identical copies of m_use (the maximum baked into O^T, P and l; log2 domain) and update them
    // with the same arithmetic.  l (shared memory) takes the column sums of the f16 P^T each tile.
    float m_use[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) m_use[i] = -INFINITY;
    const float scale2 = scale * 1.4426950408889634f; // scores in the log2 domain: p = 2^(s2 - m_use)

    for (int tile = t0; tile < t1; ++tile) {
        const uint32_t par = (uint32_t)(tile - t0) & 1u;
        // ---- the tile, dequantized, into the swizzled atoms (the previous tile's second product has finished)
#pragma unroll
        for (int i = 0; i < UNITS; ++i) {
            const int u = tid + i * THREADS;
            const int p = u / (LAT / 16), c16 = u % (LAT / 16);
            // rows past the end were loaded as zeros: 0 * 0 = 0, never a NaN from stale memory
            unsigned char *row = sm + SM_K + (c16 >> 2) * K_ATOM + p * 128;
            const int cc = (c16 & 3) * 2;
            *(uint4 *)(row + ((cc ^ (p & 7)) << 4)) = dequant8_h(make_uint2(raw[i].x, raw[i].y), rsc[i]);
            *(uint4 *)(row + (((cc + 1) ^ (p & 7)) << 4)) = dequant8_h(make_uint2(raw[i].z, raw[i].w), rsc[i]);
        }
        fence_async_smem();
        tc_fence_before();
        __syncthreads();
        // ---- S^T = K Q^T
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < LAT / 16; ++ks) {
                // descriptors advance by adding the byte offset / 16 to their address field (low word)
                const uint32_t a = ks >> 2, kk = ks & 3;
                mma_f16_ss(tb + COL_S, desc_k + ((a * K_ATOM + kk * 32) >> 4), desc_q + ((a * Q_ATOM + kk * 32) >> 4), idesc_s, ks > 0 ? 1u : 0u);
            }
            mma_commit(bar_s);
        }
        // the next tile's bytes start travelling now; they are consumed after the second product
        if (tile + 1 < t1) load_raw(tile + 1);
        if (!bar_wait(bar_s, par)) timed_out = true;
        tc_fence_after();
        // ---- scores of this thread: position 32 quad + lane of the tile, heads 16 cg .. +15 (log2 domain)
        float s[16];
        {
            uint32_t v[16];
            tmem_ld16(tb + ((uint32_t)(quad * 32) << 16) + COL_S + cg * 16, v);
            const bool live = tile * TJ + quad * 32 + lane < n;
#pragma unroll
            for (int i = 0; i < 16; ++i) s[i] = live ? __uint_as_float(v[i]) * scale2 : -INFINITY;
        }
        // ---- P^T[head][position] = 2^(s - m_use), f16, K-major swizzled atoms [64 heads][64 positions].
        // m_use is the maximum in use from earlier tiles; a score more than the margin above it sends the
        // whole CTA through the slow path below (always on the first tile, rarely afterwards).
        const int j = quad * 32 + lane; // position in the tile
        unsigned char *prow = sm + SM_P + (j >> 6) * Q_ATOM + ((j & 7) << 1);
        const int jc = (j & 63) >> 3;
        float over = -INFINITY;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int h = cg * 16 + i;
            const float e = s[i] - m_use[i];
            over = fmaxf(over, e);
            *(__half *)(prow + h * 128 + ((jc ^ (h & 7)) << 4)) = __float2half_rn(ex2_approx(e));
        }
        fence_async_smem();
        tc_fence_before();
        const int any_over = __syncthreads_or(over > RESCALE_MARGIN2 ? 1 : 0);
        if (any_over || tile == t0) {
            // ---- slow path: true tile maxima (redux over the warp's 32 positions, atomicMax over the 4
            // quadrants), m_use moved where needed, O^T and l rescaled, P^T written again
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint32_t mx = __reduce_max_sync(0xFFFFFFFFu, f_order(s[i]));
                if (lane == i) atomicMax(&tmax[cg * 16 + i], mx);
            }
            __syncthreads();
            const bool writer = quad == 0 && lane == 0; // one thread per column group publishes the factors
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float tm = f_unorder(tmax[cg * 16 + i]);
                float al = 1.0f;
                if (tile == t0) {
                    m_use[i] = tm;
                } else if (tm > m_use[i] + RESCALE_MARGIN2) {
                    al = ex2_approx(m_use[i] - tm);
                    m_use[i] = tm;
                }
                if (writer) { alpha[cg * 16 + i] = al; l_run[cg * 16 + i] *= al; }
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int h = cg * 16 + i;
                *(__half *)(prow + h * 128 + ((jc ^ (h & 7)) << 4)) = __float2half_rn(ex2_approx(s[i] - m_use[i]));
            }
            fence_async_smem();
            __syncthreads();
            if (tid < H) tmax[tid] = 0u;
            if (tile > t0) {
                // O^T columns (heads) times alpha (1 for the heads that did not move); warp = (lane quadrant, 128-row tile cg)
                tc_fence_after();
#pragma unroll 1
                for (int c0 = 0; c0 < H; c0 += 16) {
                    uint32_t v[16];
                    const uint32_t addr = tb + ((uint32_t)(quad * 32) << 16) + COL_O + cg * 64 + c0;
                    tmem_ld16(addr, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha[c0 + i]);
                    tmem_st16(addr, v);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            }
            tc_fence_before();
            __syncthreads();
        }
        // ---- O^T += V^T P^T
        if (tid == 0) {
            tc_fence_after();
            const uint32_t acc0 = tile > t0 ? 1u : 0u;
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int ks = 0; ks < TJ / 16; ++ks)
                    mma_f16_ss(tb + COL_O + mt * 64, desc_v + (((2 * mt) * K_ATOM + ks * 16 * 128) >> 4),
                               desc_p + (((ks >> 2) * Q_ATOM + (ks & 3) * 32) >> 4), idesc_o, ks > 0 ? 1u : acc0);
            mma_commit(bar_o);
        }
        // ---- l += column sums of the f16 P^T (the values the product uses): 8 threads per head, 16 positions each
        {
            const int h = tid >> 3, part = tid & 7;
            const unsigned char *pr = sm + SM_P + (part >> 2) * Q_ATOM + h * 128;
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint4 w = *(const uint4 *)(pr + ((((part & 3) * 2 + c) ^ (h & 7)) << 4));
                const __half2 *hp = (const __half2 *)&w;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __half22float2(hp[q]);
                    sum += f.x + f.y;
                }
            }
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
            sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
            if (part == 0) l_run[h] += sum;
        }
        if (!bar_wait(bar_o, par)) timed_out = true;
        tc_fence_after();
    }
    if (timed_out && lane == 0) atomicCAS(status, 0, MK_ERR_TIMEOUT);
    if (quad == 0 && lane == 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) m_used[cg * 16 + i] = m_use[i];
    }
    __syncthreads();

    // ---- results: O^T rows = output columns.  warp = (lane quadrant, 128-row tile cg); lane = column
    {
        const int col = cg * 128 + quad * 32 + lane;
        const bool has = t0 < t1;
#pragma unroll 1
        for (int c0 = 0; c0 < H; c0 += 16) {
            uint32_t v[16];
            if (has) {
                tmem_ld16(tb + ((uint32_t)(quad * 32) << 16) + COL_O + cg * 64 + c0, v);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int h = c0 + i;
                const float o = __uint_as_float(v[i]);
                if (nsplit == 1) out[((int64_t)bi * H + h) * VD + col] = o / l_run[h];
                else part_o[(((int64_t)bi * H + h) * nsplit + split) * VD + col] = o;
            }
        }
        if (nsplit > 1 && tid < H) {
            // the merge kernel works with natural-log maxima
            const int64_t p = ((int64_t)bi * H + tid) * nsplit + split;
            part_m[p] = m_used[tid] * 0.6931471805599453f;
            part_l[p] = l_run[tid];
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(TMEM_COLS) : "memory");
}

} // namespace mla_t5
