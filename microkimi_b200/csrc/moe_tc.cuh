// Batched MoE experts on the 5th-generation tensor cores: tcgen05.mma kind::mxf8f6f4 with block scales (sm_100a).
//
// For calls with many token rows (the batch-256 layer: ~5 tokens per routed expert, 256 on the shared one) the expert
// matvecs are a real contraction.  Swap-AB: 128 weight rows are the M dimension, an expert's tokens the N dimension.
//   A : the E2M1 codes exactly as the registered weight holds them - no decode.  In shared memory a 16-byte chunk carries
//       16 codes in its low 8 bytes (the tensor core's FP4 operand form: 8 data + 8 padding bytes), rows of 128 bytes
//       (128 codes) in the 128-byte-swizzled K-major layout.  The chunks of the registered (mma.sync fragment order)
//       layout are scattered there by 4-byte cp.async copies, so the weights keep ONE resident copy.
//   SFA : the ue8m0 scale bytes of the weight, unchanged, 4 blocks per step, copied into tensor memory (tcgen05.cp
//       32x128b.warpx4) in the scale-factor layout: lane r, 32-bit column q, byte k = scale of (row r + 32 q, block k).
//   B : the activations as THREE E4M3 limbs with power-of-two block scales (x = 2^e (h1 + 2^-4 h2 + 2^-8 h3) per block
//       of 32, each limb the E4M3 rounding of what the previous ones left): 12 significant bits per element, products
//       exact, f32 accumulation inside the tensor core.  One MMA per limb and block accumulates into the same columns.
//       This is NOT the engine's q8_0 activation (src/q8.rs:49-69), whose f32 block scale cannot ride on a block-scaled
//       MMA; it tracks the engine's exact-f32 path (src/mxfp4.rs:488-539) to ~1e-5 of max |y| (tests hold 1e-3).
//   D : f32 accumulators in tensor memory; the epilogue reads them with tcgen05.ld.
// Reference semantics: ds_moe / expert_forward (src/deepseek.rs:1038-1108, 74-95), batched as matvec_packed_nt batches
// (src/model.rs:2412-2447): a (token, expert) result does not depend on which other tokens share the tile.
//
// Pipeline per CTA: 8 producer warps fill a ring of 3 stages (128 columns of K each) with cp.async, one thread issues the
// scale-factor copies and the MMAs, tcgen05.commit hands a stage back.  Every wait is bounded; a wait that runs out sets
// MK_ERR_TIMEOUT in the status word and the CTA runs to its end (tensor memory is always freed).  No cluster launch, no
// multicast.
#pragma once
#include <cuda_fp8.h>

#include "mk_common.cuh"

namespace mtc {

constexpr int NT = 32;                 // token rows (pairs) per work item
constexpr int STAGES = 3, KSTEP = 128, NPROD = 256, THREADS = NPROD + 32;   // 8 producer (and epilogue) warps + the MMA warp
constexpr int A_BYTES = 128 * 128;     // one 128-row tile of a stage: [128 rows][128 B]
constexpr int B_BYTES = NT * 128;      // one limb of a stage: [32 rows][128 B]
constexpr int OFF_A0 = 0, OFF_A1 = A_BYTES, OFF_B = 2 * A_BYTES, OFF_SF = OFF_B + 3 * B_BYTES;   // SF: 5 atoms of 512 B
constexpr int STAGE_BYTES = ((OFF_SF + 5 * 512 + 1023) / 1024) * 1024;
constexpr int SM_BAR = STAGES * STAGE_BYTES;           // full[3], empty[3], done, tmem slot
constexpr int SM_TOTAL = SM_BAR + 128 + 1024;          // + slack to align the base to 1024 bytes
constexpr int TMEM_COLS = 128, COL_D0 = 0, COL_D1 = NT, COL_SF = 2 * NT;   // SF: 2 buffers x 5 atoms x 4 columns
constexpr uint32_t WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t layout) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) |
           (1ull << 46) | (layout << 61);
}
// block-scaled instruction descriptor: A = E2M1, B = E4M3, ue8m0 scales, M = 128, N = n, scale bytes `sf` of both operands
__device__ __forceinline__ uint32_t idesc_mx(int n, int sf) {
    return (5u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | ((uint32_t)sf << 29) | ((uint32_t)sf << 4);
}
__device__ __forceinline__ void mma_mx(uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc, uint32_t sfa, uint32_t sfb) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(d), "l"(da), "l"(db), "r"(idesc),
                 "r"(acc), "r"(sfa), "r"(sfb)
                 : "memory");
}
__device__ __forceinline__ void sf_copy(uint32_t taddr, uint32_t saddr) {
    const uint64_t desc = smem_desc(saddr, 16, 128, 0);   // 32 rows of 16 bytes, contiguous
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    uint32_t done = 0;
    for (uint32_t it = 0; it < WAIT_LIMIT && !done; ++it)
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp4(uint32_t dst, const void *src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp16(uint32_t dst, const void *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float (&v)[16]) {
    uint32_t u[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]),
                   "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
                 : "r"(addr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(u[i]);
}

// ---------------------------------------------------------------- activations -> three E4M3 limbs per block of 32
// One warp per (row, block): e = exponent of the block maximum - 7 (so |x| 2^-e < 256), limb k = E4M3(rest * 2^(4k)) with the
// rest taken exactly in f32; scale bytes e + 127, e + 123, e + 119 (ue8m0).  A zero block gets zero limbs.
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
    return __half2float(*(const __half *)&h);
}
__device__ __forceinline__ void limbs_of(float v, float mx, uint8_t (&limb)[3], uint8_t (&sf)[3]) {
    if (!(mx > 0.0f) || !(mx < INFINITY)) {
        limb[0] = limb[1] = limb[2] = 0; sf[0] = sf[1] = sf[2] = 127;
        return;
    }
    int e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 - 7;      // mx = m 2^E, 1 <= m < 2 (subnormal maxima read as 2^-127): e = E - 7
    e = e < -119 ? -119 : (e > 127 ? 127 : e);                          // all three scale bytes stay inside ue8m0
    const float inv = __uint_as_float((uint32_t)(127 - e) << 23);       // 2^-e, exact (e in [-119, 127] keeps it normal)
    float r = __fmul_rn(v, inv);
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        limb[k] = (uint8_t)__nv_cvt_float_to_fp8(r, __NV_SATFINITE, __NV_E4M3);
        sf[k] = (uint8_t)(e + 127 - 4 * k);
        r = __fmul_rn(__fsub_rn(r, e4m3_to_f32(limb[k])), 16.0f);
    }
}
__global__ void __launch_bounds__(256) act_limbs_kernel(const float *__restrict__ x, int rows, int cols, int64_t ldx, uint8_t *__restrict__ xl,
                                                        uint8_t *__restrict__ xsf) {
    const int64_t unit = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31, nb = cols / 32;
    if (unit >= (int64_t)rows * nb) return;
    const int64_t r = unit / nb, b = unit % nb;
    const float v = x[r * ldx + b * 32 + lane];
    float mx = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    uint8_t limb[3], sf[3];
    limbs_of(v, mx, limb, sf);
#pragma unroll
    for (int k = 0; k < 3; ++k) {
        xl[((int64_t)k * rows + r) * cols + b * 32 + lane] = limb[k];
        if (lane == 0) xsf[((int64_t)k * rows + r) * nb + b] = sf[k];
    }
}

struct TcArgs {
    const void *const *wv;       // [(E+1)*3] tiled values of the registered weights
    const void *const *wsc;      // [(E+1)*3] tiled scales
    const int32_t *items;        // [n][3] = expert, offset into sorted, count (<= NT)
    const int32_t *n_items;
    const int32_t *sorted;       // pair ids grouped by expert
    const int32_t *pair_row;
    const float *pair_weight;
    const uint8_t *xl, *xsf;     // token limbs [3][rows][d], [3][rows][d/32]
    uint8_t *actl, *actsf;       // activation limbs [3][pairs][inter], [3][pairs][inter/32]
    float *outs;                 // [pairs][d]
    int rows, pairs, d, inter;
    int64_t nbp_d, nbp_i;        // padded block counts of the registered weights
    int activation;
    float limit;
    int32_t *status;
};

// One CTA: two 128-row tiles of weights (`wa`, `wb`: tiled values of the two matrices, `rta`, `rtb` their first 16-row tile,
// nbp the padded block count, K the contraction length) against n token rows whose limbs are rows `brow[r]` of (bl, bsf).
// Leaves D0 / D1 in tensor memory columns COL_D0 / COL_D1 of `tb`.  Returns false if a wait ran out.
__device__ __forceinline__ bool tile_pair_mma(unsigned char *sm, uint32_t tb, const unsigned char *wa, const unsigned char *sa, int64_t rta,
                                              const unsigned char *wb, const unsigned char *sb, int64_t rtb, int64_t nbp, int K,
                                              const uint8_t *__restrict__ bl, const uint8_t *__restrict__ bsf, int64_t b_rows,
                                              const int *brow /* smem [NT] */, int n, int32_t *status) {
    const int tid = threadIdx.x, warp = tid >> 5;
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    const uint32_t full0 = s32(&bars[0]), empty0 = s32(&bars[STAGES]);
    const int nsteps = K / KSTEP;
    const int npad = (n + 7) & ~7;
    bool ok = true;
    if (warp < NPROD / 32) {
        // ---------------- producers.  Thread (q, bpl): word q of every chunk of block pair bpl; a chunk of the registered
        // layout is 512 bytes = 128 words, word q = 4 lane + j: lane (g, t) holds 8 codes (columns 8t .. 8t + 7) of block
        // 2 bp + (j >> 1), row g + 8 (j & 1) of a 16-row tile.
        const int p = tid, q = p & 127, bpl = p >> 7;
        const int ln = q >> 2, j = q & 3, g = ln >> 2, t = ln & 3;
        const int rowl = g + ((j & 1) ? 8 : 0), blk = bpl * 2 + (j >> 1);
        const uint32_t cdst = rowl * 128 + ((((blk << 1) + (t >> 1)) ^ (rowl & 7)) << 4) + (t & 1) * 4;
        const unsigned char *srca = wa + (rta * (nbp >> 1) + bpl) * 512 + (size_t)q * 4;
        const unsigned char *srcb = wb + (rtb * (nbp >> 1) + bpl) * 512 + (size_t)q * 4;
        const int64_t tile_stride = (nbp >> 1) * 512;      // next 16-row tile, same block pair
        const int srow = p & 127, smat = p >> 7;           // scale word of row srow of matrix smat
        const unsigned char *srcs = (smat ? sb : sa) + (((smat ? rtb : rta) + (srow >> 4)) * nbp) * 16 + (srow & 15) * 4;
        const uint32_t sdst = smat * 512 + (srow & 31) * 16 + (srow >> 5) * 4;
        for (int it = 0; it < nsteps + STAGES - 1; ++it) {
            if (it < nsteps) {
                const int st = it % STAGES;
                if (it >= STAGES && ok && !bar_wait(empty0 + st * 8, (uint32_t)((it / STAGES) - 1) & 1u)) ok = false;
                unsigned char *stage = sm + (size_t)st * STAGE_BYTES;
                const uint32_t a0 = s32(stage + OFF_A0), a1 = s32(stage + OFF_A1), bb = s32(stage + OFF_B), sf = s32(stage + OFF_SF);
                if (ok) {
                    const unsigned char *sa_it = srca + (int64_t)it * 1024, *sb_it = srcb + (int64_t)it * 1024;   // 2 block pairs per step
#pragma unroll
                    for (int r8 = 0; r8 < 8; ++r8) {
                        cp4(a0 + r8 * 2048 + cdst, sa_it + r8 * tile_stride);
                        cp4(a1 + r8 * 2048 + cdst, sb_it + r8 * tile_stride);
                    }
                    cp4(sf + sdst, srcs + (int64_t)it * 64);          // 4 blocks on: 4 * 16 scale bytes per 16-row tile group
                    // activation limbs: n rows x 128 bytes per limb, and their scale words
                    for (int w = p; w < 3 * n * 8; w += NPROD) {
                        const int limb = w / (n * 8), qq = w % (n * 8), r = qq >> 3, c = qq & 7;
                        cp16(bb + limb * B_BYTES + r * 128 + ((c ^ (r & 7)) << 4), bl + ((int64_t)limb * b_rows + brow[r]) * K + (int64_t)it * KSTEP + c * 16);
                    }
                    if (p < 3 * n) {
                        const int limb = p / n, r = p % n;
                        cp4(sf + (2 + limb) * 512 + r * 16, bsf + ((int64_t)limb * b_rows + brow[r]) * (K / 32) + (int64_t)it * 4);
                    }
                }
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            const int ready = it - (STAGES - 1);
            if (ready >= 0) {
                asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 1) : "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                bar_arrive(full0 + (ready % STAGES) * 8);
            }
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    } else if (tid == NPROD) {
        // ---------------- the MMA-issuing thread
        const uint32_t id[4] = {idesc_mx(npad, 0), idesc_mx(npad, 1), idesc_mx(npad, 2), idesc_mx(npad, 3)};
        for (int it = 0; it < nsteps; ++it) {
            const int st = it % STAGES;
            if (ok && !bar_wait(full0 + st * 8, (uint32_t)(it / STAGES) & 1u)) ok = false;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char *stage = sm + (size_t)st * STAGE_BYTES;
            const uint32_t a0 = s32(stage + OFF_A0), a1 = s32(stage + OFF_A1), bb = s32(stage + OFF_B), sf = s32(stage + OFF_SF);
            const uint32_t tsf = tb + COL_SF + (uint32_t)(it & 1) * 20;
#pragma unroll
            for (int a = 0; a < 5; ++a) sf_copy(tsf + a * 4, sf + a * 512);
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                const uint64_t da0 = smem_desc(a0 + kb * 32, 16, 1024, 2), da1 = smem_desc(a1 + kb * 32, 16, 1024, 2);
#pragma unroll
                for (int limb = 0; limb < 3; ++limb) {
                    const uint64_t db = smem_desc(bb + limb * B_BYTES + kb * 32, 16, 1024, 2);
                    const uint32_t acc = (it > 0 || kb > 0 || limb > 0) ? 1u : 0u;
                    mma_mx(tb + COL_D0, da0, db, id[kb], acc, tsf + 0, tsf + 8 + limb * 4);
                    mma_mx(tb + COL_D1, da1, db, id[kb], acc, tsf + 4, tsf + 8 + limb * 4);
                }
            }
            commit(empty0 + st * 8);      // the stage is free once these MMAs have read it
        }
        commit(s32(&bars[2 * STAGES]));   // everything issued so far has finished: the accumulators are complete
    }
    if (!ok) atomicCAS(status, 0, MK_ERR_TIMEOUT);
    return ok;
}

// Common set-up: barriers, tensor memory, zeroed stages (padding bytes and unused rows must read as zero).
__device__ __forceinline__ uint32_t tc_setup(unsigned char *sm) {
    const int tid = threadIdx.x, warp = tid >> 5;
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    uint32_t *slot = (uint32_t *)(sm + SM_BAR + 64);
    for (int i = tid; i < STAGES * STAGE_BYTES / 16; i += THREADS) ((uint4 *)sm)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&bars[s])), "r"(NPROD));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bars[STAGES + s])));
        }
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&bars[2 * STAGES])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    return *slot;
}
__device__ __forceinline__ void tc_teardown(uint32_t tb) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if ((threadIdx.x >> 5) == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(TMEM_COLS) : "memory");
}

// ---------------------------------------------------------------- gate / up + activation + limbs of the activation
// grid = (inter / 128, max_items).  D0 = w1 tile x tokens, D1 = w3 tile x tokens; then act (src/deepseek.rs:1083-1087 or
// the K3 SiTU, src/model.rs:617-621) and its three limbs per 32 rows, the input of the w2 product.
__global__ void __launch_bounds__(THREADS, 1) moe_tc_gate_up_kernel(const TcArgs a) {
    extern __shared__ unsigned char sm_raw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)sm_raw + 1023) & ~(uintptr_t)1023);
    __shared__ int brow[NT], pair_s[NT];
    __shared__ float wgt_s[NT];
    const int item = blockIdx.y;
    if (item >= *a.n_items) return;
    const int e = a.items[item * 3], off = a.items[item * 3 + 1], n = min(a.items[item * 3 + 2], NT);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < NT) {
        const int p = tid < n ? a.sorted[off + tid] : -1;
        pair_s[tid] = p;
        brow[tid] = p >= 0 ? a.pair_row[p] : 0;
        wgt_s[tid] = p >= 0 ? a.pair_weight[p] : 0.0f;
    }
    const uint32_t tb = tc_setup(sm);
    const int64_t rt = (int64_t)blockIdx.x * 8;
    bool ok = tile_pair_mma(sm, tb, (const unsigned char *)a.wv[e * 3 + 0], (const unsigned char *)a.wsc[e * 3 + 0], rt,
                            (const unsigned char *)a.wv[e * 3 + 2], (const unsigned char *)a.wsc[e * 3 + 2], rt, a.nbp_d, a.d, a.xl, a.xsf, a.rows,
                            brow, n, a.status);
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    if (!bar_wait(s32(&bars[2 * STAGES]), 0u)) { ok = false; atomicCAS(a.status, 0, MK_ERR_TIMEOUT); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        // warp = (lane quadrant q, column half): rows 32 q + lane of the tile, tokens 16 half .. 16 half + 15
        const int q = warp & 3, half = warp >> 2;
        if (warp < 8 && half * 16 < n) {
            float g[16], u[16];
            const uint32_t taddr = tb + ((uint32_t)(q * 32) << 16) + half * 16;
            tmem_ld16(taddr + COL_D0, g);
            tmem_ld16(taddr + COL_D1, u);
            const int64_t col = (int64_t)blockIdx.x * 128 + q * 32 + lane;     // index into the expert's intermediate vector
            const int nbi = a.inter / 32;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const int tk = half * 16 + c;
                if (tk >= n) break;
                float act;
                if (a.activation == MK_MOE_SITU) {
                    act = mk_situ(g[c], u[c]);
                } else {
                    const float gl = fminf(g[c], a.limit);
                    const float ul = fminf(fmaxf(u[c], -a.limit), a.limit);
                    const float silu = __fdiv_rn(gl, __fadd_rn(1.0f, (float)exp((double)(-gl))));
                    act = __fmul_rn(__fmul_rn(wgt_s[tk], silu), ul);
                }
                float mx = fabsf(act);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
                uint8_t limb[3], sf[3];
                limbs_of(act, mx, limb, sf);
                const int64_t p = pair_s[tk];
#pragma unroll
                for (int k = 0; k < 3; ++k) {
                    a.actl[((int64_t)k * a.pairs + p) * a.inter + col] = limb[k];
                    if (lane == 0) a.actsf[((int64_t)k * a.pairs + p) * nbi + (col >> 5)] = sf[k];
                }
            }
        }
    }
    tc_teardown(tb);
}

// ---------------------------------------------------------------- down projection
// grid = (ceil(d / 256), max_items).  D0 / D1 = two consecutive 128-row tiles of w2 x the activation limbs.
__global__ void __launch_bounds__(THREADS, 1) moe_tc_down_kernel(const TcArgs a) {
    extern __shared__ unsigned char sm_raw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)sm_raw + 1023) & ~(uintptr_t)1023);
    __shared__ int brow[NT];
    const int item = blockIdx.y;
    if (item >= *a.n_items) return;
    const int e = a.items[item * 3], off = a.items[item * 3 + 1], n = min(a.items[item * 3 + 2], NT);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < NT) brow[tid] = tid < n ? a.sorted[off + tid] : 0;
    const uint32_t tb = tc_setup(sm);
    const int64_t ntile = a.d / 128;
    const int64_t t0 = (int64_t)blockIdx.x * 2, t1 = t0 + 1 < ntile ? t0 + 1 : t0;   // an odd last tile is computed twice, stored once
    const unsigned char *wv = (const unsigned char *)a.wv[e * 3 + 1], *ws = (const unsigned char *)a.wsc[e * 3 + 1];
    bool ok = tile_pair_mma(sm, tb, wv, ws, t0 * 8, wv, ws, t1 * 8, a.nbp_i, a.inter, a.actl, a.actsf, a.pairs, brow, n, a.status);
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    if (!bar_wait(s32(&bars[2 * STAGES]), 0u)) { ok = false; atomicCAS(a.status, 0, MK_ERR_TIMEOUT); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
        const int q = warp & 3, half = warp >> 2;
        if (warp < 8 && half * 16 < n) {
            const uint32_t taddr = tb + ((uint32_t)(q * 32) << 16) + half * 16;
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                if (tile == 1 && t1 == t0) break;
                float v[16];
                tmem_ld16(taddr + (tile ? COL_D1 : COL_D0), v);
                const int64_t row = (t0 + tile) * 128 + q * 32 + lane;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const int tk = half * 16 + c;
                    if (tk >= n) break;
                    const int64_t p = brow[tk];
                    float o = v[c];
                    // K3 body: the routing weight multiplies the expert output (src/model.rs:2346-2351)
                    if (a.activation == MK_MOE_SITU) o = __fmul_rn(a.pair_weight[p], o);
                    a.outs[p * a.d + row] = o;
                }
            }
        }
    }
    tc_teardown(tb);
}

} // namespace mtc
