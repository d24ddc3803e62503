// Batched MoE experts on the 5th-generation tensor cores: tcgen05.mma kind::mxf8f6f4 with block scales (sm_100a).
//
// For calls with many token rows (the batch-256 layer: ~5 tokens per routed expert, 256 on the shared one) the expert
// matvecs are a real contraction.  Swap-AB: 128 weight rows are the M dimension, an expert's tokens the N dimension.
//   A : the E2M1 codes exactly as the registered weight holds them - no decode.  In shared memory a 16-byte chunk carries
//       16 codes in its low 8 bytes (the tensor core's FP4 operand form: 8 data + 8 padding bytes), rows of 128 bytes
//       (128 codes) in the 128-byte-swizzled K-major layout.  The registered layout (mma.sync fragment order) is brought
//       in as it lies by tiled TMA copies (cp.async.bulk.tensor.2d: one box = 8 row tiles x 1 KB, completion on an
//       mbarrier) into a ring of packed stages, and eight warps re-order each stage into the operand form (16-byte
//       loads, one shuffle, 8-byte stores): the weights keep ONE resident copy.
//   SFA : the ue8m0 scale bytes of the weight, unchanged, 4 blocks per step, copied into tensor memory (tcgen05.cp
//       32x128b.warpx4) in the scale-factor layout: lane r, 32-bit column q, byte k = scale of (row r + 32 q, block k).
//   B : the activations as THREE E4M3 limbs with power-of-two block scales (x = 2^e (h1 + 2^-4 h2 + 2^-8 h3) per block
//       of 32, each limb the E4M3 rounding of what the previous ones left): 12 significant bits per element, products
//       exact, f32 accumulation inside the tensor core.  The limbs are further N columns of the same MMA (column
//       limb * 16 + token, each with its own scale), so a weight tile is read from shared memory once per block; the
//       epilogue adds the three columns of a token.
//       This is NOT the engine's q8_0 activation (src/q8.rs:49-69), whose f32 block scale cannot ride on a block-scaled
//       MMA; it tracks the engine's exact-f32 path (src/mxfp4.rs:488-539) to ~1e-5 of max |y| (tests hold 1e-3).
//   D : f32 accumulators in tensor memory; the epilogue reads them with tcgen05.ld.
// Reference semantics: ds_moe / expert_forward (src/deepseek.rs:1038-1108, 74-95), batched as matvec_packed_nt batches
// (src/model.rs:2412-2447): a (token, expert) result does not depend on which other tokens share the tile.
//
// Persistent CTAs (one per SM, 14 warps), work unit = (work item of <= 16 pairs, two 128-row weight tiles), units dealt
// round-robin.  Warp 13 issues the TMA copies of a step (2 boxes of codes, 2 of scales) as soon as a packed stage is free
// and runs on into the next unit; warps 4-11, two groups that take alternate steps, fetch their step's activation limbs
// one own step ahead (cp.async into a ring of B slots), re-order the packed stage into one of three operand buffers and
// hand it to warp 12, whose first lane copies the scale factors into tensor memory and issues the MMAs into one of two
// accumulator sets; tcgen05.commit hands the operand buffer back and, at the end of a unit, the accumulators to warps
// 0-3, which run the epilogue while the next unit's products are under way.  Every wait is bounded; a wait that runs
// out sets MK_ERR_TIMEOUT in the status word and every role leaves its loop (tensor memory is always freed).  No
// cluster launch, no multicast.
//
// What bounds it (measured with per-role cycle counters on the batch-256 layer, 384 + 1 experts of 7168 x 2048): per step
// of 128 columns (16 KB of codes) the MMA warp is busy ~1000 cycles - a block-scaled MMA of M = 128 costs ~110 cycles
// whatever N is, and a step needs 8 - and the shared-memory traffic (TMA write 17 KB, re-order read 16 KB, re-order
// write 16 KB into half the banks, operand reads ~44 KB) is ~900 cycles; HBM alone would allow 712.  Weights as the N
// operand (N = 256, 4 MMAs per step, one accumulator set) measured no faster: the same shared-memory wall and the
// epilogue no longer overlaps.  The padded FP4 operand form doubles every byte on its way through shared memory; a
// weight layout that TMA can unpack itself (row-major nibbles, 16U4_ALIGN16B boxes) would remove the re-order pass.
#pragma once
#include <cuda_fp8.h>

#include "mk_common.cuh"

namespace mtc {

constexpr int NT = 16;                 // token rows (pairs) per work item
constexpr int KSTEP = 128;
constexpr int NEPI = 128, NCONV = 256, NGRP = 128, THREADS = NEPI + NCONV + 64;   // 4 epilogue + 8 converter warps (2 groups) + the MMA warp + the loader warp
constexpr int W_CONV = NEPI / 32, W_MMA = (NEPI + NCONV) / 32, W_LOAD = W_MMA + 1;
constexpr int NS = 5;                  // packed stages (HBM reads in flight)
constexpr int NM = 3;                  // operand buffers of A
constexpr int NB = 5, LB = 2;          // slots of B; limbs are fetched LB steps ahead (NB >= NM + LB)
constexpr int A_BYTES = 128 * 128;     // one 128-row tile in operand form: [128 rows][128 B]
constexpr int B_BYTES = 3 * NT * 128;  // the three limbs of a step: rows limb * NT + token, [<= 48 rows][128 B]
constexpr int P_BYTES = 2 * 8192 + 2 * 512;   // a packed stage: two tiles of codes (8 row tiles x 1 KB) + their scales (8 x 64 B each)
constexpr int OFF_A = 0;                                   // NM x (A0, A1)
constexpr int OFF_B = OFF_A + NM * 2 * A_BYTES;            // NB x limbs
constexpr int OFF_SFA = OFF_B + NB * B_BYTES;              // NM x 2 atoms of 512 B
constexpr int OFF_SFB = OFF_SFA + NM * 1024;               // NB atoms
constexpr int OFF_P = ((OFF_SFB + NB * 512 + 1023) / 1024) * 1024;   // NS packed stages
constexpr int SM_BAR = OFF_P + NS * P_BYTES;
constexpr int BAR_PFULL = 0, BAR_PEMPTY = NS, BAR_MFULL = 2 * NS, BAR_MEMPTY = 2 * NS + NM, BAR_AFULL = 2 * NS + 2 * NM, BAR_AEMPTY = BAR_AFULL + 2;
constexpr int N_BARS = BAR_AEMPTY + 2;
constexpr int SM_TOTAL = SM_BAR + 256 + 1024;              // barriers, tensor-memory slot, abort flag; + slack to align the base to 1024 bytes
constexpr int TMEM_COLS = 256, ACC_COLS = 6 * NT, COL_D1 = 3 * NT, COL_SF = 2 * ACC_COLS;   // 2 accumulator sets; SF: 2 buffers x 3 atoms x 4 columns
static_assert(N_BARS * 8 <= 192 && SM_TOTAL <= 232448 && NB >= NM + LB, "shared memory of one CTA");
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
// `abort`: a word in shared memory that any role sets when one of its waits ran out; the others then give up at once
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, volatile int *abort) {
    uint32_t done = 0;
    for (uint32_t it = 0; it < WAIT_LIMIT && !done; ++it) {
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (!done && (it & 1023u) == 1023u && *abort) break;
    }
    if (!done) *abort = 1;
    return done != 0;
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp4(uint32_t dst, const void *src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp16(uint32_t dst, const void *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void tma_2d(uint32_t dst, const void *map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst), "l"(map),
                 "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bar_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}\n" ::"r"(bar), "r"(bytes) : "memory");
}
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
    const unsigned char *maps;   // [(E+1)*3][2] tensor maps (128 B each) of the registered weights: tiled codes, tiled scales
    const int32_t *items;        // [n][3] = expert, offset into sorted, count (<= NT)
    const int32_t *n_items;
    const int32_t *sorted;       // pair ids grouped by expert
    const int32_t *pair_row;
    const float *pair_weight;
    const uint8_t *xl, *xsf;     // token limbs [3][rows][d], [3][rows][d/32]
    uint8_t *actl, *actsf;       // activation limbs [3][pairs][inter], [3][pairs][inter/32]
    float *outs;                 // [pairs][d]
    int rows, pairs, d, inter;
    int activation;
    float limit;
    int32_t *status;
};

// Set-up: barriers, tensor memory, zeroed operand buffers (padding bytes and rows no copy ever writes must read as zero).
__device__ __forceinline__ uint32_t tc_setup(unsigned char *sm) {
    const int tid = threadIdx.x, warp = tid >> 5;
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    uint32_t *slot = (uint32_t *)(sm + SM_BAR + 192);
    for (int i = tid; i < OFF_P / 16; i += THREADS) ((uint4 *)sm)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
        auto init = [&](int b, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&bars[b])), "r"(count)); };
        for (int s = 0; s < NS; ++s) { init(BAR_PFULL + s, 1); init(BAR_PEMPTY + s, NGRP / 32); }     // one arrival per warp of the group that converts the step
        for (int s = 0; s < NM; ++s) { init(BAR_MFULL + s, NGRP / 32); init(BAR_MEMPTY + s, 1); }
        for (int s = 0; s < 2; ++s) { init(BAR_AFULL + s, 1); init(BAR_AEMPTY + s, NEPI / 32); }
        slot[1] = 0;     // the abort flag
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

// DOWN = false: gate / up + activation + limbs of the activation.  Unit = (item, 128 rows of w1 and the same rows of w3),
//   K = d; D0 = w1 tile x tokens, D1 = w3 tile x tokens; then act (src/deepseek.rs:1083-1087 or the K3 SiTU,
//   src/model.rs:617-621) and its three limbs per 32 rows, the input of the w2 product.
// DOWN = true: the down projection.  Unit = (item, two consecutive 128-row tiles of w2), K = inter; a tile past the last
//   one reads as zeros (TMA fill) and is not stored.
template <bool DOWN>
__global__ void __launch_bounds__(THREADS, 1) moe_tc_kernel(const TcArgs a) {
    extern __shared__ unsigned char sm_raw[];
    unsigned char *sm = (unsigned char *)(((uintptr_t)sm_raw + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int K = DOWN ? a.inter : a.d, nsteps = K / KSTEP;
    const int ntile = (DOWN ? a.d : a.inter) / 128;
    const int X = DOWN ? (ntile + 1) / 2 : ntile;          // units per item
    const int U = *a.n_items * X, G = (int)gridDim.x, c = (int)blockIdx.x;
    if (c >= U) return;
    const int nunits = (U - c + G - 1) / G;
    const uint32_t tb = tc_setup(sm);
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    volatile int *abort = (volatile int *)(sm + SM_BAR + 196);
    const uint32_t bar0 = s32(bars), smb = s32(sm);
    bool ok = true;

    if (warp == W_LOAD) {
        // ---------------- the loader: the whole warp walks the loop (a lone lane beside 31 parked ones runs slowly),
        // lane 0 issues the four boxes of a step
        {
            int gs = 0;
            int e_next = a.items[(c / X) * 3];
            for (int k = 0; k < nunits && ok; ++k) {
                const int u = c + k * G, xt = u % X, e = e_next;
                if (k + 1 < nunits) e_next = a.items[((u + G) / X) * 3];
                const unsigned char *m0, *m1;
                int y0, y1;
                if (DOWN) { m0 = m1 = a.maps + (size_t)(e * 3 + 1) * 256; y0 = xt * 16; y1 = y0 + 8; }
                else { m0 = a.maps + (size_t)(e * 3 + 0) * 256; m1 = a.maps + (size_t)(e * 3 + 2) * 256; y0 = y1 = xt * 8; }
                for (int it = 0; it < nsteps; ++it, ++gs) {
                    const int ps = gs % NS;
                    if (gs >= NS && !bar_wait(bar0 + (BAR_PEMPTY + ps) * 8, (uint32_t)((gs / NS) - 1) & 1u, abort)) { ok = false; break; }
                    const uint32_t full = bar0 + (BAR_PFULL + ps) * 8, dst = smb + OFF_P + ps * P_BYTES;
                    if (lane == 0) {
                        bar_expect(full, (uint32_t)P_BYTES);
                        tma_2d(dst, m0, it * 256, y0, full);                 // codes: 256 words (2 block pairs) x 8 row tiles
                        tma_2d(dst + 8192, m1, it * 256, y1, full);
                        tma_2d(dst + 16384, m0 + 128, it * 16, y0, full);    // scales: 16 words (4 blocks x 16 rows) x 8 row tiles
                        tma_2d(dst + 16896, m1 + 128, it * 16, y1, full);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == W_MMA) {
        // ---------------- the MMA warp: all lanes wait, lane 0 issues
        {
            int gs = 0;
            for (int k = 0; k < nunits && ok; ++k) {
                const int nn = 3 * NT, acc = k & 1;   // padding tokens ride along: N a multiple of 16 at M = 128
                const uint32_t id[4] = {idesc_mx(nn, 0), idesc_mx(nn, 1), idesc_mx(nn, 2), idesc_mx(nn, 3)};
                if (k >= 2 && !bar_wait(bar0 + (BAR_AEMPTY + acc) * 8, (uint32_t)((k >> 1) - 1) & 1u, abort)) { ok = false; break; }
                const uint32_t d0 = tb + acc * ACC_COLS, d1 = d0 + COL_D1;
                for (int it = 0; it < nsteps; ++it, ++gs) {
                    const int mb = gs % NM, slot = gs % NB;
                    if (!bar_wait(bar0 + (BAR_MFULL + mb) * 8, (uint32_t)(gs / NM) & 1u, abort)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a0 = smb + OFF_A + mb * 2 * A_BYTES, a1 = a0 + A_BYTES, bb = smb + OFF_B + slot * B_BYTES;
                    const uint32_t tsf = tb + COL_SF + (uint32_t)(gs & 1) * 12;
                    if (lane == 0) {
                    sf_copy(tsf + 0, smb + OFF_SFA + mb * 1024);
                    sf_copy(tsf + 4, smb + OFF_SFA + mb * 1024 + 512);
                    sf_copy(tsf + 8, smb + OFF_SFB + slot * 512);
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const uint64_t da0 = smem_desc(a0 + kb * 32, 16, 1024, 2), da1 = smem_desc(a1 + kb * 32, 16, 1024, 2);
                        const uint64_t db = smem_desc(bb + kb * 32, 16, 1024, 2);
                        const uint32_t accum = (it > 0 || kb > 0) ? 1u : 0u;
                        mma_mx(d0, da0, db, id[kb], accum, tsf + 0, tsf + 8);
                        mma_mx(d1, da1, db, id[kb], accum, tsf + 4, tsf + 8);
                    }
                    commit(bar0 + (BAR_MEMPTY + mb) * 8);      // the operand buffer and the B slot are free once these MMAs have read them
                    }
                    __syncwarp();
                }
                if (ok && lane == 0) commit(bar0 + (BAR_AFULL + acc) * 8);  // the unit's accumulators are complete
            }
        }
    } else if (warp >= W_CONV) {
        // ---------------- converters: two groups of four warps, group j takes the steps gs = j (mod 2), so the barrier round
        // trips and shared-memory latencies of one step overlap with the other group's work
        const int cw = warp - W_CONV, grp = cw >> 2, gw = cw & 3, gp = (tid - NEPI) & (NGRP - 1);
        const uint8_t *bl = DOWN ? a.actl : a.xl, *bsf = DOWN ? a.actsf : a.xsf;
        const int64_t b_rows = DOWN ? a.pairs : a.rows;
        // a unit's B rows: this thread copies chunk (gp & 7) of token (gp >> 3), and the scale word of token gp % NT, limb gp / NT
        struct Rows { int n; const uint8_t *main, *sf; };
        auto rows_of = [&](int u) {
            Rows r;
            const int item = u / X, off = a.items[item * 3 + 1];
            r.n = min(a.items[item * 3 + 2], NT);
            const int t0 = gp >> 3, t1 = gp & (NT - 1);
            const int p0 = t0 < r.n ? a.sorted[off + t0] : 0, p1 = t1 < r.n ? a.sorted[off + t1] : 0;
            const int64_t r0 = DOWN ? p0 : a.pair_row[p0], r1 = DOWN ? p1 : a.pair_row[p1];
            r.main = bl + r0 * K + (gp & 7) * 16;
            r.sf = bsf + ((int64_t)(gp / NT) * b_rows + r1) * (K / 32);
            return r;
        };
        const int total = nunits * nsteps;
        int fk = 0, fit = grp;              // fetch cursor of this group: unit, step within it
        while (fit >= nsteps && fk < nunits) { fit -= nsteps; ++fk; }
        Rows cur = rows_of(c + (fk < nunits ? fk : 0) * G), nxt = cur;
        if (fk + 1 < nunits) nxt = rows_of(c + (fk + 1) * G);
        const int64_t limb_stride = b_rows * K;
        const int bt0 = gp >> 3, bch = gp & 7;
        const uint32_t bdst = (uint32_t)(bt0 * 128 + ((bch ^ (bt0 & 7)) << 4));       // limb rows 16 apart keep the swizzle phase
        const bool sf_thread = gp < 3 * NT;
        const uint32_t sfdst = (uint32_t)((gp & 31) * 16 + (gp >> 5) * 4);            // row limb * 16 + token of the scale atom = gp
        auto fetch_b = [&](int f) {         // the limbs of global step f (one of this group's) into slot f % NB
            if (f < total) {
                const int slot = f % NB;
                const uint32_t bb = smb + OFF_B + slot * B_BYTES + bdst, sfb = smb + OFF_SFB + slot * 512 + sfdst;
                if (bt0 < cur.n) {
                    const uint8_t *src = cur.main + (int64_t)fit * KSTEP;
                    cp16(bb, src);
                    cp16(bb + NT * 128, src + limb_stride);
                    cp16(bb + 2 * NT * 128, src + 2 * limb_stride);
                }
                if (sf_thread && (gp & (NT - 1)) < cur.n) cp4(sfb, cur.sf + (int64_t)fit * 4);
                fit += 2;
                while (fit >= nsteps && fk < nunits) {
                    fit -= nsteps; ++fk; cur = nxt;
                    if (fk + 1 < nunits) nxt = rows_of(c + (fk + 1) * G);
                }
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        };
        // Lane (g, t) of a packed 512-byte chunk (16 rows x 2 blocks) holds four words: word j = 8 codes (columns 8t .. 8t + 7)
        // of block (j >> 1), row g + 8 (j & 1).  Lanes t and t ^ 1 together hold the 16 codes of an operand chunk, so even
        // lanes take the partner's words 0, 1 and write block 0, odd lanes take words 2, 3 and write block 1.
        const int g = lane >> 2, t = lane & 3, odd = t & 1;
        const int cpos = (odd << 1) + (t >> 1);                    // 16-byte chunk of the row within the chunk's 2 blocks
        // this warp's chunks: row tiles gw and gw + 4, both block pairs, both matrices
        const uint32_t src_off = (uint32_t)(gw * 1024 + lane * 16);
        // row g of the 16-row tile (row g + 8, 1024 bytes on, has the same swizzle phase), chunk 4 bp + cpos of its 128 bytes
        const uint32_t d_c0 = (uint32_t)(gw * 2048 + g * 128 + ((cpos ^ g) << 4)), d_c1 = (uint32_t)(gw * 2048 + g * 128 + (((4 + cpos) ^ g) << 4));
        fetch_b(grp);
        for (int gs = grp; gs < total; gs += 2) {
            const int mb = gs % NM, ps = gs % NS;
            // operand buffer mb and B slot (gs + 2) % NB were last read by the MMAs of step gs - NM
            if (gs >= NM && ok && !bar_wait(bar0 + (BAR_MEMPTY + mb) * 8, (uint32_t)((gs / NM) - 1) & 1u, abort)) ok = false;
            fetch_b(gs + 2);
            if (ok && !bar_wait(bar0 + (BAR_PFULL + ps) * 8, (uint32_t)(gs / NS) & 1u, abort)) ok = false;
            if (!ok) break;
            const unsigned char *pk = sm + OFF_P + (size_t)ps * P_BYTES;
            unsigned char *am = sm + OFF_A + (size_t)mb * 2 * A_BYTES;
            uint4 w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = *(const uint4 *)(pk + (i >> 2) * 8192 + ((i >> 1) & 1) * 4096 + (i & 1) * 512 + src_off);
#pragma unroll
            for (int i = 0; i < 8; ++i) {          // i = (matrix, row tile half, block pair)
                const uint32_t s0 = odd ? w[i].x : w[i].z, s1 = odd ? w[i].y : w[i].w;
                const uint32_t r0 = __shfl_xor_sync(0xFFFFFFFFu, s0, 1), r1 = __shfl_xor_sync(0xFFFFFFFFu, s1, 1);
                // even lane: (mine, partner's) of words 0, 1; odd lane: (partner's, mine) of words 2, 3
                const uint2 lo = odd ? make_uint2(r0, w[i].z) : make_uint2(w[i].x, r0);
                const uint2 hi = odd ? make_uint2(r1, w[i].w) : make_uint2(w[i].y, r1);
                unsigned char *dst = am + (i >> 2) * A_BYTES + ((i >> 1) & 1) * 4 * 2048 + ((i & 1) ? d_c1 : d_c0);
                *(uint2 *)dst = lo;
                *(uint2 *)(dst + 1024) = hi;
            }
            // scales: packed [matrix][row tile][16 rows][4 blocks of the step]; one word = a row's four scale bytes
#pragma unroll
            for (int smat = 0; smat < 2; ++smat) {
                const int srow = gp;
                const uint32_t v = *(const uint32_t *)(pk + 16384 + smat * 512 + (srow >> 4) * 64 + (srow & 15) * 4);
                *(uint32_t *)(sm + OFF_SFA + mb * 1024 + smat * 512 + (srow & 31) * 16 + (srow >> 5) * 4) = v;
            }
            // one arrival per warp: the warp's reads of the packed stage are done
            __syncwarp();
            if (lane == 0) bar_arrive(bar0 + (BAR_PEMPTY + ps) * 8);
            // ... and its writes (the stores above, the cp.async of this step) are visible to the tensor core's reads
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(bar0 + (BAR_MFULL + mb) * 8);
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    } else {
        // ---------------- epilogue: warp q reads lanes 32 q .. 32 q + 31 of the accumulators (rows of the tile), all tokens
        const int q = warp;
        for (int k = 0; k < nunits; ++k) {
            const int u = c + k * G, item = u / X, xt = u % X, acc = k & 1;
            const int off = a.items[item * 3 + 1], n = min(a.items[item * 3 + 2], NT), npad = NT;
            if (!bar_wait(bar0 + (BAR_AFULL + acc) * 8, (uint32_t)(k >> 1) & 1u, abort)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tb + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
            float v0[16], v1[16], l1[16], l2[16];      // a token's three limb products sit npad columns apart
            tmem_ld16(taddr, v0);
            tmem_ld16(taddr + npad, l1);
            tmem_ld16(taddr + 2 * npad, l2);
#pragma unroll
            for (int i = 0; i < 16; ++i) v0[i] = __fadd_rn(__fadd_rn(v0[i], l1[i]), l2[i]);
            tmem_ld16(taddr + COL_D1, v1);
            tmem_ld16(taddr + COL_D1 + npad, l1);
            tmem_ld16(taddr + COL_D1 + 2 * npad, l2);
#pragma unroll
            for (int i = 0; i < 16; ++i) v1[i] = __fadd_rn(__fadd_rn(v1[i], l1[i]), l2[i]);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(bar0 + (BAR_AEMPTY + acc) * 8);            // the accumulator set may be overwritten
            if (!DOWN) {
                const int64_t col = (int64_t)xt * 128 + q * 32 + lane;     // index into the expert's intermediate vector
                const int nbi = a.inter / 32;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (i >= n) break;
                    const int64_t pid = a.sorted[off + i];
                    float act;
                    if (a.activation == MK_MOE_SITU) {
                        act = mk_situ(v0[i], v1[i]);
                    } else {
                        const float gl = fminf(v0[i], a.limit);
                        const float ul = fminf(fmaxf(v1[i], -a.limit), a.limit);
                        const float silu = __fdiv_rn(gl, __fadd_rn(1.0f, (float)exp((double)(-gl))));
                        act = __fmul_rn(__fmul_rn(a.pair_weight[pid], silu), ul);
                    }
                    float mx = fabsf(act);
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
                    uint8_t limb[3], sf[3];
                    limbs_of(act, mx, limb, sf);
#pragma unroll
                    for (int l = 0; l < 3; ++l) {
                        a.actl[((int64_t)l * a.pairs + pid) * a.inter + col] = limb[l];
                        if (lane == 0) a.actsf[((int64_t)l * a.pairs + pid) * nbi + (col >> 5)] = sf[l];
                    }
                }
            } else {
                const int64_t row0 = (int64_t)(2 * xt) * 128 + q * 32 + lane;
                const bool second = 2 * xt + 1 < ntile;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (i >= n) break;
                    const int64_t pid = a.sorted[off + i];
                    // K3 body: the routing weight multiplies the expert output (src/model.rs:2346-2351)
                    const float w = a.activation == MK_MOE_SITU ? a.pair_weight[pid] : 1.0f;
                    a.outs[pid * a.d + row0] = a.activation == MK_MOE_SITU ? __fmul_rn(w, v0[i]) : v0[i];
                    if (second) a.outs[pid * a.d + row0 + 128] = a.activation == MK_MOE_SITU ? __fmul_rn(w, v1[i]) : v1[i];
                }
            }
        }
    }
    if (!ok) atomicCAS(a.status, 0, MK_ERR_TIMEOUT);
    tc_teardown(tb);
}

} // namespace mtc
