// Batched MoE experts on the 5th-generation tensor cores: tcgen05.mma kind::mxf4 with block scales (sm_100a).
//
// For calls with many token rows (the batch-256 layer: ~5 tokens per routed expert, 256 on the shared one) the expert
// matvecs are a real contraction.  Swap-AB: 128 weight rows are the M dimension, an expert's tokens the N dimension,
// both operands FP4 (E2M1) with ue8m0 scales per 32 - the weight's own format - K = 64 per MMA.
//   A : the E2M1 codes of the weight in the engine's byte order (two codes per byte, low nibble = even column,
//       src/mxfp4.rs:19-31), blocked so that the 256 codes x 128 rows of a step are one contiguous 16 KB run in HBM
//       (tc_weight_copy_kernel); a tiled TMA copy (cp.async.bulk.tensor.2d, box = 128 bytes x 128 rows, SWIZZLE_128B, no
//       multicast) lands it as the K-major operand tile.  The mma.sync decode kernels read the weights in their fragment
//       order, so a layer created for this path holds a second copy of its experts (made on the device at
//       mk_moe_create): twice the weight memory, meant for layers that see prefill-sized batches.
//   SFA : the ue8m0 scale bytes of the weight, unchanged, as 512-byte atoms per (128-row tile, 4 blocks) in the layout
//       tcgen05.cp 32x128b.warpx4 expects: lane r, 32-bit column q, byte k = scale of (row r + 32 q, block k); an MMA
//       (2 blocks) takes bytes 0-1 or 2-3 of the word.
//   B : the activations as SIX E2M1 limbs with power-of-two block scales: per block of 32, e = the smallest exponent
//       with max|x| <= 6 * 2^e, limb l = E2M1 rounding of what the previous limbs left, at scale 2^(e - 2l): every
//       limb takes the remainder down by 4, after six it is <= 2^(e - 10) <= max|x| / 3072, every product exact, f32
//       accumulation in the tensor core.  The limbs are further N columns of the same MMA (column limb * 16 + token,
//       each with its own scale); the epilogue adds the six columns of a token.
//       This is NOT the engine's q8_0 activation (src/q8.rs:49-69), whose f32 block scale cannot ride on a block-scaled
//       MMA; it tracks the engine's exact-f32 path (src/mxfp4.rs:488-539) (tests hold 1e-3 of max |y|).
//   D : f32 accumulators in tensor memory (two sets); the epilogue reads them with tcgen05.ld.
// Reference semantics: ds_moe / expert_forward (src/deepseek.rs:1038-1108, 74-95), batched as matvec_packed_nt batches
// (src/model.rs:2412-2447): a (token, expert) result does not depend on which other tokens share the tile.
//
// Persistent CTAs (one per SM, 11 warps), work unit = (work item of <= 16 pairs, two 128-row weight tiles), a step = 256
// columns (32 KB of codes), units dealt round-robin.  Warp 10 asks L2 for a step's boxes some steps ahead
// (cp.async.bulk.prefetch) and issues the copies of a step (2 TMA boxes of codes, 2 bulk copies of scale atoms) as soon
// as a stage is free, running on into the next unit; warps 4-7 fetch the step's activation limbs (cp.async) into the
// stage's B slot and count themselves in on the same barrier; warps 8 and 9 take alternate steps: wait for the stage,
// copy the scale factors into tensor memory and issue the 8 MMAs into one of two accumulator sets, handing over
// through a named barrier so that the MMAs keep the order of the steps; tcgen05.commit hands the stage back and, at
// the end of a unit, the accumulators to warps 0-3, which run the epilogue while the next unit's products are under
// way.  Every mbarrier wait is bounded; a wait that runs out sets MK_ERR_TIMEOUT in the status word, the roles stop
// issuing and run their loops to the end (so nobody is left at a named barrier) and tensor memory is freed.  No
// cluster launch, no multicast.
//
// History of the operand path, all measured on the batch-256 layer (384 + 1 experts of 7168 x 2048, experts alone, HBM
// roofline 0.97 ms, 712 cycles per 16 KB of codes): kind::mxf8f6f4 (weights FP4 in the padded operand form, activations
// as three E4M3 limbs, K = 32 per MMA, 8 MMAs per 16 KB of codes at ~125 cycles each whatever N is) - weights kept only
// in the mma.sync fragment order and re-ordered in shared memory by eight warps 2.55 ms (shared-memory pipe 69 % busy),
// 4-byte cp.async scatter 6.4 ms, 1-KB bulk copies 4.9 ms, TMA's 4-bit unpack (16U4_ALIGN16B boxes) of row-major nibbles
// 2.43 ms, of a blocked copy 2.13 ms with the tensor pipe as the bound (~1010 cycles per 16 KB).  kind::mxf4 halves the
// MMAs per byte.  Weights as the N operand (N = 256, one accumulator set) left the epilogue unoverlapped and was no
// faster; M = 64 is refused by the hardware for block-scaled kinds with cta_group::1.
#pragma once
#include <cuda_fp8.h>

#include "mk_common.cuh"

namespace mtc {

constexpr int NT = 16;                 // token rows (pairs) per work item
constexpr int NL = 6;                  // E2M1 limbs of an activation
constexpr int KSTEP = 256;             // columns per step: one 128-byte swizzled row of packed codes
constexpr int NEPI = 128, NFETCH = 128, THREADS = NEPI + NFETCH + 96;   // 4 epilogue + 4 limb-fetch warps + 2 MMA warps + the loader warp
constexpr int W_FETCH = NEPI / 32, W_MMA = (NEPI + NFETCH) / 32, W_LOAD = W_MMA + 2;
constexpr int NS = 4;                  // stages (HBM reads in flight: NS x 34 KB)
constexpr int PF = 6;                  // the loader asks L2 for a step's boxes PF steps before it loads them
constexpr int LAG = 2;                 // the limb fetchers signal a stage LAG steps after issuing its copies
constexpr int A_BYTES = 128 * 128;     // one 128-row tile of a step: [128 rows][128 B = 256 codes]
constexpr int B_BYTES = NL * NT * 128; // the limbs of a step: rows limb * NT + token, [96 rows][128 B]
constexpr int ST_A0 = 0, ST_A1 = A_BYTES, ST_SFA = 2 * A_BYTES, ST_SFB = ST_SFA + 2048, ST_B = ST_SFB + 1024;   // SFA: 2 tiles x 2 atoms, SFB: 2 atoms
constexpr int STAGE_BYTES = ((ST_B + B_BYTES + 1023) / 1024) * 1024;
constexpr uint32_t STEP_TX = 2 * 16384 + 2 * 1024;         // bytes the loader's four copies of a step bring
constexpr int SM_BAR = NS * STAGE_BYTES;
constexpr int BAR_FULL = 0, BAR_EMPTY = NS, BAR_ACCF = 2 * NS, BAR_ACCE = 2 * NS + 2;
constexpr int N_BARS = BAR_ACCE + 2;
constexpr int SM_TOTAL = SM_BAR + 256 + 1024;              // barriers, tensor-memory slot, abort flag; + slack to align the base to 1024 bytes
constexpr int NCOL = NL * NT;                              // accumulator columns of one tile: limb * NT + token
constexpr int TMEM_COLS = 512, ACC_COLS = 2 * NCOL, COL_D1 = NCOL, COL_SF = 2 * ACC_COLS;   // 2 accumulator sets; SF: 2 buffers x 6 atoms x 4 columns
static_assert(N_BARS * 8 <= 192 && SM_TOTAL <= 232448 && COL_SF + 48 <= TMEM_COLS, "shared and tensor memory of one CTA");
constexpr uint32_t WAIT_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t layout) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) |
           (1ull << 46) | (layout << 61);
}
// block-scaled instruction descriptor of kind::mxf4: A = B = E2M1 (format 1), ue8m0 scales, M = 128, N = n, K = 64; `sf` = first
// of the two scale bytes of both operands' scale words (0 or 2)
__device__ __forceinline__ uint32_t idesc_mx(int n, int sf) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | ((uint32_t)sf << 29) | ((uint32_t)sf << 4);
}
__device__ __forceinline__ void mma_mx(uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc, uint32_t sfa, uint32_t sfb) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], p;\n\t}\n" ::"r"(d), "l"(da), "l"(db), "r"(idesc),
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
// L2 eviction priorities: the weights stream through once (evict_first), the activation limbs are read again by every
// tile of every expert their token visits (evict_last) - without the hints the stream pushes limb rows out of L2 and
// they come back from HBM
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void cp16(uint32_t dst, const void *src, uint64_t pol) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "l"(pol) : "memory");
}
__device__ __forceinline__ void tma_2d(uint32_t dst, const void *map, int x, int y, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;\n" ::"r"(dst),
                 "l"(map), "r"(x), "r"(y), "r"(bar), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// requests into L2 only (no shared memory, no completion to wait for): the same box / run a later step will load
__device__ __forceinline__ void tma_2d_prefetch(const void *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_prefetch(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(src), "r"(bytes) : "memory");
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

// ---------------------------------------------------------------- activations -> six E2M1 limbs per block of 32
// e = the smallest exponent with mx <= 6 * 2^e; limb l = the E2M1 code nearest to the remainder at scale 2^(e - 2l) (the
// remainder after a limb is at most 1 at that limb's scale, i.e. 4 <= 6 at the next); scale bytes e + 127 - 2l (ue8m0).
// Everything exact in f32.  A zero (or non-finite) block gets zero limbs.
__device__ __forceinline__ void limbs_of(float v, float mx, uint32_t (&code)[NL], uint8_t (&sf)[NL]) {
    if (!(mx > 0.0f) || !(mx < INFINITY)) {
#pragma unroll
        for (int l = 0; l < NL; ++l) { code[l] = 0u; sf[l] = 127; }
        return;
    }
    const uint32_t mb = __float_as_uint(mx);
    int e = (int)((mb >> 23) & 0xFF) - 127 - (((mb & 0x7FFFFFu) <= 0x400000u) ? 2 : 1);   // mx = m 2^E: m <= 1.5 -> E - 2, else E - 1
    e = e < -115 ? -115 : (e > 125 ? 125 : e);                                              // all six scale bytes stay inside ue8m0
    float r = __fmul_rn(v, __uint_as_float((uint32_t)(127 - e) << 23));                      // v 2^-e, exact
#pragma unroll
    for (int l = 0; l < NL; ++l) {
        const float a = fabsf(r);
        const uint32_t idx = a < 0.25f ? 0u : a < 0.75f ? 1u : a < 1.25f ? 2u : a < 1.75f ? 3u : a < 2.5f ? 4u : a < 3.5f ? 5u : a < 5.0f ? 6u : 7u;
        const float val = idx < 4u ? 0.5f * (float)idx : (idx == 4u ? 2.0f : idx == 5u ? 3.0f : idx == 6u ? 4.0f : 6.0f);
        code[l] = idx | (r < 0.0f ? 8u : 0u);
        sf[l] = (uint8_t)(e + 127 - 2 * l);
        r = __fmul_rn(__fsub_rn(r, copysignf(val, r)), 4.0f);
    }
}
// x [rows][cols] f32 -> xl [NL][rows][cols / 2] (two codes per byte, low nibble = even column), xsf [NL][rows][cols / 32].
// A thread takes 8 consecutive columns (four threads = a block of 32) and stores one 32-bit word per limb; `first` and
// `stride` walk the (row, 8 columns) units grid-stride.  cols % 32 == 0, rows of x 16-byte aligned.
__device__ __forceinline__ void act_limbs_body(const float *__restrict__ x, int rows, int cols, int64_t ldx, uint8_t *__restrict__ xl,
                                               uint8_t *__restrict__ xsf, int64_t first, int64_t stride) {
    const int per_row = cols / 8, nb = cols / 32;
    const int64_t total = (int64_t)rows * per_row, padded = (total + 31) & ~(int64_t)31;   // whole warps walk the loop (shuffles below)
    for (int64_t unit = first; unit < padded; unit += stride) {
        const bool live = unit < total;
        const int64_t r = live ? unit / per_row : 0;
        const int c8 = live ? (int)(unit % per_row) : 0;
        float v[8];
        if (live) {
            const float4 lo = *(const float4 *)(x + r * ldx + c8 * 8), hi = *(const float4 *)(x + r * ldx + c8 * 8 + 4);
            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.0f;
        }
        float mx = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(v[i]));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));     // per_row % 4 == 0: the four threads of a block are lanes 4q .. 4q + 3
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        uint32_t word[NL];
        uint8_t sf[NL];
#pragma unroll
        for (int l = 0; l < NL; ++l) word[l] = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t code[NL];
            limbs_of(v[i], mx, code, sf);
#pragma unroll
            for (int l = 0; l < NL; ++l) word[l] |= code[l] << (4 * i);
        }
        if (live) {
#pragma unroll
            for (int l = 0; l < NL; ++l) {
                *(uint32_t *)(xl + ((int64_t)l * rows + r) * (cols / 2) + c8 * 4) = word[l];
                if ((c8 & 3) == 0) xsf[((int64_t)l * rows + r) * nb + (c8 >> 2)] = sf[l];
            }
        }
    }
}

struct TcArgs {
    const unsigned char *maps;   // [(E+1)*3] tensor maps (128 B each) of the blocked copies: rows of 128 bytes, a step's box = 128 consecutive rows
    const uint8_t *atoms;        // scale atoms of matrix i at atoms + i * atom_stride: [rows / 128][K / 128][512]
    int64_t atom_stride;
    const int32_t *items;        // [n][3] = expert, offset into sorted, count (<= NT)
    const int32_t *n_items;
    const int32_t *sorted;       // pair ids grouped by expert
    const int32_t *pair_row;
    const float *pair_weight;
    const int32_t *rows_x, *rows_p;   // [items][NT]: token row / pair id of an item's tokens (one load level for the limb fetchers)
    const uint8_t *xl, *xsf;     // token limbs [NL][rows][d / 2], [NL][rows][d / 32]
    uint8_t *actl, *actsf;       // activation limbs [NL][pairs][inter / 2], [NL][pairs][inter / 32]
    float *outs;                 // [pairs][d]
    int rows, pairs, d, inter;
    int activation;
    float limit;
    int32_t *status;
};

// The tensor-core path's copy of a registered (tiled) MXFP4 matrix [rows][cols], rows % 128 == 0, cols % 256 == 0:
//   vals : nibbles blocked by (128-row tile, 256-column step): [rows / 128][cols / 256][128 rows][128 bytes] - the box a step
//          loads (256 codes x 128 rows) is one contiguous 16 KB run in HBM; within a row the engine's byte order
//          (low nibble = even column, src/mxfp4.rs:19-31)
//   atoms: scale bytes [rows / 128][cols / 128][512]: byte (r % 32) * 16 + (r / 32) * 4 + k = scale of (row r of the tile,
//          block k of the four), the layout tcgen05.cp 32x128b.warpx4 expects; a step takes two consecutive atoms
// tv / ts: the tiled values and scales (weights.cu: 512-byte chunks per 16 rows x 2 blocks; mk_scale_off).
__global__ void __launch_bounds__(256) tc_weight_copy_kernel(const uint32_t *__restrict__ tv, const uint8_t *__restrict__ ts, int64_t rows, int64_t nb,
                                                             int64_t nbp, uint32_t *__restrict__ vals, uint8_t *__restrict__ atoms) {
    const int64_t nrt = rows / 16, nsteps = nb / 8;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < nrt * (nbp / 2) * 128) {
        const int64_t chunk = idx >> 7;
        const int within = (int)(idx & 127), ln = within >> 2, j = within & 3, g = ln >> 2, t = ln & 3;
        const int64_t rt = chunk / (nbp / 2), bp = chunk % (nbp / 2);
        const int64_t row = rt * 16 + g + ((j & 1) ? 8 : 0), blk = bp * 2 + (j >> 1);
        if (blk < nb) vals[(((row >> 7) * nsteps + (blk >> 3)) * 128 + (row & 127)) * 32 + (blk & 7) * 4 + t] = tv[idx];
    }
    if (idx < rows * nb) {
        const int64_t row = idx / nb, blk = idx % nb;
        const int r = (int)(row & 127);
        atoms[((row >> 7) * (nb >> 2) + (blk >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (blk & 3)] = ts[mk_scale_off(row >> 4, nbp, blk, (int)(row & 15))];
    }
}

// Set-up: barriers, tensor memory, zeroed stages (the gap bytes of the FP4 operand form and the rows no copy ever writes
// must read as zero).
__device__ __forceinline__ uint32_t tc_setup(unsigned char *sm) {
    const int tid = threadIdx.x, warp = tid >> 5;
    uint64_t *bars = (uint64_t *)(sm + SM_BAR);
    uint32_t *slot = (uint32_t *)(sm + SM_BAR + 192);
    for (int i = tid; i < NS * STAGE_BYTES / 16; i += THREADS) ((uint4 *)sm)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (tid == 0) {
        auto init = [&](int b, int count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&bars[b])), "r"(count)); };
        for (int s = 0; s < NS; ++s) { init(BAR_FULL + s, 1 + NFETCH / 32); init(BAR_EMPTY + s, 1); }   // full: the loader's arrival with its byte count + one arrival per fetch warp
        for (int s = 0; s < 2; ++s) { init(BAR_ACCF + s, 1); init(BAR_ACCE + s, NEPI / 32); }
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
//   src/model.rs:617-621) and its six limbs per 32 rows, the input of the w2 product.
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
    const int total = nunits * nsteps;
    bool ok = true;

    if (warp == W_LOAD) {
        // ---------------- the loader: the whole warp walks the loop (a lone lane beside 31 parked ones runs slowly), lane 0
        // issues the four copies of a step
        int gs = 0;
        int e_next = a.items[(c / X) * 3];
        struct Src { const unsigned char *m0, *m1; const uint8_t *s0, *s1; int y0, y1; };      // y: first row of the tile's first step in the blocked copy
        auto src_of = [&](int e, int xt) {
            Src r;
            const int i0 = e * 3 + (DOWN ? 1 : 0), i1 = e * 3 + (DOWN ? 1 : 2);
            const int t0 = DOWN ? 2 * xt : xt, t1 = DOWN ? 2 * xt + 1 : xt;              // 128-row tiles of the two matrices
            r.m0 = a.maps + (size_t)i0 * 128; r.m1 = a.maps + (size_t)i1 * 128;
            r.s0 = a.atoms + i0 * a.atom_stride + (size_t)t0 * nsteps * 1024;
            r.s1 = a.atoms + i1 * a.atom_stride + (size_t)min(t1, ntile - 1) * nsteps * 1024;   // a tile past the end: zero codes, any scales
            r.y0 = t0 * nsteps * 128; r.y1 = t1 * nsteps * 128;
            return r;
        };
        auto prefetch = [&](const Src &r, int it) {
            tma_2d_prefetch(r.m0, 0, r.y0 + it * 128);
            tma_2d_prefetch(r.m1, 0, r.y1 + it * 128);
            bulk_prefetch(r.s0 + (size_t)it * 1024, 1024);
            bulk_prefetch(r.s1 + (size_t)it * 1024, 1024);
        };
        const uint64_t pol = policy_evict_first();
        Src cur = src_of(e_next, c % X);
        if (lane == 0) for (int it = 0; it < min(PF, nsteps); ++it) prefetch(cur, it);
        for (int k = 0; k < nunits && ok; ++k) {
            const int u = c + k * G;
            const bool more = k + 1 < nunits;
            Src nxt = cur;
            if (more) nxt = src_of(a.items[((u + G) / X) * 3], (u + G) % X);
            for (int it = 0; it < nsteps; ++it, ++gs) {
                const int st = gs % NS;
                if (lane == 0) {
                    if (it + PF < nsteps) prefetch(cur, it + PF);
                    else if (more && it + PF - nsteps < nsteps) prefetch(nxt, it + PF - nsteps);
                }
                if (gs >= NS && !bar_wait(bar0 + (BAR_EMPTY + st) * 8, (uint32_t)((gs / NS) - 1) & 1u, abort)) { ok = false; break; }
                if (lane == 0) {
                    const uint32_t full = bar0 + (BAR_FULL + st) * 8, dst = smb + st * STAGE_BYTES;
                    bar_expect(full, STEP_TX);
                    tma_2d(dst + ST_A0, cur.m0, 0, cur.y0 + it * 128, full, pol);    // 256 codes x 128 rows: 16 KB, contiguous in HBM
                    tma_2d(dst + ST_A1, cur.m1, 0, cur.y1 + it * 128, full, pol);
                    bulk_g2s(dst + ST_SFA, cur.s0 + (size_t)it * 1024, 1024, full);          // the step's two scale atoms of each tile
                    bulk_g2s(dst + ST_SFA + 1024, cur.s1 + (size_t)it * 1024, 1024, full);
                }
                __syncwarp();
            }
            cur = nxt;
        }
    } else if (warp == W_MMA || warp == W_MMA + 1) {
        // ---------------- two MMA warps on alternate steps: a barrier wait costs ~200 cycles even when the data is there, and
        // issuing a step's MMAs blocks for their ~900 cycles; one warp alone leaves the tensor pipe idle during its waits.
        // The warp of step gs waits for the stage while the other one issues step gs - 1, then takes over through a named
        // barrier (the order of the MMAs into one accumulator must be the order of the steps).  All lanes wait, lane 0 issues.
        const int wid = warp - W_MMA;
        const uint32_t id[2] = {idesc_mx(NCOL, 0), idesc_mx(NCOL, 2)};
        for (int gs = wid; gs < total; gs += 2) {
            const int k = gs / nsteps, it = gs - k * nsteps, acc = k & 1, st = gs % NS;
            if (ok && !bar_wait(bar0 + (BAR_FULL + st) * 8, (uint32_t)(gs / NS) & 1u, abort)) ok = false;
            if (ok && it == 0 && k >= 2 && !bar_wait(bar0 + (BAR_ACCE + acc) * 8, (uint32_t)((k >> 1) - 1) & 1u, abort)) ok = false;
            if (gs > 0) asm volatile("bar.sync %0, 64;" ::"r"(2 + wid) : "memory");      // the other warp has issued step gs - 1
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (ok && lane == 0) {
                const uint32_t d0 = tb + acc * ACC_COLS, d1 = d0 + COL_D1;
                const uint32_t base = smb + st * STAGE_BYTES, a0 = base + ST_A0, a1 = base + ST_A1, bb = base + ST_B;
                const uint32_t tsf = tb + COL_SF + (uint32_t)wid * 24;                     // atoms: A0 x 2, A1 x 2, B x 2
#pragma unroll
                for (int q = 0; q < 4; ++q) sf_copy(tsf + q * 4, base + ST_SFA + q * 512);
                sf_copy(tsf + 16, base + ST_SFB);
                sf_copy(tsf + 20, base + ST_SFB + 512);
#pragma unroll
                for (int kb = 0; kb < 4; ++kb) {                                           // 64 columns each: atom kb / 2, scale bytes 0-1 or 2-3
                    const uint64_t da0 = smem_desc(a0 + kb * 32, 16, 1024, 2), da1 = smem_desc(a1 + kb * 32, 16, 1024, 2);
                    const uint64_t db = smem_desc(bb + kb * 32, 16, 1024, 2);
                    const uint32_t accum = (it > 0 || kb > 0) ? 1u : 0u, at = (uint32_t)(kb >> 1) * 4;
                    mma_mx(d0, da0, db, id[kb & 1], accum, tsf + at, tsf + 16 + at);
                    mma_mx(d1, da1, db, id[kb & 1], accum, tsf + 8 + at, tsf + 16 + at);
                }
                commit(bar0 + (BAR_EMPTY + st) * 8);                       // the stage is free once these MMAs have read it
                if (it == nsteps - 1) commit(bar0 + (BAR_ACCF + acc) * 8);  // the unit's accumulators are complete
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (gs + 1 < total) asm volatile("bar.arrive %0, 64;" ::"r"(2 + (1 - wid)) : "memory");   // hand over to the warp of step gs + 1
        }
    } else if (warp >= W_FETCH) {
        // ---------------- limb fetchers: thread = (token gp >> 3, 16-byte chunk gp & 7) of the six limb rows of a step (256 codes =
        // 128 bytes per row), and, for gp < 96, the eight scale bytes of row gp = limb * NT + token
        const int gp = tid - NEPI;
        const uint8_t *bl = DOWN ? a.actl : a.xl, *bsf = DOWN ? a.actsf : a.xsf;
        const int64_t b_rows = DOWN ? a.pairs : a.rows;
        struct Rows { int n; const uint8_t *main, *sf; };
        const int32_t *rows_tab = DOWN ? a.rows_p : a.rows_x;
        auto rows_of = [&](int u) {
            // independent loads only (issued a unit ahead, they never stall the copies of the current unit)
            Rows r;
            const int item = u / X;
            r.n = min(a.items[item * 3 + 2], NT);
            const int64_t r0 = rows_tab[item * NT + (gp >> 3)], r1 = rows_tab[item * NT + (gp & (NT - 1))];
            r.main = bl + r0 * (K / 2) + (gp & 7) * 16;
            r.sf = bsf + ((int64_t)(gp / NT) * b_rows + r1) * (K / 32);
            return r;
        };
        int fk = 0, fit = 0;
        Rows cur = rows_of(c), nxt = cur;
        if (nunits > 1) nxt = rows_of(c + G);
        const int64_t limb_stride = b_rows * (K / 2);
        const int bt0 = gp >> 3, bch = gp & 7;
        const uint32_t bdst = (uint32_t)(bt0 * 128 + ((bch ^ (bt0 & 7)) << 4));       // limb rows 16 apart keep the swizzle phase
        const bool sf_thread = gp < NL * NT;
        const uint64_t pol = policy_evict_last();
        const uint32_t sfdst = (uint32_t)((gp & 31) * 16 + (gp >> 5) * 4);            // row gp of a scale atom
        for (int f = 0; f < total + LAG; ++f) {
            if (f < total) {
                const int st = f % NS;
                if (f >= NS && ok && !bar_wait(bar0 + (BAR_EMPTY + st) * 8, (uint32_t)((f / NS) - 1) & 1u, abort)) ok = false;
                if (ok) {
                    const uint32_t bb = smb + st * STAGE_BYTES + ST_B + bdst, sfb = smb + st * STAGE_BYTES + ST_SFB + sfdst;
                    if (bt0 < cur.n) {
                        const uint8_t *src = cur.main + (int64_t)fit * (KSTEP / 2);
#pragma unroll
                        for (int l = 0; l < NL; ++l) cp16(bb + l * NT * 128, src + l * limb_stride, pol);
                    }
                    if (sf_thread && (gp & (NT - 1)) < cur.n) {
                        cp4(sfb, cur.sf + (int64_t)fit * 8);                // blocks 0-3 of the step -> atom 0
                        cp4(sfb + 512, cur.sf + (int64_t)fit * 8 + 4);      // blocks 4-7 -> atom 1
                    }
                }
                if (++fit == nsteps) {
                    fit = 0; ++fk; cur = nxt;
                    if (fk + 1 < nunits) nxt = rows_of(c + (fk + 1) * G);
                }
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
            const int ready = f - LAG;
            if (ready >= 0) {
                // the copies of step `ready` have landed: visible to the tensor core's reads, one arrival per warp
                asm volatile("cp.async.wait_group %0;\n" ::"n"(LAG) : "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) bar_arrive(bar0 + (BAR_FULL + ready % NS) * 8);
            }
            if (!ok) break;
        }
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    } else {
        // ---------------- epilogue: warp q reads lanes 32 q .. 32 q + 31 of the accumulators (rows of the tile), all tokens
        const int q = warp;
        for (int k = 0; k < nunits; ++k) {
            const int u = c + k * G, item = u / X, xt = u % X, acc = k & 1;
            const int off = a.items[item * 3 + 1], n = min(a.items[item * 3 + 2], NT);
            if (!bar_wait(bar0 + (BAR_ACCF + acc) * 8, (uint32_t)(k >> 1) & 1u, abort)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr = tb + ((uint32_t)(q * 32) << 16) + acc * ACC_COLS;
            float v0[16], v1[16], t[16];      // a token's limb products sit NT columns apart; added from the finest limb up
            tmem_ld16(taddr + (NL - 1) * NT, v0);
#pragma unroll
            for (int l = NL - 2; l >= 0; --l) {
                tmem_ld16(taddr + l * NT, t);
#pragma unroll
                for (int i = 0; i < 16; ++i) v0[i] = __fadd_rn(v0[i], t[i]);
            }
            tmem_ld16(taddr + COL_D1 + (NL - 1) * NT, v1);
#pragma unroll
            for (int l = NL - 2; l >= 0; --l) {
                tmem_ld16(taddr + COL_D1 + l * NT, t);
#pragma unroll
                for (int i = 0; i < 16; ++i) v1[i] = __fadd_rn(v1[i], t[i]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) bar_arrive(bar0 + (BAR_ACCE + acc) * 8);            // the accumulator set may be overwritten
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
                    uint32_t code[NL];
                    uint8_t sf[NL];
                    limbs_of(act, mx, code, sf);
#pragma unroll
                    for (int l = 0; l < NL; ++l) {          // two columns per byte: the even lane stores its code and its neighbour's
                        const uint32_t hi = __shfl_down_sync(0xFFFFFFFFu, code[l], 1);
                        if (!(lane & 1)) a.actl[((int64_t)l * a.pairs + pid) * (a.inter / 2) + (col >> 1)] = (uint8_t)(code[l] | (hi << 4));
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
