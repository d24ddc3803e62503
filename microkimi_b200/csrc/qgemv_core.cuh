// Warp-level building blocks of the dequant-fused quantized matvec (sm_100a).
//
// One warp owns one 16-row weight tile (optionally one K slice of it) and streams
// it from HBM in mma.m16n8k32 fragment order (see mk_weight in mk_common.cuh).
// Per 32-wide block the dot of the weight row with the q8_0 activation is an
// EXACT int32 (tensor cores, s8 x s8); it is then scaled and accumulated in f32:
//   MXFP4 : acc += idot * (2^(sb-128) * xs)      (src/mxfp4.rs:409-418)
//   q8_0  : acc += (ws * xs) * idot               (src/model.rs:337-347)
// E2M1 codes are decoded in registers with byte permutes: the 3 magnitude bits of
// a code select one of the bytes {0,1,2,3,4,6,8,12} (= E2M1 x 2, src/q8.rs:22); a
// set sign bit makes the permute return 0.  One pass gives the positive part, a
// pass over the sign-flipped word the negative part; idot = dot(pos) - dot(neg).
//
// Two schedules:
//   spread  : <= 2 activation columns.  The 8 MMA columns carry 4 consecutive
//             blocks x 2 columns, so the scaling runs once per 4 blocks with every
//             lane busy; lane t accumulates blocks = t (mod 4).
//   batched : the 8 MMA columns are 8 tokens; a lane owns 4 outputs and adds the
//             block terms in ascending block order with separate multiply and add
//             (bit-identical to the CPU sums when K is not split).
#pragma once
#include <cuda_fp16.h>

#include "mk_common.cuh"

namespace mkq {

enum { W_MXFP4 = 0, W_Q8_F32 = 1, W_Q8_F16 = 2 };

template <int WF> struct Group;
template <> struct Group<W_MXFP4> { uint4 a[2]; };  // 4 blocks = 2 chunks of 512 B
template <> struct Group<W_Q8_F32> { uint4 a[4]; }; // 4 blocks = 4 chunks
template <> struct Group<W_Q8_F16> { uint4 a[4]; };

template <int WF> __host__ __device__ constexpr int chunks_per_group() { return WF == W_MXFP4 ? 2 : 4; }
// bytes of tiled values of one 16-row tile per 4-block group
template <int WF> __host__ __device__ constexpr int group_bytes() { return chunks_per_group<WF>() * 512; }

template <int WF>
__device__ __forceinline__ void load_group(Group<WF> &g, const uint4 *tile_base, int64_t group, int lane) {
    constexpr int C = chunks_per_group<WF>();
    const uint4 *p = tile_base + (group * C) * 32 + lane;
#pragma unroll
    for (int c = 0; c < C; ++c) g.a[c] = mk_ldg_stream(p + c * 32);
}

// Values the kernels receive as launch arguments so that the compiler keeps the
// shift and the bitwise NOT below as integer multiply-adds, which issue on the
// FMA pipe: the ALU pipe, which executes the byte permutes, is the bottleneck of
// the MXFP4 decode.  k16 = 65536 (x >> 16 == mulhi(x, k16)), km1 = 0xFFFFFFFF
// (~x == x * km1 + km1).  zeros: >= 16 zero bytes of device memory.
#ifndef MK_DEC
#define MK_DEC 1      // 0: xor + shifts on the ALU pipe; 1: NOT as a multiply-add (measured fastest); 2: NOT and shifts as multiply-adds
#endif
#ifndef MK_BZERO
#define MK_BZERO 0    // B operand of foreign MMA columns: 0 = AND with a lane mask, 1 = load from a page of zeros
#endif
struct Consts {
    uint32_t k16, km1;
    const int8_t *zeros;
};
// E2M1 x 2 magnitudes in reverse order, bytes {12,8,6,4} and {3,2,1,0}: indexed by
// the complemented magnitude bits of a complemented word.
#define MK_LUT2R_LO 0x0406080Cu
#define MK_LUT2R_HI 0x00010203u

// int32 block dots of block m (0..3) of a group, accumulated into cp (and cn for MXFP4).
// Positive part: selector nibbles with the sign bit set read as 0.  Negative part:
// the same permute over ~w with the reversed table (sign bit cleared <=> negative).
template <int WF>
__device__ __forceinline__ void block_mma(const Group<WF> &g, int m, uint32_t b0, uint32_t b1, int (&cp)[4], int (&cn)[4],
                                          const Consts &k) {
    if constexpr (WF == W_MXFP4) {
        const uint4 &ch = g.a[m >> 1];
        const uint32_t wg = (m & 1) ? ch.z : ch.x; // row g
        const uint32_t wh = (m & 1) ? ch.w : ch.y; // row g+8
#if MK_DEC == 0
        const uint32_t wgx = wg ^ 0x88888888u, whx = wh ^ 0x88888888u;
        mk_mma_s8(cp, mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wg), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wh),
                  mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wg >> 16), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wh >> 16), b0, b1);
        mk_mma_s8(cn, mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wgx), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, whx),
                  mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wgx >> 16), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, whx >> 16), b0, b1);
#elif MK_DEC == 1
        const uint32_t wgn = wg * k.km1 + k.km1, whn = wh * k.km1 + k.km1;
        mk_mma_s8(cp, mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wg), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wh),
                  mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wg >> 16), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wh >> 16), b0, b1);
        mk_mma_s8(cn, mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, wgn), mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, whn),
                  mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, wgn >> 16), mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, whn >> 16), b0, b1);
#else
        const uint32_t wgn = wg * k.km1 + k.km1, whn = wh * k.km1 + k.km1;
        mk_mma_s8(cp, mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wg), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, wh),
                  mk_prmt(MK_LUT2_LO, MK_LUT2_HI, __umulhi(wg, k.k16)), mk_prmt(MK_LUT2_LO, MK_LUT2_HI, __umulhi(wh, k.k16)),
                  b0, b1);
        mk_mma_s8(cn, mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, wgn), mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, whn),
                  mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, __umulhi(wgn, k.k16)),
                  mk_prmt(MK_LUT2R_LO, MK_LUT2R_HI, __umulhi(whn, k.k16)), b0, b1);
#endif
    } else {
        const uint4 &ch = g.a[m];
        mk_mma_s8(cp, ch.x, ch.y, ch.z, ch.w, b0, b1);
    }
}

// weight scales of block b for rows g and g+8; `sc` points at the tile's scales
// ([group of 4 blocks][16 rows][4 blocks])
template <int WF>
__device__ __forceinline__ void load_wscale(const void *sc, int64_t b, int g, float &sg, float &sh) {
    const int64_t o = (b >> 2) * 64 + g * 4 + (b & 3);
    if constexpr (WF == W_MXFP4) {
        const uint8_t *s = (const uint8_t *)sc + o;
        sg = mk_e8m0_half(__ldg(s));
        sh = mk_e8m0_half(__ldg(s + 32));
    } else if constexpr (WF == W_Q8_F32) {
        const float *s = (const float *)sc + o;
        sg = __ldg(s);
        sh = __ldg(s + 32);
    } else {
        const __half *s = (const __half *)sc + o;
        sg = __half2float(__ldg(s));
        sh = __half2float(__ldg(s + 32));
    }
}
// lane (g, t) takes block 4 i + t: element i * 64 + g * 4 + t = i * 64 + lane
template <int WF>
__device__ __forceinline__ void load_wscale_lane(const void *sc, int64_t i, int lane, float &sg, float &sh) {
    if constexpr (WF == W_MXFP4) {
        const uint8_t *s = (const uint8_t *)sc + i * 64 + lane;
        sg = mk_e8m0_half(__ldg(s));
        sh = mk_e8m0_half(__ldg(s + 32));
    } else if constexpr (WF == W_Q8_F32) {
        const float *s = (const float *)sc + i * 64 + lane;
        sg = __ldg(s);
        sh = __ldg(s + 32);
    } else {
        const __half *s = (const __half *)sc + i * 64 + lane;
        sg = __half2float(__ldg(s));
        sh = __half2float(__ldg(s + 32));
    }
}
// the same for the four blocks of group i at once: two vector loads, decoded block by block
template <int WF> struct WScale4;
template <> struct WScale4<W_MXFP4> {
    uint32_t a, b;
    __device__ __forceinline__ void load(const void *sc, int64_t i, int g) {
        const uint8_t *s = (const uint8_t *)sc + i * 64 + g * 4;
        a = __ldg((const uint32_t *)s);
        b = __ldg((const uint32_t *)(s + 32));
    }
    __device__ __forceinline__ void get(int m, float &sg, float &sh) const {
        sg = mk_e8m0_half((a >> (8 * m)) & 0xFFu);
        sh = mk_e8m0_half((b >> (8 * m)) & 0xFFu);
    }
};
template <> struct WScale4<W_Q8_F32> {
    float4 a, b;
    __device__ __forceinline__ void load(const void *sc, int64_t i, int g) {
        const float *s = (const float *)sc + i * 64 + g * 4;
        a = __ldg((const float4 *)s);
        b = __ldg((const float4 *)(s + 32));
    }
    __device__ __forceinline__ void get(int m, float &sg, float &sh) const {
        sg = m == 0 ? a.x : (m == 1 ? a.y : (m == 2 ? a.z : a.w));
        sh = m == 0 ? b.x : (m == 1 ? b.y : (m == 2 ? b.z : b.w));
    }
};
template <> struct WScale4<W_Q8_F16> {
    uint2 a, b;
    __device__ __forceinline__ void load(const void *sc, int64_t i, int g) {
        const __half *s = (const __half *)sc + i * 64 + g * 4;
        a = __ldg((const uint2 *)s);
        b = __ldg((const uint2 *)(s + 32));
    }
    __device__ __forceinline__ void get(int m, float &sg, float &sh) const {
        const uint32_t wa = m < 2 ? a.x : a.y, wb = m < 2 ? b.x : b.y;
        const __half2 ha = *(const __half2 *)&wa, hb = *(const __half2 *)&wb;
        sg = (m & 1) ? __high2float(ha) : __low2float(ha);
        sh = (m & 1) ? __high2float(hb) : __low2float(hb);
    }
};
template <int WF> __host__ __device__ constexpr int scale_elem_bytes() { return WF == W_MXFP4 ? 1 : (WF == W_Q8_F32 ? 4 : 2); }

// acc + idot * (sw * sx), separate multiply and add, in the reference's order
__device__ __forceinline__ float acc_term(float acc, int idot, float sw, float sx) {
    return __fadd_rn(acc, __fmul_rn(__fmul_rn(sw, sx), (float)idot));
}

// the same term with one fused multiply-add; used wherever the CPU's exact bits are
// not promised (both schedules use it, so they still agree with each other)
__device__ __forceinline__ float acc_term_fast(float acc, int idot, float sw, float sx) {
    return fmaf((float)idot, sw * sx, acc);
}

// ---- spread schedule.  `tile`: tiled values of this row tile; `sc`: its scales;
// groups ks, ks+KS, ... < ngroups are processed.  Lane (g,t) feeds MMA column g =
// slot (g&1) of block (g>>1): `xrow` is the q8 row of this lane's slot (nullptr
// when the slot is unused), xs0/xs1 the block scales of slot 0/1.
// Result: out[h][o] for rows g + 8h, already summed over the 4 lanes of a row
// group (every lane of the group holds the total).  X2: slots are the high/low
// limb of one token, one output.
template <int WF, int NSLOT, bool X2>
__device__ __forceinline__ void warp_tile_spread(const uint4 *__restrict__ tile, const void *__restrict__ sc, int64_t ngroups,
                                                 int ks, int KS, int lane, const int8_t *__restrict__ xrow,
                                                 const float *__restrict__ xs0, const float *__restrict__ xs1,
                                                 const Consts &k, float (&out)[2][X2 ? 1 : NSLOT]) {
    constexpr int NOUT = X2 ? 1 : NSLOT;
    const int g = lane >> 2, t = lane & 3;
    const int sub = g >> 1;
    float acc[2][NOUT];
#pragma unroll
    for (int o = 0; o < NOUT; ++o) acc[0][o] = acc[1][o] = 0.0f;
    // B operand of block m of a group: the real activation bytes in the lanes whose
    // column belongs to block m, a page of zeros (stride 0) in all other lanes
#if MK_BZERO
    const int8_t *xb[4];
    uint32_t xstep[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const bool real = (sub == m) && (xrow != nullptr);
        xb[m] = real ? xrow + m * 32 + t * 8 : k.zeros;
        xstep[m] = real ? 128u : 0u;
    }
#else
    const bool xvalid = xrow != nullptr;
    const int8_t *xp = xvalid ? xrow + sub * 32 + t * 8 : k.zeros;
    const uint32_t xstep1 = xvalid ? 128u : 0u;
    uint32_t mask[4];
#pragma unroll
    for (int m = 0; m < 4; ++m) mask[m] = (sub == m && xvalid) ? 0xFFFFFFFFu : 0u;
#endif
    auto process = [&](const Group<WF> &grp, int64_t i) {
        int cp[4] = {0, 0, 0, 0}, cn[4] = {0, 0, 0, 0};
#if MK_BZERO
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const uint2 xv = __ldg((const uint2 *)(xb[m] + (uint64_t)((uint32_t)i * xstep[m])));
            block_mma<WF>(grp, m, xv.x, xv.y, cp, cn, k);
        }
#else
        const uint2 xv = __ldg((const uint2 *)(xp + (uint64_t)((uint32_t)i * xstep1)));
#pragma unroll
        for (int m = 0; m < 4; ++m) block_mma<WF>(grp, m, xv.x & mask[m], xv.y & mask[m], cp, cn, k);
#endif
        // lane t now holds block 4i+t: c0/c1 = row g (slot 0/1), c2/c3 = row g+8
        const int64_t b = i * 4 + t;
        float sg, sh;
        load_wscale_lane<WF>(sc, i, lane, sg, sh);
        int d0 = cp[0], d1 = cp[1], d2 = cp[2], d3 = cp[3];
        if constexpr (WF == W_MXFP4) { d0 -= cn[0]; d1 -= cn[1]; d2 -= cn[2]; d3 -= cn[3]; }
        if constexpr (X2) {
            const float sx = __ldg(xs0 + b);
            acc[0][0] = acc_term_fast(acc[0][0], d0 * 128 + d1, sg, sx);
            acc[1][0] = acc_term_fast(acc[1][0], d2 * 128 + d3, sh, sx);
        } else {
            const float sx0 = __ldg(xs0 + b);
            acc[0][0] = acc_term_fast(acc[0][0], d0, sg, sx0);
            acc[1][0] = acc_term_fast(acc[1][0], d2, sh, sx0);
            if constexpr (NSLOT == 2) {
                const float sx1 = __ldg(xs1 + b);
                acc[0][1] = acc_term_fast(acc[0][1], d1, sg, sx1);
                acc[1][1] = acc_term_fast(acc[1][1], d3, sh, sx1);
            }
        }
    };
    // two register buffers, alternating: the next group is in flight while one is consumed
    Group<WF> ga, gb;
    int64_t i = ks;
    if (i < ngroups) load_group<WF>(ga, tile, i, lane);
    // a launch with programmatic stream serialization starts while the kernel that quantizes the activations still runs:
    // the weights above do not depend on it, the activations below do (returns at once in an ordinary launch)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    while (i < ngroups) {
        const int64_t i1 = i + KS;
        if (i1 < ngroups) load_group<WF>(gb, tile, i1, lane);
        process(ga, i);
        if (i1 >= ngroups) break;
        const int64_t i2 = i1 + KS;
        if (i2 < ngroups) load_group<WF>(ga, tile, i2, lane);
        process(gb, i1);
        i = i2;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int o = 0; o < NOUT; ++o) {
            float v = acc[h][o];
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 1);
            v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);
            out[h][o] = v;
        }
}

// ---- batched schedule.  Lane (g,t) feeds MMA column g from `xcol` (q8 row of that
// column, nullptr = unused) and owns outputs
//   !X2: acc[0] (row g, col 2t) acc[1] (row g, col 2t+1) acc[2] (row g+8, col 2t) acc[3] (row g+8, col 2t+1)
//    X2: columns 2k / 2k+1 are the limbs of token k: acc[0] (row g, token t), acc[2] (row g+8, token t)
// xs_a / xs_b: block scales of this lane's two columns (tokens), nullptr = unused.
// ORDERED = true : one accumulator per output, terms added in ascending block order
//                  (the CPU order when K is not split).
// ORDERED = false: four partial sums per output, one per block position in a group,
//                  combined as (p0+p1)+(p2+p3) - the same association the spread
//                  schedule uses, so a (token, expert) result does not depend on how
//                  many tokens share the pass.
template <int WF, bool X2, bool ORDERED>
__device__ __forceinline__ void warp_tile_batched(const uint4 *__restrict__ tile, const void *__restrict__ sc, int64_t ngroups,
                                                  int ks, int KS, int lane, const int8_t *__restrict__ xcol,
                                                  const float *__restrict__ xs_a, const float *__restrict__ xs_b,
                                                  const Consts &k, float (&acc)[4]) {
    const int g = lane >> 2, t = lane & 3;
    constexpr int NP = ORDERED ? 1 : 4;
    float part[NP][4];
#pragma unroll
    for (int p = 0; p < NP; ++p) part[p][0] = part[p][1] = part[p][2] = part[p][3] = 0.0f;
    const bool xvalid = xcol != nullptr;
    const int8_t *xp = xvalid ? xcol + t * 8 : k.zeros;
    const uint32_t xstep = xvalid ? 32u : 0u;
    auto term = [](float acc_, int idot, float sw, float sx) {
        if constexpr (ORDERED) return acc_term(acc_, idot, sw, sx);
        else return acc_term_fast(acc_, idot, sw, sx);
    };
    const float4 zero4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    auto process = [&](const Group<WF> &grp, int64_t i) {
        WScale4<WF> wsc;
        wsc.load(sc, i, g);
        // activation scales of the group's four blocks (rows of scales are 16-byte aligned: the
        // padded block count is a multiple of 4)
        const float4 xa4 = xs_a ? __ldg((const float4 *)xs_a + i) : zero4;
        const float4 xb4 = (!X2 && xs_b) ? __ldg((const float4 *)xs_b + i) : zero4;
        const float sxa_[4] = {xa4.x, xa4.y, xa4.z, xa4.w}, sxb_[4] = {xb4.x, xb4.y, xb4.z, xb4.w};
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int64_t b = i * 4 + m;
            const uint2 xv = __ldg((const uint2 *)(xp + (uint64_t)((uint32_t)b * xstep)));
            int cp[4] = {0, 0, 0, 0}, cn[4] = {0, 0, 0, 0};
            block_mma<WF>(grp, m, xv.x, xv.y, cp, cn, k);
            int d0 = cp[0], d1 = cp[1], d2 = cp[2], d3 = cp[3];
            if constexpr (WF == W_MXFP4) { d0 -= cn[0]; d1 -= cn[1]; d2 -= cn[2]; d3 -= cn[3]; }
            float(&a)[4] = part[ORDERED ? 0 : m];
            float sg, sh;
            wsc.get(m, sg, sh);
            if constexpr (X2) {
                a[0] = term(a[0], d0 * 128 + d1, sg, sxa_[m]);
                a[2] = term(a[2], d2 * 128 + d3, sh, sxa_[m]);
            } else {
                a[0] = term(a[0], d0, sg, sxa_[m]);
                a[1] = term(a[1], d1, sg, sxb_[m]);
                a[2] = term(a[2], d2, sh, sxa_[m]);
                a[3] = term(a[3], d3, sh, sxb_[m]);
            }
        }
    };
    Group<WF> ga, gb;
    int64_t i = ks;
    if (i < ngroups) load_group<WF>(ga, tile, i, lane);
    while (i < ngroups) {
        const int64_t i1 = i + KS;
        if (i1 < ngroups) load_group<WF>(gb, tile, i1, lane);
        process(ga, i);
        if (i1 >= ngroups) break;
        const int64_t i2 = i1 + KS;
        if (i2 < ngroups) load_group<WF>(ga, tile, i2, lane);
        process(gb, i1);
        i = i2;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if constexpr (ORDERED) acc[j] = part[0][j];
        else acc[j] = __fadd_rn(__fadd_rn(part[0][j], part[1][j]), __fadd_rn(part[2][j], part[3][j]));
    }
}

// pointers into a registered weight for row tile rt
template <int WF>
__device__ __forceinline__ const uint4 *tile_values(const void *values, int64_t rt, int64_t nbp) {
    return (const uint4 *)values + rt * ((nbp >> 2) * chunks_per_group<WF>()) * 32;
}
template <int WF>
__device__ __forceinline__ const void *tile_scales(const void *scales, int64_t rt, int64_t nbp) {
    return (const char *)scales + rt * nbp * 16 * scale_elem_bytes<WF>();
}

} // namespace mkq
