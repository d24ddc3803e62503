// f32 row-times-vector dots in the engine's dot() order (sm_100a).
//
// Reference: dot / dot_scalar (src/model.rs:63-82) - 8 accumulators, element j of
// each 8-chunk into accumulator j with a separate multiply and add, then
// (((a0+a1)+(a2+a3))+(a4+a5))+(a6+a7), tail elements added sequentially - and
// matvec (src/model.rs:199-247),
// which is one such dot per row.  Every kernel here reproduces those bits: 8 lanes
// own the 8 accumulators of one (row, token) pair.
//
// Used by the MoE router (rows = experts), the f32 matvec entry points and the K3
// latent MoE (routed_down / routed_up / shared expert).
#pragma once
#include "mk_common.cuh"

namespace mkf {

// the engine's reduction of the 8 accumulators held by lanes base..base+7
__device__ __forceinline__ float reduce8(float acc, int lane) {
    const int base = lane & ~7;
    const float v1 = __fadd_rn(acc, __shfl_xor_sync(0xFFFFFFFFu, acc, 1)); // a(2i) + a(2i+1)
    const float p01 = __shfl_sync(0xFFFFFFFFu, v1, base + 0), p23 = __shfl_sync(0xFFFFFFFFu, v1, base + 2);
    const float p45 = __shfl_sync(0xFFFFFFFFu, v1, base + 4), p67 = __shfl_sync(0xFFFFFFFFu, v1, base + 6);
    return __fadd_rn(__fadd_rn(__fadd_rn(p01, p23), p45), p67);
}

// Tiled form (cols a multiple of 4, rows 16-byte aligned): one CTA of 256 threads =
// NE matrix rows x NT tokens, NE * NT <= 32.  The NE matrix rows and the NT token rows
// stream through shared memory in slices of KC columns, STAGES slices in flight
// (cp.async).  (row, token) pair p = 4 * warp + (lane >> 3) -> row p / NT, token p % NT;
// its 8 lanes run the 8 accumulator chains in order.  Warps without a pair only copy.
template <int NE_, int NT_, int KC_, int STAGES_>
struct TileShape {
    static constexpr int NE = NE_, NT = NT_, KC = KC_, STAGES = STAGES_, ROWS = NE_ + NT_, LD = KC_ + 8;
    static constexpr size_t SMEM = (size_t)STAGES_ * ROWS * LD * sizeof(float);
    static_assert(NE_ * NT_ <= 32, "one octet of lanes per (row, token) pair, 32 octets per CTA");
    static_assert(NT_ == 1 || NT_ == 2 || NT_ % 4 == 0, "a warp's 4 pairs share a row or a token");
};

__device__ __forceinline__ void cp16(float *dst, const float *src) {
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(src) : "memory");
}

// dot(w[row], x[tok]) for the pair of this lane's octet; the result is meaningful in the
// lanes with (lane & 7) == 0 and *valid set.  w: [n_rows][d], x: [n_tokens][d].
template <class S>
__device__ __forceinline__ float tile_dot(const float *__restrict__ w, const float *__restrict__ x, int n_rows, int d, int n_tokens,
                                          int row0, int tok0, float *smem, int *row_out, int *tok_out, bool *valid) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, sub = lane >> 3, j = lane & 7;
    const int full = d & ~7;
    const int nch = (full + S::KC - 1) / S::KC;
    const int ntl = min(S::NT, n_tokens - tok0), nrl = min(S::NE, n_rows - row0), nrows = S::NE + ntl;
    auto issue = [&](int ch) {
        float *stage = smem + (size_t)(ch % S::STAGES) * S::ROWS * S::LD;
        const int c0 = ch * S::KC;
        for (int idx = tid; idx < nrows * (S::KC / 4); idx += 256) {
            const int r = idx / (S::KC / 4), c = c0 + (idx % (S::KC / 4)) * 4;
            if (c >= full) continue;                 // full is a multiple of 8, c of 4: c < full => c + 3 < full
            const float *src = r < S::NE ? w + (size_t)(row0 + min(r, nrl - 1)) * d + c : x + (size_t)(tok0 + r - S::NE) * d + c;
            cp16(stage + r * S::LD + (c - c0), src);
        }
    };
    for (int sidx = 0; sidx < S::STAGES - 1; ++sidx) {
        if (sidx < nch) issue(sidx);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    const int p = warp * 4 + sub;
    const int rl = p / S::NT, tl = p % S::NT;
    const bool act = warp * 4 < S::NE * S::NT && (warp * 4) / S::NT < nrl && (S::NT < 4 || (warp * 4) % S::NT < ntl);
    float acc = 0.0f;
    for (int ch = 0; ch < nch; ++ch) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(S::STAGES - 2) : "memory");
        __syncthreads();
        if (ch + S::STAGES - 1 < nch) issue(ch + S::STAGES - 1);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        if (act) {
            const float *stage = smem + (size_t)(ch % S::STAGES) * S::ROWS * S::LD;
            const float *ws = stage + min(rl, nrl - 1) * S::LD + j, *xr = stage + (S::NE + min(tl, ntl - 1)) * S::LD + j;
            const int kmax = min(S::KC, full - ch * S::KC);
#pragma unroll 32
            for (int c = 0; c < kmax; c += 8) acc = __fadd_rn(acc, __fmul_rn(ws[c], xr[c]));
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    float sres = reduce8(acc, lane);
    const int row = row0 + rl, tok = tok0 + tl;
    *valid = act && j == 0 && p < S::NE * S::NT && rl < nrl && tl < ntl;
    if (*valid)
        for (int c = full; c < d; ++c) sres = __fadd_rn(sres, __fmul_rn(__ldg(w + (size_t)row * d + c), __ldg(x + (size_t)tok * d + c)));
    *row_out = row;
    *tok_out = tok;
    return sres;
}

// Generic form (any d, any alignment): a warp = 4 rows, T tokens per lane octet, operands
// straight from global memory.  The result of (row, tok0 + t) is in out[t] of the lanes with
// (lane & 7) == 0.
template <int T>
__device__ __forceinline__ void rows_dot(const float *__restrict__ w, const float *__restrict__ x, int d, int n_tokens, int tok0,
                                         bool row_valid, int lane, float (&out)[T]) {
    const int j = lane & 7;
    float acc[T];
#pragma unroll
    for (int t = 0; t < T; ++t) acc[t] = 0.0f;
    const int full = d & ~7;
#pragma unroll 4
    for (int c = 0; c < full; c += 8) {
        const float wv = __ldg(w + c + j);
#pragma unroll
        for (int t = 0; t < T; ++t) {
            const int tok = min(tok0 + t, n_tokens - 1);
            acc[t] = __fadd_rn(acc[t], __fmul_rn(wv, __ldg(x + (size_t)tok * d + c + j)));
        }
    }
#pragma unroll
    for (int t = 0; t < T; ++t) {
        float s = reduce8(acc[t], lane);
        if (j == 0 && row_valid && tok0 + t < n_tokens)
            for (int c = full; c < d; ++c) s = __fadd_rn(s, __fmul_rn(__ldg(w + c), __ldg(x + (size_t)(tok0 + t) * d + c)));
        out[t] = s;
    }
}

// Register-tiled form for many tokens (>= 64): one CTA (128 threads) = 16 matrix rows (experts) x 16 tokens, every lane octet
// 4 rows x 4 tokens.  Each of the 16 (expert, token) pairs of an octet keeps the engine's dot(): lane j sums the columns = j (mod 8)
// in ascending order with a separate multiply and add, then the 8 partial sums fold in the engine's tree (mkf::reduce8).
// The products are issued two at a time (mul.rn.f32x2: each half rounded as the scalar instruction rounds it), the sums
// stay scalar: a packed multiply feeding a packed add came back a few ulps off the engine's bits - contracted into a
// packed multiply-add - so the two are kept in different forms.  A quarter fewer instructions in an issue-bound kernel.  Against the 2 x 16 shape
// this reads each router row and token row 4 x less often from L2.  384 experts x 256 tokens are 384 CTAs, all resident
// at once (52 KB of shared memory each), 2 or 3 per SM.  Slices of 128 columns, 3 in flight (cp.async); d % 4 == 0,
// 16-byte aligned rows.
constexpr int RG_TE = 16, RG_TT = 16, RG_KC = 128, RG_ST = 3, RG_LD = RG_KC + 8, RG_ROWS = RG_TE + RG_TT, RG_THREADS = 128;
constexpr size_t RG_SMEM = (size_t)RG_ST * RG_ROWS * RG_LD * sizeof(float);
__device__ __forceinline__ uint64_t f32x2_pack(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t f32x2_mul(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ void f32x2_unpack(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
// One CTA's 16 x 16 tile of products (matrix rows e0 .., token rows t0 ..): store(row, token, value) is called once for every
// pair inside the matrix, by the lane that holds its folded sum.
template <class Store>
__device__ __forceinline__ void reg_tile_product(const float *__restrict__ w, const float *__restrict__ x, int rows, int d, int n, int e0, int t0,
                                                 float *__restrict__ gsm, Store store) {
    const int tid = threadIdx.x, lane = tid & 31, oct = tid >> 3, j = lane & 7;
    const int ne = min(RG_TE, rows - e0), nt = min(RG_TT, n - t0);
    // octet -> experts eg, eg + 4, eg + 8, eg + 12 and tokens tg, tg + 4, tg + 8, tg + 12: the four octets of a warp share their
    // router rows (one broadcast read) and read neighbouring token rows (8 banks apart)
    const int eg = oct >> 2, tg = oct & 3;
    const int full = d & ~7, nch = (full + RG_KC - 1) / RG_KC;
    // this thread's part of a slice: column (tid & 31) * 4 of rows (tid >> 5) + 4 k
    constexpr int NCP = RG_ROWS * (RG_KC / 4) / RG_THREADS;
    const float *src[NCP];
#pragma unroll
    for (int k = 0; k < NCP; ++k) {
        const int r = (tid >> 5) + 4 * k;
        src[k] = (r < RG_TE ? w + (size_t)(e0 + min(r, ne - 1)) * d : x + (size_t)(t0 + min(r - RG_TE, nt - 1)) * d) + (tid & 31) * 4;
    }
    const int dst0 = (tid >> 5) * RG_LD + (tid & 31) * 4;
    auto issue = [&](int ch) {
        float *stage = gsm + (size_t)(ch % RG_ST) * RG_ROWS * RG_LD + dst0;
        const int c0 = ch * RG_KC;
        if (c0 + (tid & 31) * 4 >= full) return;
#pragma unroll
        for (int k = 0; k < NCP; ++k) mkf::cp16(stage + 4 * k * RG_LD, src[k] + c0);
    };
    for (int sidx = 0; sidx < RG_ST - 1; ++sidx) {
        if (sidx < nch) issue(sidx);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0.0f;
    for (int ch = 0; ch < nch; ++ch) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(RG_ST - 2) : "memory");
        __syncthreads();
        if (ch + RG_ST - 1 < nch) issue(ch + RG_ST - 1);
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        const float *stage = gsm + (size_t)(ch % RG_ST) * RG_ROWS * RG_LD;
        const float *ws = stage + eg * RG_LD + j, *xr = stage + (RG_TE + tg) * RG_LD + j;
        const int kmax = min(RG_KC, full - ch * RG_KC);
#pragma unroll 4
        for (int c = 0; c < kmax; c += 8) {
            float wv[4], xv[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) { wv[a] = ws[(4 * a) * RG_LD + c]; xv[a] = xr[(4 * a) * RG_LD + c]; }
            const uint64_t x01 = f32x2_pack(xv[0], xv[1]), x23 = f32x2_pack(xv[2], xv[3]);
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const uint64_t w2 = f32x2_pack(wv[a], wv[a]);
                float p0, p1, p2, p3;
                f32x2_unpack(f32x2_mul(w2, x01), p0, p1);
                f32x2_unpack(f32x2_mul(w2, x23), p2, p3);
                acc[a][0] = __fadd_rn(acc[a][0], p0);
                acc[a][1] = __fadd_rn(acc[a][1], p1);
                acc[a][2] = __fadd_rn(acc[a][2], p2);
                acc[a][3] = __fadd_rn(acc[a][3], p3);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
    for (int a = 0; a < 4; ++a) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float sres = mkf::reduce8(acc[a][b], lane);
            const int el = eg + 4 * a, tl = tg + 4 * b;
            if (j == 0 && el < ne && tl < nt) {
                const int e = e0 + el, tok = t0 + tl;
                for (int c = full; c < d; ++c) sres = __fadd_rn(sres, __fmul_rn(__ldg(w + (size_t)e * d + c), __ldg(x + (size_t)tok * d + c)));
                store(e, tok, sres);
            }
        }
    }
}

} // namespace mkf
