// q8_0 MLA KV cache and decode attention (sm_100a).
//
// Reference: MlaCache::push (src/model.rs:1583-1618) and mla_attn_flash_q8_mqa
// (src/model.rs:1804-1908): the nope part of K and all of V are stored q8_0 per
// head, the rope part f32 once per position; the score is
//   s = (dot(q_rope, kr) + sum_g (qs[g] * ks[g]) * idot_g) * scale
// with idot the exact int32 dot of the q8 query block with the q8 cache block,
// softmax over positions 0..=pos, output = sum_j p_j * (vq_j * vs_j) / l.
//
// Device layout (the cache is written by our own append kernel, so it is laid out
// for the two access patterns of the attention kernel):
//   K side, "position-tiled": positions are cut into tiles of 32.  For one (tile,
//     kv head) the int8 row pieces are stored [16-byte chunk][position][16 B], the
//     block scales [block][position], the rope floats [4-float chunk][position][4]:
//     with lane = position every load of a warp is one contiguous 512 B / 128 B run.
//   V side, natural: [position][kv head][vd] int8 + [position][kv head][vd/32] f32:
//     with lane = 4 output columns a warp reads one contiguous row per position.
// mk_mla_export() returns the engine's own layout.
//
// Kernel: split-KV flash decoding.  One warp owns one (sequence, head, KV split):
// phase 1 scores 32 positions at once (lane = position, dp4a block dots), an online
// softmax step follows the reference's tile recipe, phase 2 accumulates p*V
// (lane = columns).  Splits are merged by a second kernel with a log-sum-exp.
#include "mk_common.cuh"
#include "mla_tc.cuh"

struct mk_mla {
    int layout, H, nope, rope, vd, cap, nseq;
    int kvh;            // kv heads: H (per-head layout) or 1 (absorbed)
    int T;              // position tiles per sequence
    int nb, nbv, NC, RC; // nope/32, vd/32, nope/16, rope/4
    int8_t *kqt; float *kst; float *krt;   // position-tiled K side
    int8_t *vq; float *vs;                 // natural V side (absorbed: the full latent row, its first vd columns are V)
    int vrow;           // bytes per (position, kv head) of vq: vd (per-head) or nope (absorbed)
    int vsrow;          // scales per (position, kv head) of vs
    int *npos_dev;      // [nseq] positions held (device copy, for the batch call)
    int *npos;          // host
    // query staging and split partials
    int8_t *qq; float *qs; int64_t q_nbp;
    float *part_m, *part_l, *part_o;
    int max_split;
};

namespace {

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct MlaDev {
    int H, kvh, nope, rope, vd, cap, T, nb, nbv, NC, RC, vrow, vsrow;
    int8_t *kqt; float *kst; float *krt; int8_t *vq; float *vs;
};

// ------------------------------------------------------------------ append
// One warp per (position, kv head, block): q8::quantize_q8_into of 32 values
// (src/q8.rs:49-69), bit-exact, scattered into the layouts above.  Blocks
// [0, nb) are the K nope blocks, [nb, nb + nbv) the V blocks (per-head layout).
// Absorbed layout: the nb blocks of the latent row go to BOTH sides.
__global__ void __launch_bounds__(256)
mla_append_kernel(const MlaDev c, int seq, int pos0, int n, const float *__restrict__ k_rows, const float *__restrict__ v_rows,
                  int absorbed) {
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int nblk = absorbed ? c.nb : c.nb + c.nbv;
    const int64_t per_pos = (int64_t)c.kvh * nblk;
    if (wid >= (int64_t)n * per_pos) return;
    const int i = (int)(wid / per_pos);
    const int r = (int)(wid % per_pos);
    const int h = r / nblk, b = r % nblk;
    const int j = pos0 + i;
    const int tile = j >> 5, p = j & 31;
    const bool is_k = b < c.nb;
    const int hd = c.nope + c.rope;
    float v;
    if (absorbed) v = k_rows[(int64_t)i * c.nope + b * 32 + lane];
    else if (is_k) v = k_rows[((int64_t)i * c.H + h) * hd + b * 32 + lane];
    else v = v_rows[((int64_t)i * c.H + h) * c.vd + (b - c.nb) * 32 + lane];
    float mx = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    const float dx = __fdiv_rn(mx, 127.0f);
    int q = 0;
    if (dx != 0.0f) q = (int)fminf(fmaxf(roundf(__fdiv_rn(v, dx)), -127.0f), 127.0f);
    const uint32_t qb = (uint32_t)q & 0xFFu;
    const uint32_t pk = qb | (__shfl_down_sync(0xFFFFFFFFu, qb, 1) << 8) | (__shfl_down_sync(0xFFFFFFFFu, qb, 2) << 16) |
                        (__shfl_down_sync(0xFFFFFFFFu, qb, 3) << 24);
    const int64_t th = ((int64_t)seq * c.T + tile) * c.kvh + h;
    if (is_k) {
        const int ch = b * 2 + (lane >> 4);
        if ((lane & 3) == 0) *(uint32_t *)(c.kqt + ((th * c.NC + ch) * 32 + p) * 16 + (lane & 15)) = pk;
        if (lane == 0) c.kst[(th * c.nb + b) * 32 + p] = dx;
    }
    if (!is_k || absorbed) {
        const int vb = absorbed ? b : b - c.nb;
        const int64_t row = ((int64_t)seq * c.cap + j) * c.kvh + h;
        if ((lane & 3) == 0) *(uint32_t *)(c.vq + row * c.vrow + vb * 32 + lane) = pk;
        if (lane == 0) c.vs[row * c.vsrow + vb] = dx;
    }
}
// rope part of K, f32, stored once per position from head 0 (src/model.rs:1592-1593)
__global__ void mla_append_rope_kernel(const MlaDev c, int seq, int pos0, int n, const float *__restrict__ k_rows) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * c.rope) return;
    const int i = idx / c.rope, r = idx % c.rope;
    const int j = pos0 + i, tile = j >> 5, p = j & 31;
    const int hd = c.nope + c.rope;
    c.krt[((((int64_t)seq * c.T + tile) * c.RC + (r >> 2)) * 32 + p) * 4 + (r & 3)] = k_rows[(int64_t)i * c.H * hd + c.nope + r];
}

// ------------------------------------------------------------------ export to the engine's layout
__global__ void mla_export_kernel(const MlaDev c, int seq, int n, int8_t *kq, float *ks, float *kr, int8_t *vq, float *vs) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nk = (int64_t)n * c.kvh * c.nope;
    if (idx < nk) {
        const int e = (int)(idx % c.nope);
        const int h = (int)((idx / c.nope) % c.kvh);
        const int j = (int)(idx / ((int64_t)c.nope * c.kvh));
        const int64_t th = ((int64_t)seq * c.T + (j >> 5)) * c.kvh + h;
        if (kq) kq[idx] = c.kqt[((th * c.NC + (e >> 4)) * 32 + (j & 31)) * 16 + (e & 15)];
        if (ks && (e & 31) == 0) ks[idx / 32] = c.kst[(th * c.nb + (e >> 5)) * 32 + (j & 31)];
    }
    if (kr && idx < (int64_t)n * c.rope) {
        const int r = (int)(idx % c.rope), j = (int)(idx / c.rope);
        kr[idx] = c.krt[((((int64_t)seq * c.T + (j >> 5)) * c.RC + (r >> 2)) * 32 + (j & 31)) * 4 + (r & 3)];
    }
    const int64_t nv = (int64_t)n * c.kvh * c.vd;
    if (vq && idx < nv) {
        const int e = (int)(idx % c.vd);
        const int64_t row = (int64_t)seq * c.cap * c.kvh + idx / c.vd;
        vq[idx] = c.vq[row * c.vrow + e];
        if (vs && (e & 31) == 0) vs[idx / 32] = c.vs[row * c.vsrow + (e >> 5)];
    }
}

} // namespace

namespace {

#define MLA_WARPS 4

// ------------------------------------------------------------------ attention, one warp per (sequence, head, split)
// q8 query rows qq/qs come from the activation quantizer (one row per (seq, head),
// row stride ldq bytes / q_nbp scales); q_f32 gives the rope part.
template <int VW>
__global__ void __launch_bounds__(MLA_WARPS * 32)
mla_attend_kernel(const MlaDev c, const int8_t *__restrict__ qq, const float *__restrict__ qs, int64_t ldq, int64_t q_nbp,
                  const float *__restrict__ q_f32, const int *__restrict__ npos_arr, int npos_fixed, int seq0, float scale,
                  int nsplit, float *__restrict__ part_m, float *__restrict__ part_l, float *__restrict__ part_o,
                  float *__restrict__ out) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, bi = blockIdx.z; // bi: index into q/out; sequence = seq0 + bi
    const int seq = seq0 + bi;
    const int split = blockIdx.x * MLA_WARPS + warp;
    const int hk = c.kvh == 1 ? 0 : h;
    const int hd = c.nope + c.rope;
    uint4 *qq_s = (uint4 *)smem;                                  // nope bytes
    float *qs_s = (float *)(smem + c.nope);                       // nb floats
    float4 *qr_s = (float4 *)(smem + c.nope + ((c.nb * 4 + 15) & ~15)); // rope floats
    {
        const int64_t qrow = (int64_t)bi * c.H + h;
        for (int i = threadIdx.x; i < c.NC; i += blockDim.x) qq_s[i] = ((const uint4 *)(qq + qrow * ldq))[i];
        for (int i = threadIdx.x; i < c.nb; i += blockDim.x) qs_s[i] = qs[qrow * q_nbp + i];
        for (int i = threadIdx.x; i < c.RC; i += blockDim.x) qr_s[i] = ((const float4 *)(q_f32 + qrow * hd + c.nope))[i];
    }
    __syncthreads();
    const int n = npos_arr ? npos_arr[seq] : npos_fixed;
    const int ntiles = (n + 31) >> 5;
    const int tps = (ntiles + nsplit - 1) / nsplit;
    const int t0 = split * tps, t1 = min(t0 + tps, ntiles);
    float m = -INFINITY, l = 0.0f;
    float o[VW * 4];
#pragma unroll
    for (int i = 0; i < VW * 4; ++i) o[i] = 0.0f;

    if (split < nsplit) {
        for (int tile = t0; tile < t1; ++tile) {
            const int j = tile * 32 + lane;
            const bool valid = j < n;
            const int64_t th = ((int64_t)seq * c.T + tile) * c.kvh + hk;
            // ---- phase 1: lane = position
            float acc = 0.0f;
            const uint4 *kq = (const uint4 *)c.kqt + th * c.NC * 32 + lane;
            const float *ks = c.kst + th * c.nb * 32 + lane;
            for (int g = 0; g < c.nb; ++g) {
                int idot = 0;
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const uint4 kw = __ldg(kq + (g * 2 + cc) * 32);
                    const uint4 qw = qq_s[g * 2 + cc];
                    idot = dp4a_s8(kw.x, qw.x, idot);
                    idot = dp4a_s8(kw.y, qw.y, idot);
                    idot = dp4a_s8(kw.z, qw.z, idot);
                    idot = dp4a_s8(kw.w, qw.w, idot);
                }
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(qs_s[g], __ldg(ks + g * 32)), (float)idot));
            }
            float s = 0.0f;
            if (c.rope > 0) {
                // dot() order of src/model.rs:63-82: 8 accumulators over 8-wide chunks
                float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                const float4 *kr = (const float4 *)c.krt + ((int64_t)seq * c.T + tile) * c.RC * 32 + lane;
                for (int c4 = 0; c4 < c.RC; c4 += 2) {
                    const float4 k0 = __ldg(kr + c4 * 32), k1 = __ldg(kr + (c4 + 1) * 32);
                    const float4 q0 = qr_s[c4], q1 = qr_s[c4 + 1];
                    a8[0] = __fadd_rn(a8[0], __fmul_rn(q0.x, k0.x)); a8[1] = __fadd_rn(a8[1], __fmul_rn(q0.y, k0.y));
                    a8[2] = __fadd_rn(a8[2], __fmul_rn(q0.z, k0.z)); a8[3] = __fadd_rn(a8[3], __fmul_rn(q0.w, k0.w));
                    a8[4] = __fadd_rn(a8[4], __fmul_rn(q1.x, k1.x)); a8[5] = __fadd_rn(a8[5], __fmul_rn(q1.y, k1.y));
                    a8[6] = __fadd_rn(a8[6], __fmul_rn(q1.z, k1.z)); a8[7] = __fadd_rn(a8[7], __fmul_rn(q1.w, k1.w));
                }
                s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(a8[0], a8[1]), __fadd_rn(a8[2], a8[3])), __fadd_rn(a8[4], a8[5])),
                              __fadd_rn(a8[6], a8[7]));
            }
            s = __fmul_rn(__fadd_rn(s, acc), scale);
            if (!valid) s = -INFINITY;
            // ---- online softmax step over the 32-position tile
            float tm = s;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xFFFFFFFFu, tm, of));
            const float m_new = fmaxf(m, tm);
            const float corr = expf(m - m_new);
            const float p = valid ? expf(s - m_new) : 0.0f;
            float tl = p;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) tl += __shfl_xor_sync(0xFFFFFFFFu, tl, of);
            l = l * corr + tl;
            m = m_new;
#pragma unroll
            for (int i = 0; i < VW * 4; ++i) o[i] *= corr;
            // ---- phase 2: lane = 4 output columns per 128-column group
            const int cnt = min(32, n - tile * 32);
            const int64_t row0 = ((int64_t)seq * c.cap + tile * 32) * c.kvh + hk;
            for (int i = 0; i < cnt; ++i) {
                const float pi = __shfl_sync(0xFFFFFFFFu, p, i);
                const int64_t row = row0 + (int64_t)i * c.kvh;
                const uint32_t *vw = (const uint32_t *)(c.vq + row * c.vrow);
                const float *vsc = c.vs + row * c.vsrow;
#pragma unroll
                for (int w = 0; w < VW; ++w) {
                    const uint32_t word = __ldg(vw + w * 32 + lane) ^ 0x80808080u; // bytes + 128
                    const float ps = pi * __ldg(vsc + w * 4 + (lane >> 3));
                    // int8 -> f32 without a convert: 0x4B0000xx is 8388608 + xx
                    o[w * 4 + 0] = fmaf(ps, __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7440)) - 8388736.0f, o[w * 4 + 0]);
                    o[w * 4 + 1] = fmaf(ps, __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7441)) - 8388736.0f, o[w * 4 + 1]);
                    o[w * 4 + 2] = fmaf(ps, __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7442)) - 8388736.0f, o[w * 4 + 2]);
                    o[w * 4 + 3] = fmaf(ps, __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7443)) - 8388736.0f, o[w * 4 + 3]);
                }
            }
        }
    }
    if (split >= nsplit) return;
    if (nsplit == 1) {
#pragma unroll
        for (int w = 0; w < VW; ++w)
#pragma unroll
            for (int k = 0; k < 4; ++k) out[((int64_t)bi * c.H + h) * c.vd + (w * 32 + lane) * 4 + k] = __fdiv_rn(o[w * 4 + k], l);
    } else {
        const int64_t pi = ((int64_t)bi * c.H + h) * nsplit + split;
        if (lane == 0) { part_m[pi] = m; part_l[pi] = l; }
#pragma unroll
        for (int w = 0; w < VW; ++w)
            ((float4 *)(part_o + pi * c.vd))[w * 32 + lane] = make_float4(o[w * 4], o[w * 4 + 1], o[w * 4 + 2], o[w * 4 + 3]);
    }
}

// log-sum-exp merge of the split partials: grid (H, nseq), one thread per column
__global__ void mla_merge_kernel(int H, int vd, int nsplit, const float *__restrict__ part_m, const float *__restrict__ part_l,
                                 const float *__restrict__ part_o, float *__restrict__ out) {
    const int64_t bh = (int64_t)blockIdx.y * H + blockIdx.x;
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_m[bh * nsplit + s]);
    float L = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = part_m[bh * nsplit + s];
        if (ms != -INFINITY) L += part_l[bh * nsplit + s] * expf(ms - M);
    }
    for (int col = threadIdx.x; col < vd; col += blockDim.x) {
        float acc = 0.0f;
        for (int s = 0; s < nsplit; ++s) {
            const float ms = part_m[bh * nsplit + s];
            if (ms != -INFINITY) acc += part_o[(bh * nsplit + s) * vd + col] * expf(ms - M);
        }
        out[bh * vd + col] = acc / L;
    }
}

} // namespace

// ====================================================================== host side
#include <new>

static MlaDev mla_dev(const mk_mla *m) {
    MlaDev c;
    c.H = m->H; c.kvh = m->kvh; c.nope = m->nope; c.rope = m->rope; c.vd = m->vd; c.cap = m->cap; c.T = m->T;
    c.nb = m->nb; c.nbv = m->nbv; c.NC = m->NC; c.RC = m->RC; c.vrow = m->vrow; c.vsrow = m->vsrow;
    c.kqt = m->kqt; c.kst = m->kst; c.krt = m->krt; c.vq = m->vq; c.vs = m->vs;
    return c;
}

extern "C" int32_t mk_mla_free(mk_ctx *ctx, mk_mla *m) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr, "NULL argument");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    void *ptrs[] = {m->kqt, m->kst, m->krt, m->vq, m->vs, m->npos_dev, m->qq, m->qs, m->part_m, m->part_l, m->part_o};
    for (void *p : ptrs) if (p) cudaFree(p);
    delete[] m->npos;
    delete m;
    return MK_OK;
}

extern "C" int32_t mk_mla_create(mk_ctx *ctx, const mk_mla_desc *d, mk_mla **out) {
    MK_CHECK_ARG(ctx != nullptr && d != nullptr && out != nullptr, "NULL argument");
    *out = nullptr;
    MK_CHECK_ARG(d->layout == MK_MLA_PER_HEAD || d->layout == MK_MLA_ABSORBED, "unknown layout");
    MK_CHECK_ARG(d->n_heads >= 1 && d->nope >= 32 && d->nope % 32 == 0, "n_heads >= 1 and nope a positive multiple of 32 required");
    MK_CHECK_ARG(d->vd >= 128 && d->vd % 128 == 0 && d->vd <= 512, "vd must be 128, 256, 384 or 512");
    MK_CHECK_ARG(d->rope >= 0 && d->rope % 8 == 0, "rope must be a multiple of 8");
    MK_CHECK_ARG(d->max_positions >= 1 && d->n_seqs >= 1, "max_positions and n_seqs must be positive");
    if (d->layout == MK_MLA_ABSORBED) MK_CHECK_ARG(d->rope == 0 && d->vd <= d->nope, "absorbed layout: rope == 0 and vd <= nope");
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_mla *m = new (std::nothrow) mk_mla();
    if (!m) return MK_ERR_OOM;
    memset(m, 0, sizeof(*m));
    m->layout = d->layout; m->H = d->n_heads; m->nope = d->nope; m->rope = d->rope; m->vd = d->vd;
    m->cap = d->max_positions; m->nseq = d->n_seqs;
    m->kvh = d->layout == MK_MLA_ABSORBED ? 1 : d->n_heads;
    m->T = (m->cap + 31) / 32;
    m->nb = m->nope / 32; m->nbv = m->vd / 32; m->NC = m->nope / 16; m->RC = m->rope / 4;
    m->vrow = d->layout == MK_MLA_ABSORBED ? m->nope : m->vd;
    m->vsrow = d->layout == MK_MLA_ABSORBED ? m->nb : m->nbv;
    m->q_nbp = mk_ceil_div(m->nb, 4) * 4;
    m->max_split = 256;
    m->npos = new (std::nothrow) int[m->nseq]();
    const size_t tiles = (size_t)m->nseq * m->T * m->kvh;
    const size_t rows = (size_t)m->nseq * m->cap * m->kvh;
    const size_t bh = (size_t)m->nseq * m->H;
    cudaError_t e = m->npos ? cudaSuccess : cudaErrorMemoryAllocation;
    if (e == cudaSuccess) e = cudaMalloc(&m->kqt, tiles * m->nope * 32);
    if (e == cudaSuccess) e = cudaMalloc(&m->kst, tiles * m->nb * 32 * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->krt, (size_t)m->nseq * m->T * (m->rope > 0 ? m->rope : 4) * 32 * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->vq, rows * m->vrow);
    if (e == cudaSuccess) e = cudaMalloc(&m->vs, rows * m->vsrow * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->npos_dev, (size_t)m->nseq * 4);
    if (e == cudaSuccess) e = cudaMemsetAsync(m->npos_dev, 0, (size_t)m->nseq * 4, ctx->stream);
    if (e == cudaSuccess) e = cudaMalloc(&m->qq, bh * m->q_nbp * 32);
    if (e == cudaSuccess) e = cudaMalloc(&m->qs, bh * m->q_nbp * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->part_m, bh * m->max_split * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->part_l, bh * m->max_split * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->part_o, bh * m->max_split * m->vd * 4);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        mk_set_error("mk_mla_create: %s", cudaGetErrorString(e));
        mk_mla_free(ctx, m);
        return e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    *out = m;
    return MK_OK;
}

extern "C" int32_t mk_mla_reset(mk_ctx *ctx, mk_mla *m, int32_t seq) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && seq >= -1 && seq < m->nseq, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    for (int s = 0; s < m->nseq; ++s) if (seq < 0 || s == seq) m->npos[s] = 0;
    MK_CUDA(cudaMemcpyAsync(m->npos_dev, m->npos, (size_t)m->nseq * 4, cudaMemcpyHostToDevice, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}
extern "C" int32_t mk_mla_positions(mk_ctx *ctx, const mk_mla *m, int32_t seq) {
    if (!ctx || !m || seq < 0 || seq >= m->nseq) { mk_set_error("mk_mla_positions: bad argument"); return MK_ERR_ARG; }
    return m->npos[seq];
}

extern "C" int32_t mk_mla_append_dev(mk_ctx *ctx, mk_mla *m, int32_t seq, const float *k_rows, const float *v_rows, int32_t n) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && k_rows != nullptr && n >= 1, "bad argument");
    MK_CHECK_ARG(seq >= 0 && seq < m->nseq, "no such sequence");
    const bool absorbed = m->layout == MK_MLA_ABSORBED;
    MK_CHECK_ARG(absorbed || v_rows != nullptr, "v_rows is NULL");
    if (m->npos[seq] + n > m->cap) {
        mk_set_error("mk_mla_append: sequence %d holds %d of %d positions, cannot append %d", seq, m->npos[seq], m->cap, n);
        return MK_ERR_STATE;
    }
    MK_CUDA(cudaSetDevice(ctx->device));
    const MlaDev c = mla_dev(m);
    mk_prof_scope prof(ctx, MK_PROF_MLA);
    const int nblk = absorbed ? m->nb : m->nb + m->nbv;
    const int64_t warps = (int64_t)n * m->kvh * nblk;
    mla_append_kernel<<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(c, seq, m->npos[seq], n, k_rows, v_rows, absorbed ? 1 : 0);
    ctx->launches++;
    if (m->rope > 0) {
        mla_append_rope_kernel<<<(unsigned)mk_ceil_div((int64_t)n * m->rope, 128), 128, 0, ctx->stream>>>(c, seq, m->npos[seq], n, k_rows);
        ctx->launches++;
    }
    MK_CUDA(cudaGetLastError());
    m->npos[seq] += n;
    MK_CUDA(cudaMemcpyAsync(m->npos_dev + seq, m->npos + seq, 4, cudaMemcpyHostToDevice, ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_mla_append(mk_ctx *ctx, mk_mla *m, int32_t seq, const float *k_rows, const float *v_rows, int32_t n) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && k_rows != nullptr && n >= 1, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const bool absorbed = m->layout == MK_MLA_ABSORBED;
    const size_t kb = mk_align_up((size_t)n * (absorbed ? m->nope : m->H * (m->nope + m->rope)) * 4, 256);
    const size_t vb = absorbed ? 0 : (size_t)n * m->H * m->vd * 4;
    int32_t rc = mk_io_reserve(ctx, kb + vb + 256);
    if (rc != MK_OK) return rc;
    float *dk = (float *)ctx->io_dev, *dv = (float *)((char *)ctx->io_dev + kb);
    MK_CUDA(cudaMemcpyAsync(dk, k_rows, (size_t)n * (absorbed ? m->nope : m->H * (m->nope + m->rope)) * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (!absorbed) {
        MK_CHECK_ARG(v_rows != nullptr, "v_rows is NULL");
        MK_CUDA(cudaMemcpyAsync(dv, v_rows, vb, cudaMemcpyHostToDevice, ctx->stream));
    }
    rc = mk_mla_append_dev(ctx, m, seq, dk, dv, n);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

// q rows [nq][H][qdim] on the device -> out [nq][H][vd]; sequence of row b is seq0 + b;
// npos_fixed > 0 overrides the per-sequence position counts.
static int32_t mla_attend_launch(mk_ctx *ctx, mk_mla *m, const float *q, int nq, int seq0, int npos_fixed, int max_n, float scale,
                                 float *out) {
    const int qdim = m->nope + m->rope;
    // the query's nope part -> q8_0, one row per (sequence, head) (src/model.rs:1812-1821)
    int32_t rc = mk_launch_quantize_act(ctx, q, nq * m->H, m->nope, qdim, m->q_nbp, 0, m->qq, m->qs);
    if (rc != MK_OK) return rc;
    mk_prof_scope prof(ctx, MK_PROF_MLA);
    if (m->layout == MK_MLA_ABSORBED && m->H == mla_tc::H && m->nope == mla_tc::LAT && m->vd == mla_tc::VD && !ctx->mla_no_tc) {
        // tensor-core kernel: one CTA per (sequence, KV split), 64 positions per tile
        static bool attr = false;
        if (!attr) {
            MK_CUDA(cudaFuncSetAttribute(mla_tc::mla_absorbed_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mla_tc::SM_TOTAL));
            attr = true;
        }
        const int nt64 = (max_n + mla_tc::TJ - 1) / mla_tc::TJ;
        int ns = ctx->sm_count / nq;
        if (ns > nt64) ns = nt64;
        if (ns > m->max_split) ns = m->max_split;
        if (ns < 1) ns = 1;
        mla_tc::mla_absorbed_tc_kernel<<<dim3((unsigned)ns, (unsigned)nq), mla_tc::THREADS, mla_tc::SM_TOTAL, ctx->stream>>>(
            m->vq, m->vs, m->cap, m->qq, m->qs, m->q_nbp * 32, m->q_nbp, npos_fixed > 0 ? nullptr : m->npos_dev, npos_fixed, seq0,
            scale, ns, m->part_m, m->part_l, m->part_o, out);
        ctx->launches++;
        if (ns > 1) {
            mla_merge_kernel<<<dim3((unsigned)m->H, (unsigned)nq), 128, 0, ctx->stream>>>(m->H, m->vd, ns, m->part_m, m->part_l, m->part_o, out);
            ctx->launches++;
        }
        MK_CUDA(cudaGetLastError());
        return MK_OK;
    }
    const int ntiles = (max_n + 31) / 32;
    int nsplit = (int)mk_ceil_div((int64_t)ctx->sm_count * 32, (int64_t)nq * m->H);
    if (nsplit > ntiles) nsplit = ntiles;
    if (nsplit > m->max_split) nsplit = m->max_split;
    if (nsplit < 1) nsplit = 1;
    const MlaDev c = mla_dev(m);
    const dim3 grid((unsigned)mk_ceil_div(nsplit, MLA_WARPS), (unsigned)m->H, (unsigned)nq);
    const size_t smem = (size_t)m->nope + mk_align_up((size_t)m->nb * 4, 16) + (size_t)m->rope * 4 + 16;
    const int *np = npos_fixed > 0 ? nullptr : m->npos_dev;
#define MLA_LAUNCH(VW)                                                                                                   \
    mla_attend_kernel<VW><<<grid, MLA_WARPS * 32, smem, ctx->stream>>>(c, m->qq, m->qs, m->q_nbp * 32, m->q_nbp, q, np, npos_fixed, \
                                                                       seq0, scale, nsplit, m->part_m, m->part_l, m->part_o, out)
    switch (m->vd / 128) {
    case 1: MLA_LAUNCH(1); break;
    case 2: MLA_LAUNCH(2); break;
    case 3: MLA_LAUNCH(3); break;
    default: MLA_LAUNCH(4); break;
    }
#undef MLA_LAUNCH
    ctx->launches++;
    if (nsplit > 1) {
        mla_merge_kernel<<<dim3((unsigned)m->H, (unsigned)nq), 128, 0, ctx->stream>>>(m->H, m->vd, nsplit, m->part_m, m->part_l, m->part_o, out);
        ctx->launches++;
    }
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

extern "C" int32_t mk_mla_attend(mk_ctx *ctx, mk_mla *m, int32_t seq, const float *q, int32_t pos, float scale, float *out) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && q != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(seq >= 0 && seq < m->nseq, "no such sequence");
    MK_CHECK_ARG(pos >= 0 && pos < m->npos[seq], "pos must name a position the cache holds");
    MK_CUDA(cudaSetDevice(ctx->device));
    const size_t qb = mk_align_up((size_t)m->H * (m->nope + m->rope) * 4, 256), ob = (size_t)m->H * m->vd * 4;
    int32_t rc = mk_io_reserve(ctx, qb + ob);
    if (rc != MK_OK) return rc;
    float *dq = (float *)ctx->io_dev, *dout = (float *)((char *)ctx->io_dev + qb);
    MK_CUDA(cudaMemcpyAsync(dq, q, (size_t)m->H * (m->nope + m->rope) * 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = mla_attend_launch(ctx, m, dq, 1, seq, pos + 1, pos + 1, scale, dout);
    if (rc != MK_OK) return rc;
    MK_CUDA(cudaMemcpyAsync(out, dout, ob, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_mla_attend_batch_dev(mk_ctx *ctx, mk_mla *m, const float *q, float scale, float *out) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && q != nullptr && out != nullptr, "NULL argument");
    int max_n = 0;
    for (int s = 0; s < m->nseq; ++s) {
        MK_CHECK_ARG(m->npos[s] > 0, "every sequence must hold at least one position");
        if (m->npos[s] > max_n) max_n = m->npos[s];
    }
    MK_CUDA(cudaSetDevice(ctx->device));
    return mla_attend_launch(ctx, m, q, m->nseq, 0, 0, max_n, scale, out);
}

extern "C" int32_t mk_mla_export(mk_ctx *ctx, const mk_mla *m, int32_t seq, int8_t *kq, float *ks, float *kr, int8_t *vq, float *vs) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && seq >= 0 && seq < m->nseq, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const int n = m->npos[seq];
    if (n == 0) return MK_OK;
    const bool absorbed = m->layout == MK_MLA_ABSORBED;
    const size_t kqb = (size_t)n * m->kvh * m->nope, ksb = kqb / 32 * 4, krb = (size_t)n * m->rope * 4;
    const size_t vqb = absorbed ? 0 : (size_t)n * m->kvh * m->vd, vsb = vqb / 32 * 4;
    const size_t offs[5] = {0, mk_align_up(kqb, 256), mk_align_up(kqb, 256) + mk_align_up(ksb, 256),
                            mk_align_up(kqb, 256) + mk_align_up(ksb, 256) + mk_align_up(krb, 256),
                            mk_align_up(kqb, 256) + mk_align_up(ksb, 256) + mk_align_up(krb, 256) + mk_align_up(vqb, 256)};
    void *tmp = nullptr;
    MK_CUDA(cudaMalloc(&tmp, offs[4] + mk_align_up(vsb, 256) + 256));
    char *t = (char *)tmp;
    const MlaDev c = mla_dev(m);
    const int64_t total = (int64_t)n * m->kvh * (m->nope > m->vd ? m->nope : m->vd);
    mla_export_kernel<<<(unsigned)mk_ceil_div(total, 256), 256, 0, ctx->stream>>>(
        c, seq, n, (int8_t *)(t + offs[0]), (float *)(t + offs[1]), m->rope > 0 ? (float *)(t + offs[2]) : nullptr,
        absorbed ? nullptr : (int8_t *)(t + offs[3]), absorbed ? nullptr : (float *)(t + offs[4]));
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && kq) e = cudaMemcpyAsync(kq, t + offs[0], kqb, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && ks) e = cudaMemcpyAsync(ks, t + offs[1], ksb, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && kr && krb) e = cudaMemcpyAsync(kr, t + offs[2], krb, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && vq && vqb) e = cudaMemcpyAsync(vq, t + offs[3], vqb, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess && vs && vsb) e = cudaMemcpyAsync(vs, t + offs[4], vsb, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) { mk_set_error("mk_mla_export: %s", cudaGetErrorString(e)); return MK_ERR_CUDA; }
    return MK_OK;
}
