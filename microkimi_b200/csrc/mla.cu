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
#include "mla_t5.cuh"

struct mk_mla {
    int layout, H, nope, rope, vd, cap, nseq;
    int kvh;            // kv heads: H (per-head layout) or 1 (absorbed)
    int T;              // position tiles per sequence
    int nb, nbv, NC, RC; // nope/32, vd/32, nope/16, rope/4
    int8_t *kqt; float *kst; float *krt;   // position-tiled K side
    int8_t *vq; float *vs;                 // natural V side (absorbed: the full latent row, its first vd columns are V)
    unsigned char *recs; int rec_bytes;    // per-head layout: one record per (tile, head), see MlaDev
    float *rope_scores;                    // per-head layout: [nseq][H][T*32] rope part of the scores of the current call
    int vrow;           // bytes per (position, kv head) of vq: vd (per-head) or nope (absorbed)
    int vsrow;          // scales per (position, kv head) of vs
    int *npos_dev;      // [nseq] positions held (device copy, for the batch call)
    int *npos;          // host
    // query staging and split partials
    int8_t *qq; float *qs; int64_t q_nbp;
    float *part_m, *part_l, *part_o;
    int max_split;
    int causal_nq;                         // set around a causal call (mk_mla_prefill_dev), 0 otherwise
    int64_t q_rows;                        // query rows (sequence x head) the per-call scratch buffers hold
    int64_t part_slots;                    // (query row, KV split) partial results part_m / part_l / part_o hold
};

namespace {

__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct MlaDev {
    int causal;                            // 0, or the number of query rows of a causal call: all rows belong to sequence seq0, row b sees
                                           // the positions up to that of the b-th last one (the prompt's rows appended together, attended at once)
    int H, kvh, nope, rope, vd, cap, T, nb, nbv, NC, RC, vrow, vsrow;
    int8_t *kqt; float *kst; float *krt; int8_t *vq; float *vs;
    // per-head layout: ONE contiguous record per (position tile, head) instead of the arrays above:
    //   [kq: NC chunks x 32 positions x 16 B][ks: nb x 32 f32][vq: 32 positions x vd B][vs: 32 x nbv f32]
    // so that a (tile, head) is a single bulk copy.  recs == nullptr: separate arrays (absorbed layout).
    unsigned char *recs;
    int rec_bytes, off_ks, off_vq, off_vs;
    __device__ __forceinline__ int8_t *kq_tile(int64_t th) const {
        return recs ? (int8_t *)(recs + th * rec_bytes) : kqt + th * NC * 512;
    }
    __device__ __forceinline__ float *ks_tile(int64_t th) const {
        return recs ? (float *)(recs + th * rec_bytes + off_ks) : kst + th * nb * 32;
    }
    __device__ __forceinline__ int8_t *v_row(int seq, int j, int hk) const {
        return recs ? (int8_t *)(recs + (((int64_t)seq * T + (j >> 5)) * kvh + hk) * rec_bytes + off_vq + (j & 31) * vd)
                    : vq + (((int64_t)seq * cap + j) * kvh + hk) * vrow;
    }
    __device__ __forceinline__ float *vs_row(int seq, int j, int hk) const {
        return recs ? (float *)(recs + (((int64_t)seq * T + (j >> 5)) * kvh + hk) * rec_bytes + off_vs) + (j & 31) * nbv
                    : vs + (((int64_t)seq * cap + j) * kvh + hk) * vsrow;
    }
};

// ------------------------------------------------------------------ append
// One warp per (position, kv head, block): q8::quantize_q8_into of 32 values
// (src/q8.rs:49-69), bit-exact, scattered into the layouts above.  Blocks
// [0, nb) are the K nope blocks, [nb, nb + nbv) the V blocks (per-head layout).
// Absorbed layout: the nb blocks of the latent row go to BOTH sides.
__global__ void __launch_bounds__(256)
mla_append_kernel(const MlaDev c, int seq, int pos0, int n, const float *__restrict__ k_rows, const float *__restrict__ v_rows,
                  int absorbed, const int *__restrict__ pos_dev) {
    // pos_dev: the first position comes from the device-side count of the sequence (a launch that can be
    // replayed from a CUDA graph); a full cache is reported by the bump kernel that follows, nothing is written
    if (pos_dev) { pos0 = pos_dev[seq]; if (pos0 + n > c.cap) return; }
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
        if ((lane & 3) == 0) *(uint32_t *)(c.kq_tile(th) + (ch * 32 + p) * 16 + (lane & 15)) = pk;
        if (lane == 0) c.ks_tile(th)[b * 32 + p] = dx;
    }
    if (!is_k || absorbed) {
        const int vb = absorbed ? b : b - c.nb;
        // records keep V as unsigned bytes (value + 128): the attention kernel converts them
        // to f32 without a subtraction per element
        if ((lane & 3) == 0) *(uint32_t *)(c.v_row(seq, j, h) + vb * 32 + lane) = c.recs ? (pk ^ 0x80808080u) : pk;
        if (lane == 0) c.vs_row(seq, j, h)[vb] = dx;
    }
}
// rope part of K, f32, stored once per position from head 0 (src/model.rs:1592-1593)
__global__ void mla_append_rope_kernel(const MlaDev c, int seq, int pos0, int n, const float *__restrict__ k_rows,
                                       const int *__restrict__ pos_dev) {
    if (pos_dev) { pos0 = pos_dev[seq]; if (pos0 + n > c.cap) return; }
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * c.rope) return;
    const int i = idx / c.rope, r = idx % c.rope;
    const int j = pos0 + i, tile = j >> 5, p = j & 31;
    const int hd = c.nope + c.rope;
    c.krt[((((int64_t)seq * c.T + tile) * c.RC + (r >> 2)) * 32 + p) * 4 + (r & 3)] = k_rows[(int64_t)i * c.H * hd + c.nope + r];
}
// MlaCache::to_f32 (src/model.rs:1623-1676, no Hadamard): k [n][H][nope + rope] = (kq as f32) * ks, then the shared rope row;
// v [n][H][vd] = (vq as f32) * vs.  Absorbed layout: k [n][nope] only.
__global__ void mla_export_f32_kernel(const MlaDev c, int seq, int n, float *__restrict__ k, float *__restrict__ v) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int hd = c.nope + c.rope;
    const int64_t nk = (int64_t)n * c.kvh * hd;
    if (k && idx < nk) {
        const int e = (int)(idx % hd);
        const int h = (int)((idx / hd) % c.kvh);
        const int j = (int)(idx / ((int64_t)hd * c.kvh));
        const int64_t th = ((int64_t)seq * c.T + (j >> 5)) * c.kvh + h;
        if (e < c.nope) {
            const int8_t q = c.kq_tile(th)[((e >> 4) * 32 + (j & 31)) * 16 + (e & 15)];
            k[idx] = __fmul_rn((float)q, c.ks_tile(th)[(e >> 5) * 32 + (j & 31)]);
        } else {
            const int r = e - c.nope;
            k[idx] = c.krt[((((int64_t)seq * c.T + (j >> 5)) * c.RC + (r >> 2)) * 32 + (j & 31)) * 4 + (r & 3)];
        }
    }
    const int64_t nv = (int64_t)n * c.kvh * c.vd;
    if (v && idx < nv) {
        const int e = (int)(idx % c.vd);
        const int h = (int)((idx / c.vd) % c.kvh);
        const int j = (int)(idx / ((int64_t)c.vd * c.kvh));
        const int8_t q = c.recs ? (int8_t)(c.v_row(seq, j, h)[e] ^ (int8_t)0x80) : c.v_row(seq, j, h)[e];
        v[idx] = __fmul_rn((float)q, c.vs_row(seq, j, h)[e >> 5]);
    }
}

// after an append by device position: the sequence holds n more positions (or the status word says it is full)
__global__ void mla_bump_kernel(int *__restrict__ npos, int seq, int n, int cap, int32_t *__restrict__ status) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    if (npos[seq] + n > cap) atomicCAS(status, 0, MK_ERR_STATE);
    else npos[seq] += n;
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
        if (kq) kq[idx] = c.kq_tile(th)[((e >> 4) * 32 + (j & 31)) * 16 + (e & 15)];
        if (ks && (e & 31) == 0) ks[idx / 32] = c.ks_tile(th)[(e >> 5) * 32 + (j & 31)];
    }
    if (kr && idx < (int64_t)n * c.rope) {
        const int r = (int)(idx % c.rope), j = (int)(idx / c.rope);
        kr[idx] = c.krt[((((int64_t)seq * c.T + (j >> 5)) * c.RC + (r >> 2)) * 32 + (j & 31)) * 4 + (r & 3)];
    }
    const int64_t nv = (int64_t)n * c.kvh * c.vd;
    if (vq && idx < nv) {
        const int e = (int)(idx % c.vd);
        const int hv_ = (int)((idx / c.vd) % c.kvh);
        const int jv = (int)(idx / ((int64_t)c.vd * c.kvh));
        vq[idx] = c.recs ? (int8_t)(c.v_row(seq, jv, hv_)[e] ^ (int8_t)0x80) : c.v_row(seq, jv, hv_)[e];
        if (vs && (e & 31) == 0) vs[idx / 32] = c.vs_row(seq, jv, hv_)[e >> 5];
    }
}

// ------------------------------------------------------------------ attention in the CPU's own order (parity mode)
// One warp per (sequence, head), per-head layout only.  Every sum is formed exactly as mla_attn_flash_q8_mqa forms it
// (src/model.rs:1804-1908): 64-position tiles; per position the rope dot in dot()'s 8-accumulator order
// (src/model.rs:63-82), the block terms (qs * ks) * idot added in ascending block order, s = rope + 1.0 * acc, then
// * scale; tile maximum, corr = exp(m - m_new), p_i = exp(s_i - m_new) with the tile's l summed in ascending position
// order; o *= corr, then o[d] += p_i * (vq * vs) position by position; finally o / l.  Separate multiplies and adds
// throughout, exp taken in double and rounded once.  Not a fast kernel: it exists so that a whole decode token can be
// compared with the CPU token without the attention's summation order (and, downstream of it, q8 roundings) differing.
// the sequence and the number of visible positions of query row bi (see MlaDev::causal)
__device__ __forceinline__ int mla_seq(const MlaDev &c, int seq0, int bi) { return c.causal ? seq0 : seq0 + bi; }
__device__ __forceinline__ int mla_len(const MlaDev &c, const int *npos_arr, int npos_fixed, int seq, int bi) {
    const int n = npos_arr ? npos_arr[seq] : npos_fixed;
    return c.causal ? n - (c.causal - 1 - bi) : n;
}

#define MLA_STRICT_TILE 64
__global__ void __launch_bounds__(32)
mla_attend_strict_kernel(const MlaDev c, const int8_t *__restrict__ qq, const float *__restrict__ qs, int64_t ldq, int64_t q_nbp,
                         const float *__restrict__ q_f32, const int *__restrict__ npos_arr, int npos_fixed, int seq0, float scale,
                         float *__restrict__ out) {
    extern __shared__ __align__(16) unsigned char smem_strict[];
    float *q_rope = (float *)smem_strict;                 // [rope]
    float *sc_s = q_rope + c.rope;                        // [64] scores, then p
    const int lane = threadIdx.x, h = blockIdx.x, bi = blockIdx.y, seq = mla_seq(c, seq0, bi);
    const int n = mla_len(c, npos_arr, npos_fixed, seq, bi);
    const int hd = c.nope + c.rope;
    const int64_t qrow = (int64_t)bi * c.H + h;
    for (int r = lane; r < c.rope; r += 32) q_rope[r] = q_f32[qrow * hd + c.nope + r];
    __syncwarp();
    const int8_t *qh = qq + qrow * ldq;
    const float *qsh = qs + qrow * q_nbp;
    float m = -INFINITY, l = 0.0f;
    float o[16];
    const int ncol = c.vd / 32;   // columns lane, lane + 32, ... of the head's output
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = 0.0f;
    for (int t0 = 0; t0 < n; t0 += MLA_STRICT_TILE) {
        const int tn = min(MLA_STRICT_TILE, n - t0);
        // scores: lane takes positions lane and lane + 32 of the tile
        for (int i = lane; i < tn; i += 32) {
            const int j = t0 + i, tile = j >> 5, p = j & 31;
            const int64_t th = ((int64_t)seq * c.T + tile) * c.kvh + h;
            float acc8[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) acc8[a] = 0.0f;
            const float *kr = c.krt + (((int64_t)seq * c.T + tile) * c.RC) * 128 + p * 4;
            int r = 0;
            for (; r + 8 <= c.rope; r += 8)
#pragma unroll
                for (int a = 0; a < 8; ++a) {
                    const int rr = r + a;
                    acc8[a] = __fadd_rn(acc8[a], __fmul_rn(q_rope[rr], kr[(rr >> 2) * 128 + (rr & 3)]));
                }
            float sr = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc8[0], acc8[1]), __fadd_rn(acc8[2], acc8[3])), __fadd_rn(acc8[4], acc8[5])),
                                 __fadd_rn(acc8[6], acc8[7]));
            for (; r < c.rope; ++r) sr = __fadd_rn(sr, __fmul_rn(q_rope[r], kr[(r >> 2) * 128 + (r & 3)]));
            const int8_t *kq = c.kq_tile(th);
            const float *ks = c.ks_tile(th);
            float acc = 0.0f;
            for (int g = 0; g < c.nb; ++g) {
                int d = 0;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const uint4 kv = *(const uint4 *)(kq + (((g * 2 + half) * 32 + p) * 16));
                    const uint4 qv = *(const uint4 *)(qh + g * 32 + half * 16);
                    d = dp4a_s8(kv.x, qv.x, d); d = dp4a_s8(kv.y, qv.y, d); d = dp4a_s8(kv.z, qv.z, d); d = dp4a_s8(kv.w, qv.w, d);
                }
                acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(qsh[g], ks[g * 32 + p]), (float)d));
            }
            sc_s[i] = __fmul_rn(__fadd_rn(sr, __fmul_rn(1.0f, acc)), scale);
        }
        __syncwarp();
        // tile softmax step: every lane walks the tile in order, so all lanes hold the same m, corr and l
        float tm = -INFINITY;
        for (int i = 0; i < tn; ++i) tm = fmaxf(tm, sc_s[i]);
        const float m_new = fmaxf(m, tm);
        const float corr = (float)exp((double)__fsub_rn(m, m_new));
        float tile_l = 0.0f;
        for (int i = 0; i < tn; ++i) tile_l = __fadd_rn(tile_l, (float)exp((double)__fsub_rn(sc_s[i], m_new)));
        __syncwarp();
        for (int i = lane; i < tn; i += 32) sc_s[i] = (float)exp((double)__fsub_rn(sc_s[i], m_new));
        __syncwarp();
#pragma unroll
        for (int k = 0; k < 16; ++k) if (k < ncol) o[k] = __fmul_rn(o[k], corr);
        l = __fadd_rn(__fmul_rn(l, corr), tile_l);
        m = m_new;
        for (int i = 0; i < tn; ++i) {
            const int j = t0 + i;
            const float pw = sc_s[i];
            const int8_t *vq = c.v_row(seq, j, h);
            const float *vs = c.vs_row(seq, j, h);
#pragma unroll
            for (int k = 0; k < 16; ++k)
                if (k < ncol) {
                    const int dcol = k * 32 + lane;
                    const int raw = c.recs ? (int)(uint8_t)vq[dcol] - 128 : (int)vq[dcol];   // records keep V biased by +128
                    const float v = __fmul_rn((float)raw, vs[k]);
                    o[k] = __fadd_rn(o[k], __fmul_rn(pw, v));
                }
        }
        __syncwarp();
    }
#pragma unroll
    for (int k = 0; k < 16; ++k)
        if (k < ncol) out[qrow * c.vd + k * 32 + lane] = __fdiv_rn(o[k], l);
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
    const int seq = mla_seq(c, seq0, bi);
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
    const int n = mla_len(c, npos_arr, npos_fixed, seq, bi);
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
            const uint4 *kq = (const uint4 *)c.kq_tile(th) + lane;
            const float *ks = c.ks_tile(th) + lane;
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
            for (int i = 0; i < cnt; ++i) {
                const float pi = __shfl_sync(0xFFFFFFFFu, p, i);
                const uint32_t *vw = (const uint32_t *)c.v_row(seq, tile * 32 + i, hk);
                const float *vsc = c.vs_row(seq, tile * 32 + i, hk);
#pragma unroll
                for (int w = 0; w < VW; ++w) {
                    const uint32_t word = __ldg(vw + w * 32 + lane) ^ (c.recs ? 0u : 0x80808080u); // bytes + 128
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

// ------------------------------------------------------------------ rope scores (per-head layout)
// The f32 rope row of a position is shared by all heads, so its dot with every head's
// rope query is computed once per call by this small kernel instead of once per head in
// the streaming kernel: rs[(seq_row, head)][position] = dot(q_rope[head], kr[position])
// in the 8-accumulator order of the engine's dot() (src/model.rs:63-82).
// grid = (position tiles, query rows); one CTA stages the 32 rope rows and all rope queries.
__global__ void __launch_bounds__(256)
mla_rope_scores_kernel(const MlaDev c, const float *__restrict__ q_f32, const int *__restrict__ npos_arr, int npos_fixed,
                       int seq0, float *__restrict__ rs) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tile = blockIdx.x, bi = blockIdx.y, seq = mla_seq(c, seq0, bi);
    const int n = mla_len(c, npos_arr, npos_fixed, seq, bi);
    if (tile * 32 >= n) return;
    float4 *kr_s = (float4 *)smem;                       // [RC][32]
    float4 *q_s = kr_s + c.RC * 32;                      // [H][RC]
    const int hd = c.nope + c.rope;
    const float4 *src = (const float4 *)c.krt + ((int64_t)seq * c.T + tile) * c.RC * 32;
    for (int i = threadIdx.x; i < c.RC * 32; i += blockDim.x) kr_s[i] = __ldg(src + i);
    for (int i = threadIdx.x; i < c.H * c.RC; i += blockDim.x)
        q_s[i] = *(const float4 *)(q_f32 + ((int64_t)bi * c.H + i / c.RC) * hd + c.nope + (i % c.RC) * 4);
    __syncthreads();
    const int p = threadIdx.x & 31;
    for (int h = threadIdx.x >> 5; h < c.H; h += blockDim.x >> 5) {
        float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c4 = 0; c4 < c.RC; c4 += 2) {
            const float4 k0 = kr_s[c4 * 32 + p], k1 = kr_s[(c4 + 1) * 32 + p];
            const float4 q0 = q_s[h * c.RC + c4], q1 = q_s[h * c.RC + c4 + 1];
            a8[0] = __fadd_rn(a8[0], __fmul_rn(q0.x, k0.x)); a8[1] = __fadd_rn(a8[1], __fmul_rn(q0.y, k0.y));
            a8[2] = __fadd_rn(a8[2], __fmul_rn(q0.z, k0.z)); a8[3] = __fadd_rn(a8[3], __fmul_rn(q0.w, k0.w));
            a8[4] = __fadd_rn(a8[4], __fmul_rn(q1.x, k1.x)); a8[5] = __fadd_rn(a8[5], __fmul_rn(q1.y, k1.y));
            a8[6] = __fadd_rn(a8[6], __fmul_rn(q1.z, k1.z)); a8[7] = __fadd_rn(a8[7], __fmul_rn(q1.w, k1.w));
        }
        rs[((int64_t)bi * c.H + h) * c.T * 32 + tile * 32 + p] =
            __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(a8[0], a8[1]), __fadd_rn(a8[2], a8[3])), __fadd_rn(a8[4], a8[5])),
                      __fadd_rn(a8[6], a8[7]));
    }
}

// The same with the position's rope row held in registers (RC float4 per lane) and only the queries in
// shared memory: the kernel above reads 4 shared-memory vectors per 8 multiply-adds and is bound by
// shared-memory bandwidth; here a head costs RC broadcast reads against 8 RC multiply-adds.  The 8
// accumulators and their reduction keep the engine's shape, but each term is a fused multiply-add
// (one rounding less than the engine's separate multiply and add): the attention output is compared with the
// CPU recipe by tolerance, not bit for bit, and this pre-pass is FP32-issue-bound (64 terms per position
// and head against 4 per instruction in the int8 part).
template <int RC>
__global__ void __launch_bounds__(256)
mla_rope_scores_reg_kernel(const MlaDev c, const float *__restrict__ q_f32, const int *__restrict__ npos_arr, int npos_fixed,
                           int seq0, float *__restrict__ rs) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int tile = blockIdx.x, bi = blockIdx.y, seq = mla_seq(c, seq0, bi);
    const int n = mla_len(c, npos_arr, npos_fixed, seq, bi);
    if (tile * 32 >= n) return;
    float4 *q_s = (float4 *)smem;                        // [H][RC]
    const int hd = c.nope + c.rope;
    const int p = threadIdx.x & 31;
    const float4 *src = (const float4 *)c.krt + ((int64_t)seq * c.T + tile) * RC * 32;
    float4 k[RC];
    // the rope row first: its (cold) loads travel while the queries are staged
#pragma unroll
    for (int c4 = 0; c4 < RC; ++c4) k[c4] = __ldg(src + c4 * 32 + p);
    for (int i = threadIdx.x; i < c.H * RC; i += blockDim.x)
        q_s[i] = __ldg((const float4 *)(q_f32 + ((int64_t)bi * c.H + i / RC) * hd + c.nope + (i % RC) * 4));
    __syncthreads();
    for (int h = threadIdx.x >> 5; h < c.H; h += blockDim.x >> 5) {
        float a8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int c4 = 0; c4 < RC; c4 += 2) {
            const float4 q0 = q_s[h * RC + c4], q1 = q_s[h * RC + c4 + 1];
            a8[0] = fmaf(q0.x, k[c4].x, a8[0]); a8[1] = fmaf(q0.y, k[c4].y, a8[1]);
            a8[2] = fmaf(q0.z, k[c4].z, a8[2]); a8[3] = fmaf(q0.w, k[c4].w, a8[3]);
            a8[4] = fmaf(q1.x, k[c4 + 1].x, a8[4]); a8[5] = fmaf(q1.y, k[c4 + 1].y, a8[5]);
            a8[6] = fmaf(q1.z, k[c4 + 1].z, a8[6]); a8[7] = fmaf(q1.w, k[c4 + 1].w, a8[7]);
        }
        rs[((int64_t)bi * c.H + h) * c.T * 32 + tile * 32 + p] =
            __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(a8[0], a8[1]), __fadd_rn(a8[2], a8[3])), __fadd_rn(a8[4], a8[5])),
                      __fadd_rn(a8[6], a8[7]));
    }
}

// ------------------------------------------------------------------ per-head layout, vd == 128
// One warp per (sequence, head, KV split), 8 warps (8 consecutive heads, same split) per CTA.
// The record of a (position tile, head) - 9216 contiguous bytes at the micro head dims -
// is brought into shared memory by TWO bulk async copies (cp.async.bulk, completion on an
// mbarrier each): its K half (int8 rows + scales) and its V half.  Each warp runs its own
// pipeline with one buffer per half: while phase 1 reads K(t), V(t) is in flight; while
// phase 2 reads V(t), K(t+1) is in flight - half a record per warp is always outstanding,
// 9.2 KB of shared memory per warp let 3 CTAs share an SM, and no CTA-wide barrier is
// needed.  Every mbarrier wait is bounded; on expiry the kernel records MK_ERR_TIMEOUT
// and returns.
// Phase 2 reads V with 16-byte shared loads: 8 lanes cover the 128 columns of one position,
// the 4 lane groups take 4 positions at a time, partial accumulators are summed at the end.
#define PH_WARPS 4
#define PH_WAIT_LIMIT (1 << 22)

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait: false (and the status word set) when the copy never lands
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int32_t *status) {
    for (int it = 0; it < PH_WAIT_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    atomicCAS(status, 0, MK_ERR_TIMEOUT);
    return false;
}
// global -> shared bulk copy of `bytes` (multiple of 16, both addresses 16-byte aligned), no multicast
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__global__ void __launch_bounds__(PH_WARPS * 32, 5)
mla_attend_ph128_kernel(const MlaDev c, const int8_t *__restrict__ qq, const float *__restrict__ qs, int64_t ldq, int64_t q_nbp,
                        const float *__restrict__ rope_scores, const int *__restrict__ npos_arr, int npos_fixed, int seq0,
                        float scale, int nsplit, float *__restrict__ part_m, float *__restrict__ part_l,
                        float *__restrict__ part_o, float *__restrict__ out, int32_t *__restrict__ status) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * PH_WARPS + warp, bi = blockIdx.z, seq = mla_seq(c, seq0, bi), split = blockIdx.x;
    const bool hv = h < c.H;
    const int hh = hv ? h : c.H - 1;
    // shared memory: [warp][record: K half | V half] | [warp][query staging] | [warp][2] mbarriers (K, V)
    const int rec = c.rec_bytes;
    const int qw_bytes = c.nope + ((c.nb * 4 + 15) & ~15);
    unsigned char *stage0 = smem + (size_t)warp * rec;
    unsigned char *mine = smem + (size_t)PH_WARPS * rec + (size_t)warp * qw_bytes;
    uint64_t *bars = (uint64_t *)(smem + (size_t)PH_WARPS * rec + (size_t)PH_WARPS * qw_bytes) + warp * 2;
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
    const uint32_t st0 = (uint32_t)__cvta_generic_to_shared(stage0);
    uint4 *qq_s = (uint4 *)mine;
    float *qs_s = (float *)(mine + c.nope);
    if (lane == 0) {
        mbar_init(bar0, 1);
        mbar_init(bar0 + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {
        const int64_t qrow = (int64_t)bi * c.H + hh;
        for (int i = lane; i < c.NC; i += 32) qq_s[i] = ((const uint4 *)(qq + qrow * ldq))[i];
        for (int i = lane; i < c.nb; i += 32) qs_s[i] = qs[qrow * q_nbp + i];
    }
    __syncwarp();
    const int n = mla_len(c, npos_arr, npos_fixed, seq, bi);
    const int ntiles = (n + 31) >> 5;
    const int tps = (ntiles + nsplit - 1) / nsplit;
    const int t0 = split * tps, t1 = min(t0 + tps, ntiles);
    float m = -INFINITY, l = 0.0f;
    float o[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i] = 0.0f;
    const int cg = lane & 7, pg = lane >> 3; // column group (16 columns), position subgroup
    const unsigned char *rec_base = c.recs + (((int64_t)seq * c.T) * c.kvh + hh) * rec;
    const int64_t rec_step = (int64_t)c.kvh * rec; // next tile, same head

    const uint32_t kbytes = (uint32_t)c.off_vq, vbytes = (uint32_t)(rec - c.off_vq); // K half, V half
    if (lane == 0 && t0 < t1) {
        const unsigned char *src = rec_base + (int64_t)t0 * rec_step;
        mbar_expect_tx(bar0, kbytes);
        bulk_g2s(st0, src, kbytes, bar0);
        mbar_expect_tx(bar0 + 8, vbytes);
        bulk_g2s(st0 + kbytes, src + kbytes, vbytes, bar0 + 8);
    }
    bool alive = true;
    const float *rs_row = rope_scores + ((int64_t)bi * c.H + hh) * c.T * 32;
    for (int tile = t0, it = 0; tile < t1; ++tile, ++it) {
        const float s_rope = __ldg(rs_row + tile * 32 + lane); // issued before the wait: its latency overlaps
        if (!mbar_wait_bounded(bar0, it & 1, status)) { alive = false; break; }
        const unsigned char *sb = stage0;
        const int j = tile * 32 + lane;
        const bool valid = j < n;
        // ---- phase 1: lane = position
        float acc = 0.0f;
        const uint4 *kq = (const uint4 *)sb + lane;
        const float *ks = (const float *)(sb + c.off_ks) + lane;
        for (int g = 0; g < c.nb; ++g) {
            int idot = 0;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const uint4 kw = kq[(g * 2 + cc) * 32];
                const uint4 qw = qq_s[g * 2 + cc];
                idot = dp4a_s8(kw.x, qw.x, idot);
                idot = dp4a_s8(kw.y, qw.y, idot);
                idot = dp4a_s8(kw.z, qw.z, idot);
                idot = dp4a_s8(kw.w, qw.w, idot);
            }
            acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(qs_s[g], ks[g * 32]), (float)idot));
        }
        __syncwarp(); // every lane has read the K half: refill it with the next tile's
        if (lane == 0 && tile + 1 < t1) {
            // order this warp's generic-proxy reads before the async-proxy write
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar0, kbytes);
            bulk_g2s(st0, rec_base + (int64_t)(tile + 1) * rec_step, kbytes, bar0);
        }
        float s = s_rope;
        s = __fmul_rn(__fadd_rn(s, acc), scale);
        if (!valid) s = -INFINITY;
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
        for (int i = 0; i < 16; ++i) o[i] *= corr;
        // ---- phase 2: positions past the end have p = 0 and stale-but-finite int8 bytes
        if (!mbar_wait_bounded(bar0 + 8, it & 1, status)) { alive = false; break; }
        const uint4 *vq4 = (const uint4 *)(sb + c.off_vq);
        const float *vsc = (const float *)(sb + c.off_vs);
        // A stored byte u = v + 128 placed in the low byte of a zero word IS the f32 denormal
        // u * 2^-149 (exact); with the weight pre-scaled by 2^100 one FMA per element
        // accumulates p*sc*u * 2^-49 exactly as it would p*sc*u - no int->float convert and
        // no subtraction per element.  The -128 * sum(p*sc) of the bias is removed once per tile.
        float ssum = 0.0f;
#pragma unroll
        for (int i8 = 0; i8 < 8; ++i8) {
            const int pi = i8 * 4 + pg;
            const float pv = __shfl_sync(0xFFFFFFFFu, p, pi);
            const uint4 vw = vq4[pi * 8 + cg];
            const float sc = vsc[pi * c.nbv + (cg >> 1)];
            const float ps = (pi + tile * 32 < n) ? pv * sc * 0x1p100f : 0.0f;
            ssum += ps;
            const uint32_t w4[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                o[w * 4 + 0] = fmaf(ps, __uint_as_float(w4[w] & 0xFFu), o[w * 4 + 0]);
                o[w * 4 + 1] = fmaf(ps, __uint_as_float(__byte_perm(w4[w], 0u, 0x4441)), o[w * 4 + 1]);
                o[w * 4 + 2] = fmaf(ps, __uint_as_float(__byte_perm(w4[w], 0u, 0x4442)), o[w * 4 + 2]);
                o[w * 4 + 3] = fmaf(ps, __uint_as_float(w4[w] >> 24), o[w * 4 + 3]);
            }
        }
        {
            const float bias = ssum * 0x1p-142f; // 128 * 2^-149 per unit of the pre-scaled weight
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] -= bias;
        }
        __syncwarp(); // every lane has read the V half: refill it with the next tile's
        if (lane == 0 && tile + 1 < t1) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect_tx(bar0 + 8, vbytes);
            bulk_g2s(st0 + kbytes, rec_base + (int64_t)(tile + 1) * rec_step + kbytes, vbytes, bar0 + 8);
        }
    }
    if (!alive) {
        // a copy never landed: give any copy still in flight a bounded chance to finish, then leave
        for (int k = 0; k < 2; ++k)
            for (int itw = 0; itw < (1 << 16); ++itw)
                if (mbar_try_wait(bar0 + 8 * k, 0) || mbar_try_wait(bar0 + 8 * k, 1)) break;
        return;
    }
    // sum the 4 position subgroups (fixed order), undo the 2^-49 of the denormal trick;
    // lanes 0..7 then hold 16 columns each
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float v = o[i];
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 8);
        v += __shfl_xor_sync(0xFFFFFFFFu, v, 16);
        o[i] = v * 0x1p49f;
    }
    if (!hv || pg != 0) return;
    if (nsplit == 1) {
        float *dst = out + ((int64_t)bi * c.H + h) * c.vd + cg * 16;
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = __fdiv_rn(o[i], l);
    } else {
        const int64_t pi = ((int64_t)bi * c.H + h) * nsplit + split;
        if (cg == 0) { part_m[pi] = m; part_l[pi] = l; }
        float4 *dst = (float4 *)(part_o + pi * c.vd + cg * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_float4(o[i * 4], o[i * 4 + 1], o[i * 4 + 2], o[i * 4 + 3]);
    }
}

// log-sum-exp merge of the split partials: grid (H, nseq, column chunks of 128), one thread per column;
// the split weights exp(m_s - M) / L are formed once per CTA in shared memory (nsplit <= 1024)
__global__ void __launch_bounds__(128) mla_merge_kernel(int H, int vd, int nsplit, const float *__restrict__ part_m,
                                                        const float *__restrict__ part_l, const float *__restrict__ part_o,
                                                        float *__restrict__ out) {
    __shared__ float wgt[1024];
    __shared__ float red[4];
    const int64_t bh = (int64_t)blockIdx.y * H + blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float M = -INFINITY;
    for (int s = tid; s < nsplit; s += 128) M = fmaxf(M, part_m[bh * nsplit + s]);
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
    if (lane == 0) red[warp] = M;
    __syncthreads();
    M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float L = 0.0f;
    for (int s = tid; s < nsplit; s += 128) {
        const float ms = part_m[bh * nsplit + s];
        const float w = ms != -INFINITY ? expf(ms - M) : 0.0f;
        wgt[s] = w;
        L += part_l[bh * nsplit + s] * w;
    }
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xFFFFFFFFu, L, o);
    if (lane == 0) red[warp] = L;
    __syncthreads();
    L = (red[0] + red[1]) + (red[2] + red[3]);
    const int col = blockIdx.z * 128 + tid;
    if (col >= vd) return;
    float acc0 = 0.0f, acc1 = 0.0f;
    const float *po = part_o + bh * nsplit * vd + col;
    int s = 0;
    // 16 independent loads in flight per thread (with the splits of a long context - 148 at 65536 positions - a loop of
    // dependent round trips to L2 took longer than the attention itself); the sums keep their order: even splits into
    // acc0, odd ones into acc1, ascending
    for (; s + 16 <= nsplit; s += 16) {
        float w[16], v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            w[u] = wgt[s + u];
            v[u] = w[u] != 0.0f ? __ldcg(po + (int64_t)(s + u) * vd) : 0.0f;       // an empty split's partial is never read
        }
#pragma unroll
        for (int u = 0; u < 16; u += 2) {
            if (w[u] != 0.0f) acc0 += v[u] * w[u];
            if (w[u + 1] != 0.0f) acc1 += v[u + 1] * w[u + 1];
        }
    }
    for (; s + 1 < nsplit; s += 2) {
        const float w0 = wgt[s], w1 = wgt[s + 1];
        if (w0 != 0.0f) acc0 += po[(int64_t)s * vd] * w0;       // an empty split's partial is never read
        if (w1 != 0.0f) acc1 += po[(int64_t)(s + 1) * vd] * w1;
    }
    if (s < nsplit && wgt[s] != 0.0f) acc0 += po[(int64_t)s * vd] * wgt[s];
    out[bh * vd + col] = (acc0 + acc1) / L;
}

} // namespace

// ====================================================================== host side
#include <algorithm>
#include <new>

static MlaDev mla_dev(const mk_mla *m) {
    MlaDev c;
    c.H = m->H; c.kvh = m->kvh; c.nope = m->nope; c.rope = m->rope; c.vd = m->vd; c.cap = m->cap; c.T = m->T;
    c.nb = m->nb; c.nbv = m->nbv; c.NC = m->NC; c.RC = m->RC; c.vrow = m->vrow; c.vsrow = m->vsrow;
    c.kqt = m->kqt; c.kst = m->kst; c.krt = m->krt; c.vq = m->vq; c.vs = m->vs;
    c.recs = m->recs; c.rec_bytes = m->rec_bytes;
    c.causal = m->causal_nq;
    c.off_ks = m->nope * 32; c.off_vq = c.off_ks + m->nb * 128; c.off_vs = c.off_vq + m->vd * 32;
    return c;
}

extern "C" int32_t mk_mla_free(mk_ctx *ctx, mk_mla *m) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr, "NULL argument");
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    void *ptrs[] = {m->kqt, m->kst, m->krt, m->vq, m->vs, m->recs, m->rope_scores, m->npos_dev, m->qq, m->qs, m->part_m, m->part_l, m->part_o};
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
    const size_t bh = (size_t)m->nseq * m->H;
    const size_t tiles = (size_t)m->nseq * m->T * m->kvh;
    const size_t rows = (size_t)m->nseq * m->cap * m->kvh;
    cudaError_t e = m->npos ? cudaSuccess : cudaErrorMemoryAllocation;
    const bool absorbed_l = d->layout == MK_MLA_ABSORBED;
    m->rec_bytes = m->nope * 32 + m->nb * 128 + m->vd * 32 + m->nbv * 128;
    if (e == cudaSuccess && !absorbed_l) e = cudaMalloc((void **)&m->recs, tiles * (size_t)m->rec_bytes);
    if (e == cudaSuccess && !absorbed_l) e = cudaMemsetAsync(m->recs, 0, tiles * (size_t)m->rec_bytes, ctx->stream);
    if (e == cudaSuccess && !absorbed_l) e = cudaMalloc(&m->rope_scores, bh * (size_t)m->T * 32 * 4);
    if (e == cudaSuccess && absorbed_l) e = cudaMalloc(&m->kqt, tiles * m->nope * 32);
    if (e == cudaSuccess && absorbed_l) e = cudaMalloc(&m->kst, tiles * m->nb * 32 * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->krt, (size_t)m->nseq * m->T * (m->rope > 0 ? m->rope : 4) * 32 * 4);
    if (e == cudaSuccess && absorbed_l) e = cudaMalloc(&m->vq, rows * m->vrow);
    if (e == cudaSuccess && absorbed_l) e = cudaMalloc(&m->vs, rows * m->vsrow * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->npos_dev, (size_t)m->nseq * 4);
    if (e == cudaSuccess) e = cudaMemsetAsync(m->npos_dev, 0, (size_t)m->nseq * 4, ctx->stream);
    if (e == cudaSuccess) e = cudaMalloc(&m->qq, bh * m->q_nbp * 32);
    if (e == cudaSuccess) e = cudaMalloc(&m->qs, bh * m->q_nbp * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->part_m, bh * m->max_split * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->part_l, bh * m->max_split * 4);
    if (e == cudaSuccess) e = cudaMalloc(&m->part_o, bh * m->max_split * m->vd * 4);
    m->q_rows = (int64_t)bh;
    m->part_slots = (int64_t)bh * m->max_split;
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
    mla_append_kernel<<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(c, seq, m->npos[seq], n, k_rows, v_rows, absorbed ? 1 : 0, nullptr);
    ctx->launches++;
    if (m->rope > 0) {
        mla_append_rope_kernel<<<(unsigned)mk_ceil_div((int64_t)n * m->rope, 128), 128, 0, ctx->stream>>>(c, seq, m->npos[seq], n, k_rows, nullptr);
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
    if (ctx->mla_strict && m->layout == MK_MLA_PER_HEAD && m->vd <= 512) {
        const MlaDev cs = mla_dev(m);
        mla_attend_strict_kernel<<<dim3((unsigned)m->H, (unsigned)nq), 32, (size_t)(m->rope + MLA_STRICT_TILE) * 4 + 16, ctx->stream>>>(
            cs, m->qq, m->qs, m->q_nbp * 32, m->q_nbp, q, npos_fixed > 0 ? nullptr : m->npos_dev, npos_fixed, seq0, scale, out);
        ctx->launches++;
        MK_CUDA(cudaGetLastError());
        return MK_OK;
    }
    if (m->layout == MK_MLA_ABSORBED && m->H == mla_t5::H && m->nope == mla_t5::LAT && m->vd == mla_t5::VD && !ctx->mla_no_tc &&
        !ctx->mla_no_t5) {
        // tcgen05 kernel: one CTA per (sequence, KV split), 128 positions per tile, accumulators in tensor memory
        static mk_once_per_device attr5;
        if (attr5.pending(ctx->device)) {
            MK_CUDA(cudaFuncSetAttribute(mla_t5::mla_absorbed_t5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mla_t5::SM_TOTAL));
            attr5.mark(ctx->device);
        }
        const int nt128 = (max_n + mla_t5::TJ - 1) / mla_t5::TJ;
        int ns = ctx->sm_count / nq;
        if (ns > nt128) ns = nt128;
        if (ns > m->max_split) ns = m->max_split;
        if (ctx->mla_max_split > 0 && ns > ctx->mla_max_split) ns = ctx->mla_max_split;
        if (ns < 1) ns = 1;
        mla_t5::mla_absorbed_t5_kernel<<<dim3((unsigned)ns, (unsigned)nq), mla_t5::THREADS, mla_t5::SM_TOTAL, ctx->stream>>>(
            m->vq, m->vs, m->cap, m->qq, m->qs, m->q_nbp * 32, m->q_nbp, npos_fixed > 0 ? nullptr : m->npos_dev, npos_fixed, seq0,
            scale, ns, m->part_m, m->part_l, m->part_o, out, ctx->status_dev);
        ctx->launches++;
        if (ns > 1) {
            mla_merge_kernel<<<dim3((unsigned)m->H, (unsigned)nq, (unsigned)mk_ceil_div(m->vd, 128)), 128, 0, ctx->stream>>>(m->H, m->vd, ns, m->part_m, m->part_l, m->part_o, out);
            ctx->launches++;
        }
        MK_CUDA(cudaGetLastError());
        return MK_OK;
    }
    if (m->layout == MK_MLA_ABSORBED && m->H == mla_tc::H && m->nope == mla_tc::LAT && m->vd == mla_tc::VD && !ctx->mla_no_tc) {
        // mma.sync tensor-core kernel: one CTA per (sequence, KV split), 64 positions per tile
        static mk_once_per_device attr;
        if (attr.pending(ctx->device)) {
            MK_CUDA(cudaFuncSetAttribute(mla_tc::mla_absorbed_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, mla_tc::SM_TOTAL));
            attr.mark(ctx->device);
        }
        const int nt64 = (max_n + mla_tc::TJ - 1) / mla_tc::TJ;
        int ns = ctx->sm_count / nq;
        if (ns > nt64) ns = nt64;
        if (ns > m->max_split) ns = m->max_split;
        if (ctx->mla_max_split > 0 && ns > ctx->mla_max_split) ns = ctx->mla_max_split;
        if (ns < 1) ns = 1;
        mla_tc::mla_absorbed_tc_kernel<<<dim3((unsigned)ns, (unsigned)nq), mla_tc::THREADS, mla_tc::SM_TOTAL, ctx->stream>>>(
            m->vq, m->vs, m->cap, m->qq, m->qs, m->q_nbp * 32, m->q_nbp, npos_fixed > 0 ? nullptr : m->npos_dev, npos_fixed, seq0,
            scale, ns, m->part_m, m->part_l, m->part_o, out);
        ctx->launches++;
        if (ns > 1) {
            mla_merge_kernel<<<dim3((unsigned)m->H, (unsigned)nq, (unsigned)mk_ceil_div(m->vd, 128)), 128, 0, ctx->stream>>>(m->H, m->vd, ns, m->part_m, m->part_l, m->part_o, out);
            ctx->launches++;
        }
        MK_CUDA(cudaGetLastError());
        return MK_OK;
    }
    if (m->layout == MK_MLA_PER_HEAD && m->vd == 128 && m->rope > 0 && !ctx->mla_no_tc &&
        (size_t)PH_WARPS * m->rec_bytes + PH_WARPS * ((size_t)m->nope + m->nb * 4 + 16 + (size_t)m->rope * 4) + 256 <= 220 * 1024) {
        const int ntiles_p = (max_n + 31) / 32;
        const int hgroups = (int)mk_ceil_div(m->H, PH_WARPS);
        int ns = (int)mk_ceil_div((int64_t)ctx->sm_count * 10, (int64_t)nq * hgroups);
        if (ns > ntiles_p) ns = ntiles_p;
        if (ns > m->max_split) ns = m->max_split;
        if (ctx->mla_max_split > 0 && ns > ctx->mla_max_split) ns = ctx->mla_max_split;
        if ((int64_t)ns * nq * m->H > m->part_slots) ns = (int)(m->part_slots / ((int64_t)nq * m->H));
        if (ns < 1) ns = 1;
        const MlaDev cph = mla_dev(m);
        const size_t qw = (size_t)m->nope + mk_align_up((size_t)m->nb * 4, 16);
        const size_t smem_ph = (size_t)PH_WARPS * m->rec_bytes + PH_WARPS * qw + PH_WARPS * 2 * 8 + 128;
        {
            if (m->RC == 16 && (size_t)m->H * 256 <= 48 * 1024) {
                // rope 64: the position's rope row lives in registers
                mla_rope_scores_reg_kernel<16><<<dim3((unsigned)ntiles_p, (unsigned)nq), 256, (size_t)m->H * 16 * 16, ctx->stream>>>(
                    cph, q, npos_fixed > 0 ? nullptr : m->npos_dev, npos_fixed, seq0, m->rope_scores);
            } else {
                const size_t smem_rs = ((size_t)m->RC * 32 + (size_t)m->H * m->RC) * 16;
                static mk_once_per_device attr_rs;
                if (attr_rs.pending(ctx->device)) { MK_CUDA(cudaFuncSetAttribute(mla_rope_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); attr_rs.mark(ctx->device); }
                MK_CHECK_ARG(smem_rs <= 200 * 1024, "rope dims too large");
                mla_rope_scores_kernel<<<dim3((unsigned)ntiles_p, (unsigned)nq), 256, smem_rs, ctx->stream>>>(
                    cph, q, npos_fixed > 0 ? nullptr : m->npos_dev, npos_fixed, seq0, m->rope_scores);
            }
            ctx->launches++;
        }
        static mk_once_per_device attr_ph;
        if (attr_ph.pending(ctx->device)) { MK_CUDA(cudaFuncSetAttribute(mla_attend_ph128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)); attr_ph.mark(ctx->device); }
        mla_attend_ph128_kernel<<<dim3((unsigned)ns, (unsigned)hgroups, (unsigned)nq), PH_WARPS * 32, smem_ph, ctx->stream>>>(
            cph, m->qq, m->qs, m->q_nbp * 32, m->q_nbp, m->rope_scores, npos_fixed > 0 ? nullptr : m->npos_dev, npos_fixed, seq0, scale, ns,
            m->part_m, m->part_l, m->part_o, out, ctx->status_dev);
        ctx->launches++;
        if (ns > 1) {
            mla_merge_kernel<<<dim3((unsigned)m->H, (unsigned)nq, (unsigned)mk_ceil_div(m->vd, 128)), 128, 0, ctx->stream>>>(m->H, m->vd, ns, m->part_m, m->part_l, m->part_o, out);
            ctx->launches++;
        }
        MK_CUDA(cudaGetLastError());
        return MK_OK;
    }
    const int ntiles = (max_n + 31) / 32;
    int nsplit = (int)mk_ceil_div((int64_t)ctx->sm_count * 32, (int64_t)nq * m->H);
    if (nsplit > ntiles) nsplit = ntiles;
    if (nsplit > m->max_split) nsplit = m->max_split;
    if (ctx->mla_max_split > 0 && nsplit > ctx->mla_max_split) nsplit = ctx->mla_max_split;
    if ((int64_t)nsplit * nq * m->H > m->part_slots) nsplit = (int)(m->part_slots / ((int64_t)nq * m->H));
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
        mla_merge_kernel<<<dim3((unsigned)m->H, (unsigned)nq, (unsigned)mk_ceil_div(m->vd, 128)), 128, 0, ctx->stream>>>(m->H, m->vd, nsplit, m->part_m, m->part_l, m->part_o, out);
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

extern "C" int32_t mk_mla_export_f32(mk_ctx *ctx, const mk_mla *m, int32_t seq, float *k, float *v) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && seq >= 0 && seq < m->nseq, "bad argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    const int n = m->npos[seq];
    if (n == 0) return MK_OK;
    const bool absorbed = m->layout == MK_MLA_ABSORBED;
    const size_t kb = (size_t)n * m->kvh * (m->nope + m->rope) * 4, vb = absorbed ? 0 : (size_t)n * m->kvh * m->vd * 4;
    int32_t rc = mk_io_reserve(ctx, mk_align_up(kb, 256) + vb + 256);
    if (rc != MK_OK) return rc;
    float *dk = (float *)ctx->io_dev, *dv = (float *)((char *)ctx->io_dev + mk_align_up(kb, 256));
    const MlaDev c = mla_dev(m);
    const int64_t total = (int64_t)n * m->kvh * (m->nope + m->rope > m->vd ? m->nope + m->rope : m->vd);
    mla_export_f32_kernel<<<(unsigned)mk_ceil_div(total, 256), 256, 0, ctx->stream>>>(c, seq, n, k ? dk : nullptr, (v && !absorbed) ? dv : nullptr);
    ctx->launches++;
    MK_CUDA(cudaGetLastError());
    if (k) MK_CUDA(cudaMemcpyAsync(k, dk, kb, cudaMemcpyDeviceToHost, ctx->stream));
    if (v && !absorbed) MK_CUDA(cudaMemcpyAsync(v, dv, vb, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}
// MlaCache::assign_f32 (src/model.rs:1678-1692): the sequence is emptied and the rows are pushed again (requantized)
extern "C" int32_t mk_mla_import_f32(mk_ctx *ctx, mk_mla *m, int32_t seq, const float *k, const float *v, int32_t n) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && seq >= 0 && seq < m->nseq && k != nullptr && n >= 0, "bad argument");
    MK_CHECK_ARG(n <= m->cap, "more positions than the cache holds");
    int32_t rc = mk_mla_reset(ctx, m, seq);
    if (rc != MK_OK || n == 0) return rc;
    const bool absorbed = m->layout == MK_MLA_ABSORBED;
    const int64_t krow = absorbed ? m->nope : (int64_t)m->H * (m->nope + m->rope), vrow = (int64_t)m->H * m->vd;
    for (int j0 = 0; j0 < n; j0 += 4096) {      // bounded staging
        const int nn = n - j0 < 4096 ? n - j0 : 4096;
        rc = mk_mla_append(ctx, m, seq, k + (int64_t)j0 * krow, absorbed ? nullptr : v + (int64_t)j0 * vrow, nn);
        if (rc != MK_OK) return rc;
    }
    return MK_OK;
}

// One decode step of one sequence whose launches do not depend on the position: append by the device-side
// count, bump the count, attend over everything held with grids sized for the cache's capacity.
extern "C" int32_t mk_mla_decode_step_dev(mk_ctx *ctx, mk_mla *m, int32_t seq, const float *k_row, const float *v_row, const float *q,
                                          float scale, float *out) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && k_row != nullptr && q != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(seq >= 0 && seq < m->nseq, "no such sequence");
    const bool absorbed = m->layout == MK_MLA_ABSORBED;
    MK_CHECK_ARG(absorbed || v_row != nullptr, "v_row is NULL");
    if (m->npos[seq] + 1 > m->cap) {
        mk_set_error("mk_mla_decode_step_dev: sequence %d already holds %d of %d positions", seq, m->npos[seq], m->cap);
        return MK_ERR_STATE;
    }
    MK_CUDA(cudaSetDevice(ctx->device));
    const MlaDev c = mla_dev(m);
    {
        mk_prof_scope prof(ctx, MK_PROF_MLA);
        const int nblk = absorbed ? m->nb : m->nb + m->nbv;
        const int64_t warps = (int64_t)m->kvh * nblk;
        mla_append_kernel<<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(c, seq, 0, 1, k_row, v_row, absorbed ? 1 : 0, m->npos_dev);
        ctx->launches++;
        if (m->rope > 0) {
            mla_append_rope_kernel<<<(unsigned)mk_ceil_div((int64_t)m->rope, 128), 128, 0, ctx->stream>>>(c, seq, 0, 1, k_row, m->npos_dev);
            ctx->launches++;
        }
        mla_bump_kernel<<<1, 32, 0, ctx->stream>>>(m->npos_dev, seq, 1, m->cap, ctx->status_dev);
        ctx->launches++;
        MK_CUDA(cudaGetLastError());
    }
    m->npos[seq] += 1;
    return mla_attend_launch(ctx, m, q, 1, seq, 0, m->cap, scale, out);
}
// Scratch of the attention calls (quantized queries, rope scores, split partials) for `rows` query rows (row = sequence x
// head, or prompt position x head in a causal call) with up to 32 KV splits each; grows, never shrinks.
static int32_t mla_reserve_rows(mk_ctx *ctx, mk_mla *m, int64_t rows) {
    if (rows <= m->q_rows && rows * 32 <= m->part_slots) return MK_OK;
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    ctx->alloc_epoch++;         // recorded decode steps point into the old buffers: their holder re-records
    const int64_t r = std::max(rows, m->q_rows), slots = std::max(rows * 32, m->part_slots);
    void **bufs[] = {(void **)&m->rope_scores, (void **)&m->qq, (void **)&m->qs, (void **)&m->part_m, (void **)&m->part_l, (void **)&m->part_o};
    const size_t sizes[] = {m->layout == MK_MLA_ABSORBED ? 0 : (size_t)r * m->T * 32 * 4, (size_t)r * m->q_nbp * 32, (size_t)r * m->q_nbp * 4,
                            (size_t)slots * 4, (size_t)slots * 4, (size_t)slots * m->vd * 4};
    for (int i = 0; i < 6; ++i) {
        if (*bufs[i]) { cudaFree(*bufs[i]); *bufs[i] = nullptr; }
        if (sizes[i]) MK_CUDA(cudaMalloc(bufs[i], sizes[i]));
    }
    m->q_rows = r;
    m->part_slots = slots;
    return MK_OK;
}

// A run of n consecutive positions of one sequence in one go (the attention part of mla_prefill, src/model.rs:2033-2115):
// the n rows are appended at the device-side count, then query row b attends to everything up to its own position - the
// same arithmetic per (row, head) as n calls of mk_mla_decode_step_dev (in the strict mode the same bits: one warp walks
// a row's positions in order), with the launches shared.  The absorbed layout takes the steps one by one.
extern "C" int32_t mk_mla_prefill_dev(mk_ctx *ctx, mk_mla *m, int32_t seq, const float *k_rows, const float *v_rows, const float *q_rows, int32_t n,
                                      float scale, float *out) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && k_rows != nullptr && q_rows != nullptr && out != nullptr && n >= 1, "bad argument");
    MK_CHECK_ARG(seq >= 0 && seq < m->nseq, "no such sequence");
    const bool absorbed = m->layout == MK_MLA_ABSORBED;
    MK_CHECK_ARG(absorbed || v_rows != nullptr, "v_rows is NULL");
    if (m->npos[seq] + n > m->cap) {
        mk_set_error("mk_mla_prefill_dev: sequence %d holds %d of %d positions, %d more do not fit", seq, m->npos[seq], m->cap, n);
        return MK_ERR_STATE;
    }
    const int64_t qrow = (int64_t)m->H * (m->nope + m->rope), krow = absorbed ? m->nope : qrow, vrow = (int64_t)m->H * m->vd;
    if (absorbed || n == 1) {
        for (int t = 0; t < n; ++t) {
            int32_t rc = mk_mla_decode_step_dev(ctx, m, seq, k_rows + t * krow, absorbed ? nullptr : v_rows + t * vrow, q_rows + t * qrow, scale,
                                                out + t * vrow);
            if (rc != MK_OK) return rc;
        }
        return MK_OK;
    }
    MK_CUDA(cudaSetDevice(ctx->device));
    int32_t rc = mla_reserve_rows(ctx, m, (int64_t)n * m->H);
    if (rc != MK_OK) return rc;
    const MlaDev c = mla_dev(m);
    {
        mk_prof_scope prof(ctx, MK_PROF_MLA);
        const int64_t warps = (int64_t)n * m->kvh * (m->nb + m->nbv);
        mla_append_kernel<<<(unsigned)mk_ceil_div(warps * 32, 256), 256, 0, ctx->stream>>>(c, seq, 0, n, k_rows, v_rows, 0, m->npos_dev);
        ctx->launches++;
        if (m->rope > 0) {
            mla_append_rope_kernel<<<(unsigned)mk_ceil_div((int64_t)n * m->rope, 128), 128, 0, ctx->stream>>>(c, seq, 0, n, k_rows, m->npos_dev);
            ctx->launches++;
        }
        mla_bump_kernel<<<1, 32, 0, ctx->stream>>>(m->npos_dev, seq, n, m->cap, ctx->status_dev);
        ctx->launches++;
        MK_CUDA(cudaGetLastError());
    }
    m->npos[seq] += n;
    m->causal_nq = n;
    rc = mla_attend_launch(ctx, m, q_rows, n, seq, 0, m->npos[seq], scale, out);
    m->causal_nq = 0;
    return rc;
}

// The host-side count of a sequence follows a replayed step (the device-side count moved inside the graph).
void mk_mla_note_replay(mk_mla *m, int seq) { if (m && seq >= 0 && seq < m->nseq && m->npos[seq] < m->cap) m->npos[seq] += 1; }

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

