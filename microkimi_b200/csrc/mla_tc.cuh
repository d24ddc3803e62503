// Absorbed-layout MLA decode attention on the tensor cores (sm_100a).
//
// 64 heads attend to ONE shared q8_0 latent row per position (576 = 512 + 64 wide,
// V = its first 512 columns): 139 kFLOP per 648-byte row, far above what CUDA
// cores sustain, so the contraction runs as f16 x f16 -> f32 MMAs:
//   * a tile of 64 positions is read once from HBM (natural layout, one contiguous
//     36,864 + 4,608 byte run), dequantized (int8 * f32 block scale, rounded once to
//     f16) into shared memory and used twice: as K for S = Q K^T and as V for O += P V;
//   * Q (the q8_0-quantized query of the reference recipe, dequantized and rounded
//     once to f16) sits in shared memory for the whole kernel;
//   * online softmax per head over 64-position tiles (src/model.rs:1854-1870),
//     split-KV over CTAs with the log-sum-exp merge kernel of mla.cu.
// Against the reference recipe (exact int32 block dots, f32 scaling) the operands
// carry one f16 rounding each (2^-11 relative); products and sums are f32.
// CTA = 16 warps: warp (hr, wq) owns heads [16 hr, 16 hr + 16); in the S phase it
// scores positions [16 wq, 16 wq + 16) of the tile, in the PV phase it owns output
// columns [128 wq, 128 wq + 128).
#pragma once
#include <cuda_fp16.h>

#include "mk_common.cuh"

namespace mla_tc {

constexpr int H = 64, LAT = 576, VD = 512, NBLK = 18, TJ = 64;
constexpr int ROWB = LAT * 2 + 16;        // padded f16 row: 1168 B = 73 x 16 B (odd -> conflict-free ldmatrix)
constexpr int PROWB = TJ * 2 + 16;        // padded P row: 144 B
constexpr int SM_Q = 0, SM_K = SM_Q + H * ROWB, SM_P = SM_K + TJ * ROWB, SM_MAX = SM_P + H * PROWB,
              SM_SUM = SM_MAX + H * 4 * 4, SM_TOTAL = SM_SUM + H * 4 * 4;
constexpr int THREADS = 512;
constexpr int UNITS = TJ * (LAT / 8) / THREADS; // 8-byte units of a tile per thread = 9

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 8 int8 values (two words) times one f32 scale -> 8 f16 (one rounding each)
__device__ __forceinline__ uint4 dequant8(uint2 w, float s) {
    const uint32_t x0 = w.x ^ 0x80808080u, x1 = w.y ^ 0x80808080u; // bytes + 128
    // 0x64uu as f16 is 1024 + uu: exact integers, then -1152 gives the int8 value exactly
    const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
    __half2 h[4];
    uint32_t m;
    m = __byte_perm(x0, 0x64646464u, 0x4140); h[0] = __hsub2(*(__half2 *)&m, off);
    m = __byte_perm(x0, 0x64646464u, 0x4342); h[1] = __hsub2(*(__half2 *)&m, off);
    m = __byte_perm(x1, 0x64646464u, 0x4140); h[2] = __hsub2(*(__half2 *)&m, off);
    m = __byte_perm(x1, 0x64646464u, 0x4342); h[3] = __hsub2(*(__half2 *)&m, off);
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        const __half2 r = __floats2half2_rn(f.x * s, f.y * s);
        o[i] = *(const uint32_t *)&r;
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void __launch_bounds__(THREADS, 1)
mla_absorbed_tc_kernel(const int8_t *__restrict__ vq, const float *__restrict__ vs, int cap, const int8_t *__restrict__ qq,
                       const float *__restrict__ qs, int64_t ldq, int64_t q_nbp, const int *__restrict__ npos_arr,
                       int npos_fixed, int seq0, float scale, int nsplit, float *__restrict__ part_m,
                       float *__restrict__ part_l, float *__restrict__ part_o, float *__restrict__ out) {
    extern __shared__ __align__(16) unsigned char sm[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int hr = warp & 3, wq = warp >> 2;
    const int bi = blockIdx.y, seq = seq0 + bi, split = blockIdx.x;
    const uint32_t sm_base = (uint32_t)__cvta_generic_to_shared(sm);
    float *red_max = (float *)(sm + SM_MAX), *red_sum = (float *)(sm + SM_SUM);

    const int n = npos_arr ? npos_arr[seq] : npos_fixed;
    const int ntiles = (n + TJ - 1) / TJ;
    const int tps = (ntiles + nsplit - 1) / nsplit;
    const int t0 = split * tps, t1 = min(t0 + tps, ntiles);

    // ---- Q: q8 rows (quantized by the activation quantizer) -> f16 in shared memory
    for (int u = tid; u < H * (LAT / 8); u += THREADS) {
        const int h = u / (LAT / 8), c8 = u % (LAT / 8);
        const int64_t row = (int64_t)bi * H + h;
        const uint2 w = *(const uint2 *)(qq + row * ldq + c8 * 8);
        const float s = qs[row * q_nbp + (c8 >> 2)];
        *(uint4 *)(sm + SM_Q + h * ROWB + c8 * 16) = dequant8(w, s);
    }

    const int8_t *vbase = vq + (int64_t)seq * cap * LAT;
    const float *sbase = vs + (int64_t)seq * cap * NBLK;
    uint2 raw[UNITS];
    float rsc[UNITS];
    auto load_raw = [&](int tile) {
#pragma unroll
        for (int i = 0; i < UNITS; ++i) {
            const int u = tid + i * THREADS;
            const int p = u / (LAT / 8), c8 = u % (LAT / 8);
            const int j = tile * TJ + p;
            if (j < n) {
                raw[i] = __ldg((const uint2 *)(vbase + (int64_t)j * LAT + c8 * 8));
                rsc[i] = __ldg(sbase + (int64_t)j * NBLK + (c8 >> 2));
            } else {
                raw[i] = make_uint2(0u, 0u);
                rsc[i] = 0.0f;
            }
        }
    };

    float acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    const int row0 = hr * 16 + g, row1 = row0 + 8;

    if (t0 < t1) load_raw(t0);
    for (int tile = t0; tile < t1; ++tile) {
        __syncthreads(); // the previous tile's PV phase has finished reading K and P
#pragma unroll
        for (int i = 0; i < UNITS; ++i) {
            const int u = tid + i * THREADS;
            const int p = u / (LAT / 8), c8 = u % (LAT / 8);
            // rows past the end were loaded as zeros: 0 * 0 = 0, never a NaN from stale memory
            *(uint4 *)(sm + SM_K + p * ROWB + c8 * 16) = dequant8(raw[i], rsc[i]);
        }
        if (tile + 1 < t1) load_raw(tile + 1);
        __syncthreads();

        // ---- S = Q K^T for heads [16hr, +16) x positions [16wq, +16)
        float s[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
        {
            const uint32_t a_addr = sm_base + SM_Q + (hr * 16 + (lane & 15)) * ROWB + (lane >> 4) * 16;
            const uint32_t b_addr = sm_base + SM_K + (wq * 16 + (lane & 7) + (lane >> 4) * 8) * ROWB + ((lane >> 3) & 1) * 16;
#pragma unroll 4
            for (int ks = 0; ks < LAT / 16; ++ks) {
                uint32_t a[4], b[4];
                ldmatrix_x4(a, a_addr + ks * 32);
                ldmatrix_x4(b, b_addr + ks * 32);
                mma_f16(s[0], a, b[0], b[1]);
                mma_f16(s[1], a, b[2], b[3]);
            }
        }
        // scale, mask, tile maximum per head row
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int j0 = tile * TJ + wq * 16 + nt * 8 + 2 * t;
            s[nt][0] = j0 < n ? s[nt][0] * scale : -INFINITY;
            s[nt][1] = j0 + 1 < n ? s[nt][1] * scale : -INFINITY;
            s[nt][2] = j0 < n ? s[nt][2] * scale : -INFINITY;
            s[nt][3] = j0 + 1 < n ? s[nt][3] * scale : -INFINITY;
            mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
        if (t == 0) { red_max[row0 * 4 + wq] = mx0; red_max[row1 * 4 + wq] = mx1; }
        __syncthreads();
        const float4 rm0 = *(const float4 *)(red_max + row0 * 4), rm1 = *(const float4 *)(red_max + row1 * 4);
        const float mn0 = fmaxf(m_run[0], fmaxf(fmaxf(rm0.x, rm0.y), fmaxf(rm0.z, rm0.w)));
        const float mn1 = fmaxf(m_run[1], fmaxf(fmaxf(rm1.x, rm1.y), fmaxf(rm1.z, rm1.w)));
        const float corr0 = expf(m_run[0] - mn0), corr1 = expf(m_run[1] - mn1);
        float sum0 = 0.0f, sum1 = 0.0f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float p0 = expf(s[nt][0] - mn0), p1 = expf(s[nt][1] - mn0);
            const float p2 = expf(s[nt][2] - mn1), p3 = expf(s[nt][3] - mn1);
            sum0 += p0 + p1;
            sum1 += p2 + p3;
            const int col = wq * 16 + nt * 8 + 2 * t;
            *(__half2 *)(sm + SM_P + row0 * PROWB + col * 2) = __floats2half2_rn(p0, p1);
            *(__half2 *)(sm + SM_P + row1 * PROWB + col * 2) = __floats2half2_rn(p2, p3);
        }
        sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 1); sum0 += __shfl_xor_sync(0xFFFFFFFFu, sum0, 2);
        sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 1); sum1 += __shfl_xor_sync(0xFFFFFFFFu, sum1, 2);
        if (t == 0) { red_sum[row0 * 4 + wq] = sum0; red_sum[row1 * 4 + wq] = sum1; }
        __syncthreads();
        const float4 rs0 = *(const float4 *)(red_sum + row0 * 4), rs1 = *(const float4 *)(red_sum + row1 * 4);
        l_run[0] = l_run[0] * corr0 + ((rs0.x + rs0.y) + (rs0.z + rs0.w));
        l_run[1] = l_run[1] * corr1 + ((rs1.x + rs1.y) + (rs1.z + rs1.w));
        m_run[0] = mn0;
        m_run[1] = mn1;
#pragma unroll
        for (int i = 0; i < 16; ++i) { acc[i][0] *= corr0; acc[i][1] *= corr0; acc[i][2] *= corr1; acc[i][3] *= corr1; }

        // ---- O += P V for heads [16hr, +16) x columns [128wq, +128)
        {
            const uint32_t a_addr = sm_base + SM_P + (hr * 16 + (lane & 15)) * PROWB + (lane >> 4) * 16;
            const uint32_t b_addr = sm_base + SM_K + ((lane & 7) + ((lane >> 3) & 1) * 8) * ROWB + (wq * 128 + (lane >> 4) * 8) * 2;
#pragma unroll
            for (int kk = 0; kk < TJ / 16; ++kk) {
                uint32_t a[4];
                ldmatrix_x4(a, a_addr + kk * 32);
#pragma unroll
                for (int nb = 0; nb < 8; ++nb) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, b_addr + kk * 16 * ROWB + nb * 32);
                    mma_f16(acc[2 * nb], a, b[0], b[1]);
                    mma_f16(acc[2 * nb + 1], a, b[2], b[3]);
                }
            }
        }
    }

    // ---- results: rows row0/row1, columns 128wq + 8i + 2t, +1
    if (nsplit == 1) {
        const float inv0 = 1.0f / l_run[0], inv1 = 1.0f / l_run[1];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int col = wq * 128 + i * 8 + 2 * t;
            *(float2 *)(out + ((int64_t)bi * H + row0) * VD + col) = make_float2(acc[i][0] * inv0, acc[i][1] * inv0);
            *(float2 *)(out + ((int64_t)bi * H + row1) * VD + col) = make_float2(acc[i][2] * inv1, acc[i][3] * inv1);
        }
    } else {
        const int64_t p0 = ((int64_t)bi * H + row0) * nsplit + split, p1 = ((int64_t)bi * H + row1) * nsplit + split;
        if (wq == 0 && t == 0) {
            part_m[p0] = m_run[0]; part_l[p0] = l_run[0];
            part_m[p1] = m_run[1]; part_l[p1] = l_run[1];
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int col = wq * 128 + i * 8 + 2 * t;
            *(float2 *)(part_o + p0 * VD + col) = make_float2(acc[i][0], acc[i][1]);
            *(float2 *)(part_o + p1 * VD + col) = make_float2(acc[i][2], acc[i][3]);
        }
    }
}

} // namespace mla_tc
