// The whole decode token of the K3 engine on one GPU (or expert-parallel over the GPUs of a node):
// Model::from_bin + Model::forward (src/model.rs:906-1025, 2889-3031) over the device calls of this library.
//
//   embed row -> for every layer: AttnRes + rmsnorm -> KDA block (kda_forward, src/model.rs:1179-1232) or MLA
//   block (mla_forward, :1939-2022) -> residual -> AttnRes + rmsnorm -> dense MLP (dense_forward, :2382-2396) or
//   MoE (moe_forward, :2150-2380) -> residual; final AttnRes + rmsnorm -> q8_0 lm_head + greedy pick.
//
// Everything a token needs is resident on the GPU, and every launch of a token has the same shape at every
// position (the MLA caches count their positions on the device), so the token is captured once as a CUDA graph
// and replayed.  Projections that read the same vector are stacked into one f32 matrix at load: every row of a
// stacked matvec is the dot() the engine computes for that row, so stacking changes no bit.
#include <algorithm>
#include <new>
#include <string>
#include <vector>

#include "f32gemv.cuh"
#include "mk_common.cuh"

namespace {

// a[t][i] *= sigmoid(g[t * ldg + i]) for the rows of a prompt (the gate of mla_forward, src/model.rs:2017-2019; exp in double
// precision, rounded once, as mk_sigmoid_gate_dev takes it)
__global__ void __launch_bounds__(256) sigmoid_gate_rows_kernel(float *__restrict__ a, const float *__restrict__ g, int64_t count, int64_t ldg) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (i >= count) return;
    const float x = g[t * ldg + i];
    a[t * count + i] = __fmul_rn(a[t * count + i], __fdiv_rn(1.0f, __fadd_rn(1.0f, (float)exp((double)(-x)))));
}

__global__ void embed_row_kernel(const float *__restrict__ embed, const int32_t *__restrict__ token, int vocab, int d,
                                 float *__restrict__ hidden, int32_t *__restrict__ status) {
    int t = *token;
    if (t < 0 || t >= vocab) {   // a token id outside the vocabulary: reported, row 0 stands in
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(status, 0, MK_ERR_ARG);
        t = 0;
    }
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < d) hidden[j] = embed[(int64_t)t * d + j];
}
// out[j] = a[j] + b[j] (src/model.rs:2943-2952, 2994-2996: p[j] += attn_out[j]; hidden[j] = prefix2[j] + mlp_out[j])
__global__ void vec_add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int n) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < n) out[j] = __fadd_rn(a[j], b[j]);
}
// K[h] = kb[h][..nope] ++ k_rot ; V[h] = kb[h][nope..nope+v] (src/model.rs:1964-1973)
__global__ void mla_assemble_kernel(const float *__restrict__ kb, const float *__restrict__ k_rot, int H, int nope, int rope, int vd,
                                    float *__restrict__ k_new, float *__restrict__ v_new, int64_t ld_rot) {
    // blockIdx.y = token: kb [tokens][H (nope + v)], k_rot rows ld_rot floats apart, k_new [tokens][H (nope + rope)], v_new [tokens][H v]
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int qh = nope + rope, per = qh + vd;
    if (i >= H * per) return;
    const int64_t t = blockIdx.y;
    kb += t * H * (nope + vd);
    k_rot += t * ld_rot;
    k_new += t * H * qh;
    v_new += t * H * vd;
    const int h = i / per, r = i % per;
    if (r < nope) k_new[h * qh + r] = kb[h * (nope + vd) + r];
    else if (r < qh) k_new[h * qh + r] = k_rot[r - nope];
    else v_new[h * vd + (r - qh)] = kb[h * (nope + vd) + nope + (r - qh)];
}
// rows of n tokens' embeddings (layer-major prefill)
__global__ void embed_rows_kernel(const float *__restrict__ embed, const int32_t *__restrict__ tokens, int vocab, int d, float *__restrict__ out,
                                  int32_t *__restrict__ status) {
    int t = tokens[blockIdx.y];
    if (t < 0 || t >= vocab) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicCAS(status, 0, MK_ERR_ARG);
        t = 0;
    }
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < d) out[(int64_t)blockIdx.y * d + j] = embed[(int64_t)t * d + j];
}
// The glue between two blocks in ONE launch (src/model.rs:2905-2920, 2943-2959, 2994-2996, 3014-3017):
//   prefix = a [+ (b [+ c])]     residual adds: hidden = prefix2 + mlp_out with mlp_out = routed + shared, or prefix + attn_out
//   [push]  = prefix             the layer input becomes an AttnRes block row (after the mix below has used the old rows)
//   mixed  = attn_res(prefix, blocks[0 .. nb), w)   softmax over the RMS-normed scores, probability-weighted RAW rows;
//                                                   nb == 0 at the very first mix of a token: mixed = prefix
//   x      = rmsnorm(mixed, ln)
// One CTA; every sum in the engine's order: dot() with its 8 accumulators by one warp per row (mkf::reduce8), the
// softmax sequentially, exp in double precision rounded once.  Shared memory: prefix[d], mixed[d], scores[nb + 1].
__global__ void __launch_bounds__(512) glue_kernel(const float *__restrict__ a, const float *__restrict__ b, const float *__restrict__ c,
                                                   float *__restrict__ prefix_out, float *__restrict__ push_row,
                                                   const float *__restrict__ blocks, int nb, const float *__restrict__ w,
                                                   const float *__restrict__ ln, float eps, int d, float *__restrict__ x_out, int stage,
                                                   int64_t tok_vec, int64_t tok_blocks) {
    // one CTA per token (layer-major prefill: gridDim.x tokens; decode: one): token t's vectors lie t * tok_vec floats on,
    // its AttnRes block rows t * tok_blocks floats on
    {
        const int64_t ov = (int64_t)blockIdx.x * tok_vec, ob = (int64_t)blockIdx.x * tok_blocks;
        a += ov;
        if (b) b += ov;
        if (c) c += ov;
        if (prefix_out) prefix_out += ov;
        if (push_row) push_row += ob;
        blocks += ob;
        x_out += ov;
    }
    // stage: the nb block rows are copied into shared memory first (one round of coalesced loads for all rows, instead
    // of one exposed load latency per row and pass) - the launch then reserved room for them behind the scores
    extern __shared__ float gsm[];
    float *pre = gsm, *mix = gsm + d, *sc = gsm + 2 * d;
    const float *rows = blocks;
    if (stage && nb > 0) {
        float *rs = gsm + 2 * d + ((nb + 1 + 3) & ~3);
        for (int i = threadIdx.x; i < nb * d; i += blockDim.x) rs[i] = blocks[i];
        rows = rs;
    }
    __shared__ float s_inv;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5, j8 = lane & 7, full = d & ~7;
    for (int j = tid; j < d; j += blockDim.x) {
        float v = a[j];
        if (b) v = __fadd_rn(v, c ? __fadd_rn(b[j], c[j]) : b[j]);
        pre[j] = v;
        if (prefix_out) prefix_out[j] = v;
        if (push_row) push_row[j] = v;
    }
    __syncthreads();
    const float *src = pre;
    if (nb > 0) {
        for (int row = warp; row <= nb; row += nw) {     // score of block row `row`, the prefix last (as attn_res_score_kernel)
            const float *v = row < nb ? rows + (int64_t)row * d : pre;
            float acc = 0.0f;
            for (int k = 0; k < full; k += 8) acc = __fadd_rn(acc, __fmul_rn(v[k + j8], v[k + j8]));
            float ss = mkf::reduce8(acc, lane);
            for (int k = full; k < d; ++k) ss = __fadd_rn(ss, __fmul_rn(v[k], v[k]));
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)d), eps)));
            acc = 0.0f;
            for (int k = 0; k < full; k += 8) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(v[k + j8], inv), w[k + j8]));
            float s1 = mkf::reduce8(acc, lane);
            for (int k = full; k < d; ++k) s1 = __fadd_rn(s1, __fmul_rn(__fmul_rn(v[k], inv), w[k]));
            if (lane == 0) sc[row] = s1;
        }
        __syncthreads();
        if (tid == 0) {
            float mx = -INFINITY;
            for (int i = 0; i <= nb; ++i) mx = fmaxf(mx, sc[i]);
            float z = 0.0f;
            for (int i = 0; i <= nb; ++i) { sc[i] = (float)exp((double)__fsub_rn(sc[i], mx)); z = __fadd_rn(z, sc[i]); }
            for (int i = 0; i <= nb; ++i) sc[i] = __fdiv_rn(sc[i], z);
        }
        __syncthreads();
        for (int j = tid; j < d; j += blockDim.x) {
            float o = 0.0f;
            for (int i = 0; i < nb; ++i) o = __fadd_rn(o, __fmul_rn(sc[i], rows[(int64_t)i * d + j]));
            mix[j] = __fadd_rn(o, __fmul_rn(sc[nb], pre[j]));
        }
        __syncthreads();
        src = mix;
    }
    if (warp == 0) {
        float acc = 0.0f;
        for (int k = 0; k < full; k += 8) acc = __fadd_rn(acc, __fmul_rn(src[k + j8], src[k + j8]));
        float ss = mkf::reduce8(acc, lane);
        for (int k = full; k < d; ++k) ss = __fadd_rn(ss, __fmul_rn(src[k], src[k]));
        if (lane == 0) s_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)d), eps)));
    }
    __syncthreads();
    for (int j = tid; j < d; j += blockDim.x) x_out[j] = __fmul_rn(__fmul_rn(src[j], s_inv), ln[j]);
}
__global__ void copy_i32_kernel(const int32_t *__restrict__ src, int32_t *__restrict__ dst) { *dst = *src; }
// MXFP4 blobs of one layer (packed then scales, each blob where the file put it inside the staged span) -> the tiled
// device layout of a weight arena; one grid row per matrix (the arithmetic of retile_mxfp4_kernel in weights.cu).
__global__ void retile_mxfp4_batch_kernel(const uint8_t *__restrict__ span, const uint64_t *__restrict__ blob_off, uint8_t *__restrict__ arena,
                                          uint64_t stride_v, uint64_t stride_s, uint64_t scales_base, int first, int step, int64_t rows,
                                          int64_t cols, int64_t nrt, int64_t nb, int64_t nbp) {
    const int w = first + (int)blockIdx.y * step;   // entry of the (expert, matrix) list
    const uint8_t *packed = span + blob_off[w];
    const uint8_t *scales = packed + rows * cols / 2;
    uint32_t *tv = (uint32_t *)(arena + (uint64_t)w * stride_v);
    uint8_t *ts = arena + scales_base + (uint64_t)w * stride_s;
    const int64_t nwords = nrt * (nbp / 2) * 128;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < nwords) {
        const int64_t chunk = idx >> 7;
        const int within = (int)(idx & 127);
        const int lane = within >> 2, j = within & 3;
        const int g = lane >> 2, t = lane & 3;
        const int64_t rt = chunk / (nbp / 2), bp = chunk % (nbp / 2);
        const int64_t row = rt * 16 + g + ((j & 1) ? 8 : 0);
        const int64_t b = bp * 2 + (j >> 1);
        uint32_t v = 0;
        if (row < rows && b < nb) {
            const uint8_t *p = packed + row * (cols / 2) + b * 16 + t * 4;   // blobs are only byte-aligned inside the span
            v = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
        }
        tv[idx] = v;
    }
    const int64_t nsc = nrt * nbp * 16;
    if (idx < nsc) {
        const int r16 = (int)(idx & 15);
        const int64_t rb = idx >> 4;
        const int64_t rt = rb / nbp, b = rb % nbp;
        const int64_t row = rt * 16 + r16;
        ts[mk_scale_off(rt, nbp, b, r16)] = (row < rows && b < nb) ? scales[row * nb + b] : (uint8_t)0;
    }
}

struct Layer {
    bool is_mla = false, is_moe = false;
    int nb_before = 0;       // AttnRes block rows before this layer's first mix
    bool pushes = false;     // l % attn_res_block == 0: the layer input becomes a block row
    float *input_ln = nullptr, *post_ln = nullptr, *sa_w = nullptr, *mlp_w = nullptr;
    // KDA: rows of w_x = q, k, v, g_proj (proj each), f_a (fa), b_proj (heads)
    float *w_x = nullptr, *f_b = nullptr, *o_proj = nullptr;
    int w_x_rows = 0;
    mk_kda *kda = nullptr;
    // MLA: rows of w_x = q_a (qa), kv_a (kva + rope), g_proj (H v)
    float *q_a_ln = nullptr, *q_b = nullptr, *kv_a_ln = nullptr, *kv_b = nullptr;
    mk_mla *cache = nullptr;
    // FFN
    float *dgu = nullptr, *dd = nullptr;     // dense: [gate; up] stacked, down
    mk_moe *moe = nullptr;
    void *expert_arena = nullptr;
    std::vector<mk_weight> expert_w;          // records into the arena (not owners)
    mk_weight rd, ru, sg, sd, su;             // f32 records for the MoE descriptor (not owners)
};

} // namespace

struct mk_model {
    mk_model_config cfg;
    mk_model_opts opts;
    int world, rank;
    std::vector<void *> owned;      // device allocations freed with the model
    int64_t weight_bytes = 0;
    std::vector<Layer> layers;
    float *embed = nullptr, *norm_f = nullptr, *out_w = nullptr;
    mk_weight *head = nullptr;      // q8_0 rows [head_row0, head_row0 + head_rows) of lm_head
    int64_t head_row0 = 0, head_rows = 0;
    mk_gather *gather = nullptr;
    mk_moe_ep *ep = nullptr;
    // activations
    float *hidden = nullptr, *res = nullptr, *x = nullptr, *attn_out = nullptr, *p2 = nullptr, *mlp_out = nullptr, *blocks = nullptr;
    float *sh_out = nullptr;        // the MoE's shared-expert output when it is added by the next glue launch
    float *embed_row = nullptr;     // the token's embedding row
    int max_blocks = 0;
    float *y = nullptr, *g_low = nullptr, *o = nullptr;                                     // KDA
    float *qan = nullptr, *q = nullptr, *kpn = nullptr, *kb = nullptr, *k_new = nullptr, *v_new = nullptr, *attn = nullptr; // MLA
    float *au = nullptr, *act = nullptr;                                                    // dense
    float *logits = nullptr;
    float *layer_hidden = nullptr;   // opts.keep_layer_hidden: [n_layers][4][d] taps of the last token (see mk_model_layer_hidden)
    int32_t *tok = nullptr, *next = nullptr;
    int positions = 0;
    // layer-major prefill (mk_model_prefill): activations of up to pf_cap tokens, allocated at the first call
    int pf_cap = 0;
    int32_t *pf_tok = nullptr;
    float *pf_hidden = nullptr, *pf_x = nullptr, *pf_attn_out = nullptr, *pf_p2 = nullptr, *pf_mlp_out = nullptr, *pf_blocks = nullptr, *pf_embed = nullptr;
    float *pf_y = nullptr, *pf_g_low = nullptr, *pf_o = nullptr, *pf_fa = nullptr;
    float *pf_qa = nullptr, *pf_qan = nullptr, *pf_q = nullptr, *pf_kva = nullptr, *pf_kpn = nullptr, *pf_kb = nullptr, *pf_k_new = nullptr, *pf_v_new = nullptr, *pf_attn = nullptr;
    float *pf_au = nullptr, *pf_act = nullptr;
    int64_t launches_per_token = 0;
    uint8_t handles[128] = {0};     // world > 1: IPC handles of this rank's expert-row table and logits buffer
    // the recorded token.  With several GPUs the exchange kernels alternate between two buffer parities by step number, and
    // the recorded launches carry the pointers of the parities they were recorded with: one recording per combination of
    // (expert exchange parity, lm_head exchange parity) at the start of a token, made when first needed
    cudaGraphExec_t graphs[4] = {nullptr, nullptr, nullptr, nullptr};
    uint32_t ep_steps_per_token = 0, gather_steps_per_token = 0;
    void *graph_ws = nullptr;       // the context's shared workspace as the recorded launches saw it
    uint64_t graph_epoch = 0;       // the context's allocation epoch at the recording: a layer that grew its buffers since (a
                                    // longer prompt chunk than any before) left the recorded launches with stale pointers
    int warm = 0;
};

namespace {

struct Loader {
    mk_ctx *ctx;
    const mk_bin *bin;
    mk_model *m;
    int32_t rc = MK_OK;
    std::string err;

    const void *find(const std::string &name, int dtype, uint64_t bytes) {
        if (rc != MK_OK) return nullptr;
        int32_t dt = 0;
        const void *p = nullptr;
        uint64_t sz = 0;
        if (mk_bin_find(bin, name.c_str(), &dt, nullptr, nullptr, &p, &sz) != MK_OK || dt != dtype || sz != bytes) {
            rc = MK_ERR_ARG;
            err = "tensor " + name + " is missing or has the wrong type or size";
            return nullptr;
        }
        return p;
    }
    void *dev_alloc(size_t bytes) {
        if (rc != MK_OK) return nullptr;
        void *d = nullptr;
        const cudaError_t e = cudaMalloc(&d, bytes ? bytes : 4);
        if (e != cudaSuccess) { rc = e == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA; err = cudaGetErrorString(e); return nullptr; }
        m->owned.push_back(d);
        return d;
    }
    float *zeros(size_t count) {
        float *d = (float *)dev_alloc(count * 4);
        if (d && cudaMemsetAsync(d, 0, count * 4, ctx->stream) != cudaSuccess) { rc = MK_ERR_CUDA; err = "memset failed"; }
        return d;
    }
    void upload(void *dst, const void *src, size_t bytes) {
        if (rc != MK_OK) return;
        // the source is a file mapping (pageable): the copy returns when the bytes have left it
        if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) { rc = MK_ERR_CUDA; err = "upload failed"; }
    }
    // one f32 tensor [count]
    float *f32(const std::string &name, uint64_t count) {
        const void *p = find(name, MK_DTYPE_F32, count * 4);
        float *d = (float *)dev_alloc((size_t)count * 4);
        if (p && d) { upload(d, p, (size_t)count * 4); m->weight_bytes += (int64_t)count * 4; }
        return d;
    }
    // several f32 matrices [rows_i, cols] stacked by rows
    float *stacked(const std::vector<std::pair<std::string, uint64_t>> &parts, uint64_t cols, int *rows_out) {
        uint64_t rows = 0;
        for (auto &p : parts) rows += p.second;
        float *d = (float *)dev_alloc((size_t)rows * cols * 4);
        uint64_t r = 0;
        for (auto &p : parts) {
            const void *src = find(p.first, MK_DTYPE_F32, p.second * cols * 4);
            if (src && d) upload(d + r * cols, src, (size_t)p.second * cols * 4);
            r += p.second;
        }
        m->weight_bytes += (int64_t)rows * cols * 4;
        if (rows_out) *rows_out = (int)rows;
        return d;
    }
    // norm.weight * proj.weight, combined at load (src/model.rs:911-915)
    float *combined(const std::string &norm, const std::string &proj, uint64_t d) {
        const float *a = (const float *)find(norm, MK_DTYPE_F32, d * 4), *b = (const float *)find(proj, MK_DTYPE_F32, d * 4);
        float *dv = (float *)dev_alloc((size_t)d * 4);
        if (a && b && dv) {
            std::vector<float> t(d);
            for (uint64_t i = 0; i < d; ++i) t[i] = a[i] * b[i];
            if (cudaMemcpy(dv, t.data(), (size_t)d * 4, cudaMemcpyHostToDevice) != cudaSuccess) { rc = MK_ERR_CUDA; err = "upload failed"; }
            m->weight_bytes += (int64_t)d * 4;
        }
        return dv;
    }
};

mk_weight f32_record(float *values, int64_t rows, int64_t cols) {
    mk_weight w;
    memset(&w, 0, sizeof(w));
    w.fmt = MK_FMT_F32; w.rows = rows; w.cols = cols; w.values = values; w.values_bytes = (size_t)rows * cols * 4;
    return w;
}

// The routed experts [e0, e1) of one MoE layer: the span of the file that holds their blobs goes to the GPU in one
// copy and one launch re-tiles all of them into an arena (values of every matrix, then scales of every matrix).
int32_t load_experts(Loader &L, Layer &ly, int layer, int e0, int e1) {
    const mk_model_config &c = L.m->cfg;
    const int64_t I = c.moe_inter, R = c.routed_hidden;
    const int n = (e1 - e0) * 3;
    ly.expert_w.assign((size_t)c.n_experts * 3, mk_weight());
    for (auto &w : ly.expert_w) memset(&w, 0, sizeof(w));
    if (n <= 0) return MK_OK;
    static const char *const wn[3] = {"w1", "w2", "w3"};
    std::vector<const uint8_t *> src((size_t)n);
    const uint64_t blob = (uint64_t)I * R / 2 + (uint64_t)I * R / 32;
    const uint8_t *lo = nullptr, *hi = nullptr;
    for (int e = e0; e < e1; ++e)
        for (int k = 0; k < 3; ++k) {
            const std::string name = "layers." + std::to_string(layer) + ".block_sparse_moe.experts." + std::to_string(e) + "." + wn[k];
            int32_t dt = 0, nd = 0;
            uint32_t dims[4] = {0, 0, 0, 0};
            const void *p = nullptr;
            uint64_t sz = 0;
            const int64_t rows = k == 1 ? R : I, cols = k == 1 ? I : R;
            if (mk_bin_find(L.bin, name.c_str(), &dt, &nd, dims, &p, &sz) != MK_OK || dt != MK_DTYPE_MXFP4 || nd != 2 || dims[0] != rows ||
                dims[1] != cols || sz != blob) {
                mk_set_error("mk_model_open: expert tensor %s is missing, not MXFP4 or of the wrong shape", name.c_str());
                return MK_ERR_ARG;
            }
            const uint8_t *b = (const uint8_t *)p;
            src[(size_t)(e - e0) * 3 + k] = b;
            if (!lo || b < lo) lo = b;
            if (!hi || b + blob > hi) hi = b + blob;
        }
    // w1 / w3 are [I, R], w2 is [R, I]: the same element count, but different tilings; keep one stride for all
    auto tiled_bytes = [](int64_t rows, int64_t cols, size_t *vb, size_t *sb) {
        const int64_t nrt = mk_ceil_div(rows, 16), nbp = mk_ceil_div(cols / 32, 4) * 4;
        *vb = (size_t)nrt * (nbp / 2) * 512;
        *sb = (size_t)nrt * nbp * 16;
    };
    size_t vb13, sb13, vb2, sb2;
    tiled_bytes(I, R, &vb13, &sb13);
    tiled_bytes(R, I, &vb2, &sb2);
    const size_t stride_v = mk_align_up(vb13 > vb2 ? vb13 : vb2, 256), stride_s = mk_align_up(sb13 > sb2 ? sb13 : sb2, 256);
    const size_t scales_base = stride_v * (size_t)n, arena_bytes = scales_base + stride_s * (size_t)n;
    const size_t span = (size_t)(hi - lo);
    cudaError_t e_ = cudaMalloc(&ly.expert_arena, arena_bytes);
    void *stage = nullptr;
    uint64_t *off_dev = nullptr;
    if (e_ == cudaSuccess) e_ = cudaMalloc(&stage, span);
    if (e_ == cudaSuccess) e_ = cudaMalloc((void **)&off_dev, (size_t)n * 8);
    std::vector<uint64_t> off((size_t)n);
    for (int i = 0; i < n; ++i) off[(size_t)i] = (uint64_t)(src[(size_t)i] - lo);
    if (e_ == cudaSuccess) e_ = cudaMemcpyAsync(stage, lo, span, cudaMemcpyHostToDevice, L.ctx->stream);
    if (e_ == cudaSuccess) e_ = cudaMemcpyAsync(off_dev, off.data(), (size_t)n * 8, cudaMemcpyHostToDevice, L.ctx->stream);
    // one launch per matrix kind (w1, w2, w3 of every expert): grid rows = experts
    for (int k = 0; k < 3 && e_ == cudaSuccess; ++k) {
        const int64_t rows = k == 1 ? R : I, cols = k == 1 ? I : R;
        const int64_t nrt = mk_ceil_div(rows, 16), nb = cols / 32, nbp = mk_ceil_div(nb, 4) * 4;
        const int64_t work = nrt * (nbp / 2) * 128 > nrt * nbp * 16 ? nrt * (nbp / 2) * 128 : nrt * nbp * 16;
        retile_mxfp4_batch_kernel<<<dim3((unsigned)mk_ceil_div(work, 256), (unsigned)(e1 - e0)), 256, 0, L.ctx->stream>>>(
            (const uint8_t *)stage, off_dev, (uint8_t *)ly.expert_arena, stride_v, stride_s, scales_base, k, 3, rows, cols, nrt, nb, nbp);
        L.ctx->launches++;
        e_ = cudaGetLastError();
    }
    if (e_ == cudaSuccess) e_ = cudaStreamSynchronize(L.ctx->stream);
    if (stage) cudaFree(stage);
    if (off_dev) cudaFree(off_dev);
    if (e_ != cudaSuccess) {
        mk_set_error("mk_model_open: experts of layer %d: %s", layer, cudaGetErrorString(e_));
        return e_ == cudaErrorMemoryAllocation ? MK_ERR_OOM : MK_ERR_CUDA;
    }
    for (int e = e0; e < e1; ++e)
        for (int k = 0; k < 3; ++k) {
            const size_t i = (size_t)(e - e0) * 3 + k;
            mk_weight &w = ly.expert_w[(size_t)e * 3 + k];
            w.fmt = MK_FMT_MXFP4;
            w.rows = k == 1 ? R : I; w.cols = k == 1 ? I : R;
            w.nrt = mk_ceil_div(w.rows, 16); w.nb = w.cols / 32; w.nbp = mk_ceil_div(w.nb, 4) * 4;
            w.values = (uint8_t *)ly.expert_arena + i * stride_v;
            w.scales = (uint8_t *)ly.expert_arena + scales_base + i * stride_s;
            w.values_bytes = k == 1 ? vb2 : vb13; w.scales_bytes = k == 1 ? sb2 : sb13;
        }
    L.m->weight_bytes += (int64_t)arena_bytes;
    return MK_OK;
}

void free_model(mk_ctx *ctx, mk_model *m) {
    if (!m) return;
    cudaStreamSynchronize(ctx->stream);
    for (cudaGraphExec_t &g : m->graphs) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
    for (Layer &ly : m->layers) {
        if (ly.kda) mk_kda_free(ctx, ly.kda);
        if (ly.cache) mk_mla_free(ctx, ly.cache);
        if (ly.moe) mk_moe_free(ctx, ly.moe);
        if (ly.expert_arena) cudaFree(ly.expert_arena);
    }
    if (m->head) mk_weight_free(ctx, m->head);
    if (m->gather) mk_gather_free(ctx, m->gather);
    if (m->ep) mk_moe_ep_free(ctx, m->ep);
    for (void *p : m->owned) cudaFree(p);
    float *pf[] = {m->pf_hidden, m->pf_x, m->pf_attn_out, m->pf_p2, m->pf_mlp_out, m->pf_blocks, m->pf_embed, m->pf_y, m->pf_g_low, m->pf_o, m->pf_fa,
                   m->pf_qa, m->pf_qan, m->pf_q, m->pf_kva, m->pf_kpn, m->pf_kb, m->pf_k_new, m->pf_v_new, m->pf_attn, m->pf_au, m->pf_act};
    for (float *p : pf) if (p) cudaFree(p);
    if (m->pf_tok) cudaFree(m->pf_tok);
    delete m;
}

} // namespace

extern "C" int32_t mk_model_open(mk_ctx *ctx, const mk_bin *bin, const mk_model_opts *opts, mk_model **out) {
    MK_CHECK_ARG(ctx != nullptr && bin != nullptr && opts != nullptr && out != nullptr, "NULL argument");
    *out = nullptr;
    mk_model_config c;
    mk_bin_config(bin, &c);
    if (c.has_layer_lists || c.is_deepseek) {
        mk_set_error("mk_model_open: explicit per-layer type lists and the DeepSeek architecture are not supported");
        return MK_ERR_UNSUPPORTED;
    }
    const int world = opts->world > 1 ? opts->world : 1, rank = opts->world > 1 ? opts->rank : 0;
    MK_CHECK_ARG(world <= 8 && rank >= 0 && rank < world, "need 0 <= rank < world <= 8");
    MK_CHECK_ARG(opts->max_positions >= 1, "max_positions must be positive");
    const int64_t d = c.d, proj = (int64_t)c.kda_heads * c.kda_dim, qh = c.mla_nope + c.mla_rope, H = c.mla_heads;
    const int64_t qb = H * qh, kvb = H * (c.mla_nope + c.mla_v), cdim = c.mla_kva + c.mla_rope, hv = H * c.mla_v;
    MK_CHECK_ARG(c.n_layers >= 1 && d % 32 == 0 && c.vocab >= 1 && c.attn_res_block >= 1, "bad model dims");
    MK_CHECK_ARG(proj % 4 == 0 && c.kda_fa % 4 == 0 && c.mla_qa % 4 == 0 && cdim % 4 == 0 && c.mla_kva % 4 == 0 && c.dense_inter % 4 == 0,
                 "projection widths must be multiples of 4 (slices of a stacked result stay 16-byte aligned)");
    MK_CHECK_ARG(c.n_experts % world == 0 && c.vocab % world == 0, "n_experts and vocab must divide by the number of ranks");
    MK_CHECK_ARG((size_t)(2 * d + c.n_layers / c.attn_res_block + 4) * 4 <= 48 * 1024, "hidden size too large for the residual/AttnRes/norm kernel (two rows in shared memory)");
    MK_CUDA(cudaSetDevice(ctx->device));
    mk_model *m = new (std::nothrow) mk_model();
    if (!m) return MK_ERR_OOM;
    m->cfg = c; m->opts = *opts; m->world = world; m->rank = rank;
    Loader L{ctx, bin, m};
    auto fail = [&](int32_t rc, const std::string &why) {
        if (!why.empty()) mk_set_error("mk_model_open: %s", why.c_str());
        free_model(ctx, m);
        return rc;
    };
    m->embed = L.f32("embed_tokens.weight", (uint64_t)c.vocab * d);
    m->norm_f = L.f32("norm.weight", d);
    m->out_w = L.combined("output_attn_res_norm.weight", "output_attn_res_proj.weight", d);
    const int max_blocks = (int)(c.n_layers / c.attn_res_block + 2);
    m->max_blocks = max_blocks;
    m->embed_row = L.zeros(d);
    m->blocks = L.zeros((size_t)max_blocks * d);
    m->sh_out = L.zeros(d);
    m->hidden = L.zeros(d); m->res = L.zeros(d); m->x = L.zeros(d); m->attn_out = L.zeros(d); m->p2 = L.zeros(d); m->mlp_out = L.zeros(d);
    m->y = L.zeros((size_t)(4 * proj + c.kda_fa + c.kda_heads) > (size_t)(c.mla_qa + cdim + hv) ? (size_t)(4 * proj + c.kda_fa + c.kda_heads)
                                                                                             : (size_t)(c.mla_qa + cdim + hv));
    m->g_low = L.zeros(proj); m->o = L.zeros(proj);
    m->qan = L.zeros(c.mla_qa); m->q = L.zeros(qb); m->kpn = L.zeros(c.mla_kva); m->kb = L.zeros(kvb);
    m->k_new = L.zeros(qb); m->v_new = L.zeros(hv); m->attn = L.zeros(hv);
    m->au = L.zeros((size_t)2 * c.dense_inter); m->act = L.zeros(c.dense_inter);
    m->logits = L.zeros(c.vocab);
    if (opts->keep_layer_hidden) m->layer_hidden = L.zeros((size_t)c.n_layers * 4 * d);
    m->tok = (int32_t *)L.zeros(1); m->next = (int32_t *)L.zeros(1);
    if (L.rc != MK_OK) return fail(L.rc, L.err);

    m->layers.resize(c.n_layers);
    int nb = 0;
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        Layer &ly = m->layers[l];
        const std::string p = "layers." + std::to_string(l) + ".";
        ly.is_mla = l % 4 == 3 || l == c.n_layers - 1;   // Config::is_mla (src/config.rs:127-132)
        ly.is_moe = l >= c.first_k_dense;                // Config::is_moe (src/config.rs:133-138)
        ly.nb_before = nb;
        ly.pushes = l % c.attn_res_block == 0;
        if (ly.pushes) ++nb;
        ly.input_ln = L.f32(p + "input_layernorm.weight", d);
        ly.post_ln = L.f32(p + "post_attention_layernorm.weight", d);
        ly.sa_w = L.combined(p + "self_attention_res_norm.weight", p + "self_attention_res_proj.weight", d);
        ly.mlp_w = L.combined(p + "mlp_res_norm.weight", p + "mlp_res_proj.weight", d);
        if (ly.is_mla) {
            ly.w_x = L.stacked({{p + "self_attn.q_a_proj.weight", c.mla_qa}, {p + "self_attn.kv_a_proj_with_mqa.weight", (uint64_t)cdim},
                                {p + "self_attn.g_proj.weight", (uint64_t)hv}}, d, &ly.w_x_rows);
            ly.q_a_ln = L.f32(p + "self_attn.q_a_layernorm.weight", c.mla_qa);
            ly.q_b = L.f32(p + "self_attn.q_b_proj.weight", (uint64_t)qb * c.mla_qa);
            ly.kv_a_ln = L.f32(p + "self_attn.kv_a_layernorm.weight", c.mla_kva);
            ly.kv_b = L.f32(p + "self_attn.kv_b_proj.weight", (uint64_t)kvb * c.mla_kva);
            ly.o_proj = L.f32(p + "self_attn.o_proj.weight", (uint64_t)d * hv);
            if (L.rc != MK_OK) return fail(L.rc, L.err);
            mk_mla_desc md = {MK_MLA_PER_HEAD, (int32_t)H, (int32_t)c.mla_nope, (int32_t)c.mla_rope, (int32_t)c.mla_v, opts->max_positions, 1};
            const int32_t rc = mk_mla_create(ctx, &md, &ly.cache);
            if (rc != MK_OK) return fail(rc, "");
        } else {
            ly.w_x = L.stacked({{p + "self_attn.q_proj.weight", (uint64_t)proj}, {p + "self_attn.k_proj.weight", (uint64_t)proj},
                                {p + "self_attn.v_proj.weight", (uint64_t)proj}, {p + "self_attn.g_proj.weight", (uint64_t)proj},
                                {p + "self_attn.f_a_proj.weight", c.kda_fa}, {p + "self_attn.b_proj.weight", c.kda_heads}}, d, &ly.w_x_rows);
            ly.f_b = L.f32(p + "self_attn.f_b_proj.weight", (uint64_t)proj * c.kda_fa);
            ly.o_proj = L.f32(p + "self_attn.o_proj.weight", (uint64_t)d * proj);
            mk_kda_desc kd;
            memset(&kd, 0, sizeof(kd));
            kd.heads = (int32_t)c.kda_heads; kd.dim = (int32_t)c.kda_dim; kd.kconv = (int32_t)c.kda_conv; kd.gate_lb = c.gate_lb; kd.rms_eps = c.rms_eps;
            kd.q_conv = (const float *)L.find(p + "self_attn.q_conv1d.weight", MK_DTYPE_F32, (uint64_t)proj * c.kda_conv * 4);
            kd.k_conv = (const float *)L.find(p + "self_attn.k_conv1d.weight", MK_DTYPE_F32, (uint64_t)proj * c.kda_conv * 4);
            kd.v_conv = (const float *)L.find(p + "self_attn.v_conv1d.weight", MK_DTYPE_F32, (uint64_t)proj * c.kda_conv * 4);
            kd.a_log = (const float *)L.find(p + "self_attn.A_log", MK_DTYPE_F32, (uint64_t)c.kda_dim * 4);
            kd.dt_bias = (const float *)L.find(p + "self_attn.dt_bias", MK_DTYPE_F32, (uint64_t)proj * 4);
            kd.o_norm = (const float *)L.find(p + "self_attn.o_norm.weight", MK_DTYPE_F32, (uint64_t)c.kda_dim * 4);
            if (L.rc != MK_OK) return fail(L.rc, L.err);
            const int32_t rc = mk_kda_create(ctx, &kd, &ly.kda);
            if (rc != MK_OK) return fail(rc, "");
        }
        if (ly.is_moe) {
            const std::string q = p + "block_sparse_moe.";
            const float *gate_w = (const float *)L.find(q + "gate.weight", MK_DTYPE_F32, (uint64_t)c.n_experts * d * 4);
            const float *gate_b = (const float *)L.find(q + "gate.e_score_correction_bias", MK_DTYPE_F32, (uint64_t)c.n_experts * 4);
            const float *rnorm = (const float *)L.find(q + "routed_expert_norm.weight", MK_DTYPE_F32, (uint64_t)c.routed_hidden * 4);
            // routed_down, shared gate and shared up read the same vector: one stacked matrix, one launch per token
            float *stk = L.stacked({{q + "routed_expert_down_proj.weight", c.routed_hidden}, {q + "shared_experts.gate_proj.weight", c.shared_inter},
                                    {q + "shared_experts.up_proj.weight", c.shared_inter}}, d, nullptr);
            ly.rd = f32_record(stk, c.routed_hidden, d);
            ly.sg = f32_record(stk ? stk + (size_t)c.routed_hidden * d : nullptr, c.shared_inter, d);
            ly.su = f32_record(stk ? stk + (size_t)(c.routed_hidden + c.shared_inter) * d : nullptr, c.shared_inter, d);
            ly.ru = f32_record(L.f32(q + "routed_expert_up_proj.weight", (uint64_t)d * c.routed_hidden), d, c.routed_hidden);
            ly.sd = f32_record(L.f32(q + "shared_experts.down_proj.weight", (uint64_t)d * c.shared_inter), d, c.shared_inter);
            if (L.rc != MK_OK) return fail(L.rc, L.err);
            const int per = (int)c.n_experts / world;
            int32_t rc = load_experts(L, ly, (int)l, rank * per, (rank + 1) * per);
            if (rc != MK_OK) return fail(rc, "");
            std::vector<const mk_weight *> table((size_t)c.n_experts * 3, nullptr);
            for (size_t i = 0; i < table.size(); ++i) table[i] = ly.expert_w[i].values ? &ly.expert_w[i] : nullptr;
            mk_moe_desc md;
            memset(&md, 0, sizeof(md));
            md.n_experts = (int32_t)c.n_experts; md.top_k = (int32_t)c.top_k; md.d = (int32_t)d; md.inter = (int32_t)c.moe_inter;
            md.activation = MK_MOE_SITU; md.gate_w = gate_w; md.gate_b = gate_b; md.experts = table.data(); md.router = MK_ROUTER_SIGMOID;
            md.latent = (int32_t)c.routed_hidden; md.rms_eps = c.rms_eps; md.routed_down = &ly.rd; md.routed_up = &ly.ru; md.routed_norm = rnorm;
            md.shared_f32[0] = &ly.sg; md.shared_f32[1] = &ly.sd; md.shared_f32[2] = &ly.su;
            md.act_mode = MK_ACT_Q8 | (opts->strict ? MK_ACT_STRICT : 0);
            rc = mk_moe_create(ctx, &md, &ly.moe);
            if (rc != MK_OK) return fail(rc, "");
            m->weight_bytes += (int64_t)c.n_experts * d * 4;
        } else {
            ly.dgu = L.stacked({{p + "mlp.gate_proj.weight", c.dense_inter}, {p + "mlp.up_proj.weight", c.dense_inter}}, d, nullptr);
            ly.dd = L.f32(p + "mlp.down_proj.weight", (uint64_t)d * c.dense_inter);
        }
        if (L.rc != MK_OK) return fail(L.rc, L.err);
    }
    // q8_0 copy of (this rank's rows of) lm_head, quantized on the GPU (Q8Head::from_f32, src/model.rs:921-925)
    m->head_rows = c.vocab / world;
    m->head_row0 = (int64_t)rank * m->head_rows;
    const float *lm = (const float *)L.find("lm_head.weight", MK_DTYPE_F32, (uint64_t)c.vocab * d * 4);
    if (L.rc != MK_OK) return fail(L.rc, L.err);
    int32_t rc = mk_weight_q8_from_f32(ctx, lm + m->head_row0 * d, m->head_rows, d, MK_SCALE_F32, 0, &m->head);
    if (rc != MK_OK) return fail(rc, "");
    m->weight_bytes += mk_weight_bytes(m->head);
    if (world > 1) {
        rc = mk_gather_create(ctx, rank, world, c.vocab, 1, &m->gather, m->handles + 64);
        if (rc != MK_OK) return fail(rc, "");
        mk_moe *first = nullptr;
        for (Layer &ly : m->layers) if (ly.moe) { first = ly.moe; break; }
        if (first) {
            rc = mk_moe_ep_create(ctx, first, rank, world, 1, &m->ep, m->handles);
            if (rc != MK_OK) return fail(rc, "");
        }
    }
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    *out = m;
    return MK_OK;
}

extern "C" int32_t mk_model_free(mk_ctx *ctx, mk_model *m) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr, "NULL argument");
    cudaSetDevice(ctx->device);
    free_model(ctx, m);
    return MK_OK;
}
extern "C" int32_t mk_model_positions(mk_ctx *ctx, const mk_model *m) {
    if (!ctx || !m) { mk_set_error("mk_model_positions: NULL argument"); return MK_ERR_ARG; }
    return m->positions;
}
extern "C" int64_t mk_model_weight_bytes(const mk_model *m) { return m ? m->weight_bytes : -1; }
extern "C" int64_t mk_model_launches_per_token(const mk_model *m) { return m ? m->launches_per_token : -1; }

extern "C" int32_t mk_model_reset(mk_ctx *ctx, mk_model *m) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr, "NULL argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    for (Layer &ly : m->layers) {
        int32_t rc = MK_OK;
        if (ly.kda) rc = mk_kda_reset(ctx, ly.kda);
        if (ly.cache) rc = mk_mla_reset(ctx, ly.cache, -1);
        if (rc != MK_OK) return rc;
    }
    m->positions = 0;
    return MK_OK;
}

extern "C" int32_t mk_model_ep_handles(mk_ctx *ctx, mk_model *m, uint8_t *handles) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && handles != nullptr, "NULL argument");
    MK_CHECK_ARG(m->world > 1 && m->gather != nullptr, "the model was opened for one GPU");
    memcpy(handles, m->handles, 128);
    return MK_OK;
}
extern "C" int32_t mk_model_ep_connect(mk_ctx *ctx, mk_model *m, const uint8_t *all) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && all != nullptr, "NULL argument");
    MK_CHECK_ARG(m->world > 1 && m->gather != nullptr, "the model was opened for one GPU");
    std::vector<uint8_t> a((size_t)m->world * 64), b((size_t)m->world * 64);
    for (int r = 0; r < m->world; ++r) {
        memcpy(&a[(size_t)r * 64], all + (size_t)r * 128, 64);
        memcpy(&b[(size_t)r * 64], all + (size_t)r * 128 + 64, 64);
    }
    int32_t rc = m->ep ? mk_moe_ep_connect(ctx, m->ep, a.data()) : MK_OK;
    if (rc != MK_OK) return rc;
    return mk_gather_connect(ctx, m->gather, b.data());
}

namespace {

// Every launch of one token, on the context's stream.  Reads m->tok, leaves m->logits and m->next.
int32_t enqueue_token(mk_ctx *ctx, mk_model *m) {
    const mk_model_config &c = m->cfg;
    const int d = (int)c.d, proj = (int)(c.kda_heads * c.kda_dim), H = (int)c.mla_heads, nope = (int)c.mla_nope, rope = (int)c.mla_rope;
    const int vd = (int)c.mla_v, qh = nope + rope, qa = (int)c.mla_qa, kva = (int)c.mla_kva, cdim = kva + rope, hv = H * vd, fa = (int)c.kda_fa;
    const float eps = c.rms_eps;
    cudaStream_t st = ctx->stream;
    int32_t rc;
#define RC(call) do { rc = (call); if (rc != MK_OK) return rc; } while (0)
    // residual inputs of the next glue launch: hidden = ga [+ (gb [+ gc])]
    const float *ga = m->embed_row, *gb = nullptr, *gc = nullptr;
    embed_row_kernel<<<(unsigned)mk_ceil_div(d, 256), 256, 0, st>>>(m->embed, m->tok, (int)c.vocab, d, m->embed_row, ctx->status_dev);
    ctx->launches++;
    const size_t gsm_plain = (size_t)(2 * d + m->max_blocks + 2) * 4, gsm_staged = (size_t)(2 * d + m->max_blocks + 8 + (size_t)m->max_blocks * d) * 4;
    const int gstage = gsm_staged <= 48 * 1024 ? 1 : 0;      // rows staged when they fit the default shared-memory limit
    const size_t gsm_bytes = gstage ? gsm_staged : gsm_plain;
    auto tap = [&](uint32_t l, int k, const float *src) -> int32_t {
        if (m->layer_hidden) MK_CUDA(cudaMemcpyAsync(m->layer_hidden + ((size_t)l * 4 + k) * d, src, (size_t)d * 4, cudaMemcpyDeviceToDevice, st));
        return MK_OK;
    };
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        Layer &ly = m->layers[l];
        int nb = ly.nb_before;
        // hidden of this layer (the previous layer's residual adds), AttnRes mix over the old block rows, rmsnorm -> x
        glue_kernel<<<1, 512, gsm_bytes, st>>>(ga, gb, gc, m->hidden, ly.pushes ? m->blocks + (size_t)nb * d : nullptr, m->blocks, nb, ly.sa_w,
                                               ly.input_ln, eps, d, m->x, gstage, 0, 0);
        ctx->launches++;
        if (l > 0) RC(tap(l - 1, 3, m->hidden));
        bool have_prefix = true;
        if (ly.pushes) { ++nb; have_prefix = false; }
        if (ly.is_mla) {
            float *y = m->y;
            RC(mk_launch_f32_gemv(ctx, ly.w_x, ly.w_x_rows, d, m->x, 1, y, ly.w_x_rows, 0));          // q_a, kv_a, g_proj of x
            RC(mk_launch_rmsnorm(ctx, y, ly.q_a_ln, 1, qa, eps, m->qan));
            RC(mk_launch_f32_gemv(ctx, ly.q_b, (int64_t)H * qh, qa, m->qan, 1, m->q, (int64_t)H * qh, 0));
            RC(mk_launch_rmsnorm(ctx, y + qa, ly.kv_a_ln, 1, kva, eps, m->kpn));
            RC(mk_launch_f32_gemv(ctx, ly.kv_b, (int64_t)H * (nope + vd), kva, m->kpn, 1, m->kb, (int64_t)H * (nope + vd), 0));
            mla_assemble_kernel<<<(unsigned)mk_ceil_div((int64_t)H * (qh + vd), 256), 256, 0, st>>>(m->kb, y + qa + kva, H, nope, rope, vd, m->k_new, m->v_new, 0);
            ctx->launches++;
            const float scale = powf((float)qh, -0.5f);   // (mla_qh as f32).powf(-0.5) (src/model.rs:1977)
            const int strict_was = ctx->mla_strict;
            if (m->opts.strict) ctx->mla_strict = 1;      // the attention sums in the CPU's order as well
            rc = mk_mla_decode_step_dev(ctx, ly.cache, 0, m->k_new, m->v_new, m->q, scale, m->attn);
            ctx->mla_strict = strict_was;
            if (rc != MK_OK) return rc;
            RC(mk_sigmoid_gate_dev(ctx, m->attn, y + qa + cdim, hv));
            RC(mk_launch_f32_gemv(ctx, ly.o_proj, d, hv, m->attn, 1, m->attn_out, d, 0));
        } else {
            float *y = m->y;
            RC(mk_launch_f32_gemv(ctx, ly.w_x, ly.w_x_rows, d, m->x, 1, y, ly.w_x_rows, 0));          // q, k, v, g2, f_a, beta of x
            RC(mk_launch_f32_gemv(ctx, ly.f_b, proj, fa, y + 4 * proj, 1, m->g_low, proj, 0));
            RC(mk_kda_step_dev(ctx, ly.kda, y, y + proj, y + 2 * proj, m->g_low, y + 4 * proj + fa, y + 3 * proj, m->o));
            RC(mk_launch_f32_gemv(ctx, ly.o_proj, d, proj, m->o, 1, m->attn_out, d, 0));
        }
        // prefix2 = prefix + attn_out (or attn_out alone when the prefix became a block row), mix, rmsnorm -> x
        glue_kernel<<<1, 512, gsm_bytes, st>>>(m->attn_out, have_prefix ? m->hidden : nullptr, nullptr, m->p2, nullptr, m->blocks, nb, ly.mlp_w,
                                               ly.post_ln, eps, d, m->x, gstage, 0, 0);
        ctx->launches++;
        RC(tap(l, 0, m->attn_out));
        RC(tap(l, 1, m->p2));
        gc = nullptr;
        if (ly.is_moe) {
            if (m->ep) {
                RC(mk_moe_forward_ep_dev(ctx, ly.moe, m->ep, m->x, 1, m->mlp_out, nullptr, nullptr));
            } else {
                rc = mk_moe_forward_k3_split(ctx, ly.moe, m->x, m->mlp_out, m->sh_out);
                if (rc == MK_OK) gc = m->sh_out;          // added by the next glue launch: prefix2 + (routed + shared)
                else if (rc == MK_ERR_UNSUPPORTED) RC(mk_moe_forward_dev(ctx, ly.moe, m->x, 1, m->mlp_out, nullptr, nullptr));
                else return rc;
            }
        } else {
            const int di = (int)c.dense_inter;
            RC(mk_launch_f32_gemv(ctx, ly.dgu, 2 * di, d, m->x, 1, m->au, 2 * di, 0));
            RC(mk_launch_situ(ctx, m->au, m->au + di, di, m->act));
            RC(mk_launch_f32_gemv(ctx, ly.dd, d, di, m->act, 1, m->mlp_out, d, 0));
        }
        if (m->layer_hidden) {
            if (gc) {   // the tap shows the layer's FFN output as the engine forms it: routed + shared
                vec_add_kernel<<<(unsigned)mk_ceil_div(d, 256), 256, 0, st>>>(m->mlp_out, gc, m->res, d);
                ctx->launches++;
                RC(tap(l, 2, m->res));
            } else {
                RC(tap(l, 2, m->mlp_out));
            }
        }
        ga = m->p2; gb = m->mlp_out;
    }
    const int nb_final = m->layers.back().nb_before + (m->layers.back().pushes ? 1 : 0);
    glue_kernel<<<1, 512, gsm_bytes, st>>>(ga, gb, gc, m->hidden, nullptr, m->blocks, nb_final, m->out_w, m->norm_f, eps, d, m->x, gstage, 0, 0);
    ctx->launches++;
    RC(tap(c.n_layers - 1, 3, m->hidden));
    if (m->gather) {
        const float *full = nullptr;
        RC(mk_matvec_q8_gather_dev(ctx, m->head, m->gather, m->x, 1, m->head_row0, &full, m->next));
        MK_CUDA(cudaMemcpyAsync(m->logits, full, (size_t)c.vocab * 4, cudaMemcpyDeviceToDevice, st));
    } else {
        RC(mk_matvec_q8_dev(ctx, m->head, m->x, m->logits, 1, MK_ACT_Q8 | (m->opts.strict ? MK_ACT_STRICT : 0), m->next));
    }
#undef RC
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}


// Layer-major prefill of n tokens (Model::prefill_impl, src/model.rs:3097-3260, with the sequential recurrence of
// kda_prefill, src/model.rs:1291-1300, which the engine takes below its chunking threshold and calls bit-identical to
// kda_forward per position): per layer the projections, the FFN and the AttnRes glue run once for all tokens - every
// output row is the dot() of the single-token path, so batching changes no bit - while the KDA step and the MLA cache
// append + attention, which carry state from one position to the next, run token by token inside the layer.
// Leaves the caches as n single-token calls would, and logits / pick of the LAST token in m->logits / m->next.
int32_t ensure_prefill_buffers(mk_ctx *ctx, mk_model *m, int n) {
    if (n <= m->pf_cap) return MK_OK;
    const mk_model_config &c = m->cfg;
    const size_t d = c.d, proj = (size_t)c.kda_heads * c.kda_dim, H = c.mla_heads, qh = c.mla_nope + c.mla_rope, hv = H * c.mla_v;
    const size_t ywidth = std::max<size_t>(4 * proj + c.kda_fa + c.kda_heads, c.mla_qa + c.mla_kva + c.mla_rope + hv);
    int cap = m->pf_cap ? m->pf_cap : 16;
    while (cap < n) cap *= 2;
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    struct Want { float **p; size_t count; };
    const Want wants[] = {
        {&m->pf_hidden, d}, {&m->pf_x, d}, {&m->pf_attn_out, d}, {&m->pf_p2, d}, {&m->pf_mlp_out, d}, {&m->pf_embed, d},
        {&m->pf_blocks, (size_t)m->max_blocks * d}, {&m->pf_y, ywidth}, {&m->pf_g_low, proj}, {&m->pf_o, proj}, {&m->pf_fa, c.kda_fa},
        {&m->pf_qa, c.mla_qa}, {&m->pf_qan, c.mla_qa}, {&m->pf_q, H * qh}, {&m->pf_kva, c.mla_kva}, {&m->pf_kpn, c.mla_kva},
        {&m->pf_kb, H * (c.mla_nope + c.mla_v)}, {&m->pf_k_new, H * qh}, {&m->pf_v_new, hv}, {&m->pf_attn, hv},
        {&m->pf_au, 2 * (size_t)c.dense_inter}, {&m->pf_act, c.dense_inter},
    };
    for (const Want &w : wants) {
        if (*w.p) cudaFree(*w.p);
        *w.p = nullptr;
        MK_CUDA(cudaMalloc(w.p, std::max<size_t>(w.count, 1) * cap * sizeof(float)));
        MK_CUDA(cudaMemsetAsync(*w.p, 0, std::max<size_t>(w.count, 1) * cap * sizeof(float), ctx->stream));
    }
    if (m->pf_tok) cudaFree(m->pf_tok);
    m->pf_tok = nullptr;
    MK_CUDA(cudaMalloc(&m->pf_tok, (size_t)cap * sizeof(int32_t)));
    m->pf_cap = cap;
    return MK_OK;
}

int32_t enqueue_prefill(mk_ctx *ctx, mk_model *m, int n) {
    const mk_model_config &c = m->cfg;
    const int d = (int)c.d, proj = (int)(c.kda_heads * c.kda_dim), H = (int)c.mla_heads, nope = (int)c.mla_nope, rope = (int)c.mla_rope;
    const int vd = (int)c.mla_v, qh = nope + rope, qa = (int)c.mla_qa, kva = (int)c.mla_kva, cdim = kva + rope, hv = H * vd, fa = (int)c.kda_fa;
    const float eps = c.rms_eps;
    cudaStream_t st = ctx->stream;
    int32_t rc;
#define RC(call) do { rc = (call); if (rc != MK_OK) return rc; } while (0)
    const int64_t bstride = (int64_t)m->max_blocks * d;      // a token's AttnRes block rows
    const float *ga = m->pf_embed, *gb = nullptr;
    embed_rows_kernel<<<dim3((unsigned)mk_ceil_div(d, 256), (unsigned)n), 256, 0, st>>>(m->embed, m->pf_tok, (int)c.vocab, d, m->pf_embed, ctx->status_dev);
    ctx->launches++;
    const size_t gsm_plain = (size_t)(2 * d + m->max_blocks + 2) * 4, gsm_staged = (size_t)(2 * d + m->max_blocks + 8 + (size_t)m->max_blocks * d) * 4;
    const int gstage = gsm_staged <= 48 * 1024 ? 1 : 0;
    const size_t gsm_bytes = gstage ? gsm_staged : gsm_plain;
    // a strided slice [n][w] of the stacked projections (row stride ld) as contiguous rows
    auto slice = [&](float *dst, const float *src, int w, int64_t ld) -> int32_t {
        MK_CUDA(cudaMemcpy2DAsync(dst, (size_t)w * 4, src, (size_t)ld * 4, (size_t)w * 4, (size_t)n, cudaMemcpyDeviceToDevice, st));
        return MK_OK;
    };
    for (uint32_t l = 0; l < c.n_layers; ++l) {
        Layer &ly = m->layers[l];
        int nb = ly.nb_before;
        glue_kernel<<<(unsigned)n, 512, gsm_bytes, st>>>(ga, gb, nullptr, m->pf_hidden, ly.pushes ? m->pf_blocks + (size_t)nb * d : nullptr, m->pf_blocks, nb,
                                                       ly.sa_w, ly.input_ln, eps, d, m->pf_x, gstage, d, bstride);
        ctx->launches++;
        bool have_prefix = true;
        if (ly.pushes) { ++nb; have_prefix = false; }
        const int64_t ldy = ly.w_x_rows;
        float *y = m->pf_y;
        RC(mk_launch_f32_gemv(ctx, ly.w_x, ly.w_x_rows, d, m->pf_x, n, y, ldy, 0));
        if (ly.is_mla) {
            RC(slice(m->pf_qa, y, qa, ldy));
            RC(mk_launch_rmsnorm(ctx, m->pf_qa, ly.q_a_ln, n, qa, eps, m->pf_qan));
            RC(mk_launch_f32_gemv(ctx, ly.q_b, (int64_t)H * qh, qa, m->pf_qan, n, m->pf_q, (int64_t)H * qh, 0));
            RC(slice(m->pf_kva, y + qa, kva, ldy));
            RC(mk_launch_rmsnorm(ctx, m->pf_kva, ly.kv_a_ln, n, kva, eps, m->pf_kpn));
            RC(mk_launch_f32_gemv(ctx, ly.kv_b, (int64_t)H * (nope + vd), kva, m->pf_kpn, n, m->pf_kb, (int64_t)H * (nope + vd), 0));
            mla_assemble_kernel<<<dim3((unsigned)mk_ceil_div((int64_t)H * (qh + vd), 256), (unsigned)n), 256, 0, st>>>(
                m->pf_kb, y + qa + kva, H, nope, rope, vd, m->pf_k_new, m->pf_v_new, ldy);
            ctx->launches++;
            const float scale = powf((float)qh, -0.5f);
            const int strict_was = ctx->mla_strict;
            if (m->opts.strict) ctx->mla_strict = 1;
            // the n rows appended together, then every row's causal attention in shared launches
            rc = mk_mla_prefill_dev(ctx, ly.cache, 0, m->pf_k_new, m->pf_v_new, m->pf_q, n, scale, m->pf_attn);
            if (rc == MK_OK) {
                sigmoid_gate_rows_kernel<<<dim3((unsigned)mk_ceil_div(hv, 256), (unsigned)n), 256, 0, st>>>(m->pf_attn, y + qa + cdim, hv, ldy);
                ctx->launches++;
            }
            ctx->mla_strict = strict_was;
            if (rc != MK_OK) return rc;
            RC(mk_launch_f32_gemv(ctx, ly.o_proj, d, hv, m->pf_attn, n, m->pf_attn_out, d, 0));
        } else {
            RC(slice(m->pf_fa, y + 4 * proj, fa, ldy));
            RC(mk_launch_f32_gemv(ctx, ly.f_b, proj, fa, m->pf_fa, n, m->pf_g_low, proj, 0));
            // conv state and recurrence, position by position inside one launch (the state stays in registers)
            RC(mk_kda_steps_dev(ctx, ly.kda, n, y, y + proj, y + 2 * proj, m->pf_g_low, y + 4 * proj + fa, y + 3 * proj, m->pf_o, ldy, proj, proj));
            RC(mk_launch_f32_gemv(ctx, ly.o_proj, d, proj, m->pf_o, n, m->pf_attn_out, d, 0));
        }
        glue_kernel<<<(unsigned)n, 512, gsm_bytes, st>>>(m->pf_attn_out, have_prefix ? m->pf_hidden : nullptr, nullptr, m->pf_p2, nullptr, m->pf_blocks, nb,
                                                       ly.mlp_w, ly.post_ln, eps, d, m->pf_x, gstage, d, bstride);
        ctx->launches++;
        if (ly.is_moe) {
            RC(mk_moe_forward_dev(ctx, ly.moe, m->pf_x, n, m->pf_mlp_out, nullptr, nullptr));
        } else {
            const int di = (int)c.dense_inter;
            RC(mk_launch_f32_gemv(ctx, ly.dgu, 2 * di, d, m->pf_x, n, m->pf_au, 2 * di, 0));
            // gate rows and up rows of a token are the halves of its au row
            for (int t = 0; t < n; ++t) RC(mk_launch_situ(ctx, m->pf_au + (size_t)t * 2 * di, m->pf_au + (size_t)t * 2 * di + di, di, m->pf_act + (size_t)t * di));
            RC(mk_launch_f32_gemv(ctx, ly.dd, d, di, m->pf_act, n, m->pf_mlp_out, d, 0));
        }
        ga = m->pf_p2; gb = m->pf_mlp_out;
    }
    // the last token alone: final AttnRes mix + norm, lm_head, pick
    const int nb_final = m->layers.back().nb_before + (m->layers.back().pushes ? 1 : 0);
    const size_t last = (size_t)(n - 1);
    glue_kernel<<<1, 512, gsm_bytes, st>>>(ga + last * d, gb + last * d, nullptr, m->hidden, nullptr, m->pf_blocks + last * bstride, nb_final, m->out_w,
                                           m->norm_f, eps, d, m->x, gstage, 0, 0);
    ctx->launches++;
    RC(mk_matvec_q8_dev(ctx, m->head, m->x, m->logits, 1, MK_ACT_Q8 | (m->opts.strict ? MK_ACT_STRICT : 0), m->next));
#undef RC
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

} // namespace

extern "C" int32_t mk_model_forward_dev(mk_ctx *ctx, mk_model *m, const int32_t *token, float *logits, int32_t *next) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr, "NULL argument");
    if (m->positions + 1 > m->opts.max_positions) {
        mk_set_error("mk_model_forward: the sequence already holds max_positions = %d tokens", m->opts.max_positions);
        return MK_ERR_STATE;
    }
    MK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    // the token of this step: the caller's, or the pick the previous step left on the device
    copy_i32_kernel<<<1, 1, 0, st>>>(token ? token : m->next, m->tok);
    ctx->launches++;
    // a CUDA graph cannot be recorded from the legacy default stream: there the token is launched kernel by kernel
    const bool real_stream = st != nullptr && st != cudaStreamLegacy && st != cudaStreamPerThread;
    const bool graph_ok = m->opts.use_graph && !ctx->prof_on && real_stream;
    int32_t rc = MK_OK;
    if (m->graph_ws != ctx->ws || m->graph_epoch != ctx->alloc_epoch) {
        // since the token was recorded another call on this context grew the shared workspace, or a layer re-allocated its
        // per-call buffers (a prompt chunk longer than any before): the recorded launches point at freed memory, so
        // the recordings are dropped and made again
        for (cudaGraphExec_t &g : m->graphs) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
    }
    const uint32_t ep0 = m->ep ? mk_moe_ep_steps(m->ep) : 0u, ga0 = m->gather ? mk_gather_steps(m->gather) : 0u;
    cudaGraphExec_t &graph = m->graphs[(ep0 & 1u) * 2 + (ga0 & 1u)];
    if (graph_ok && graph) {
        MK_CUDA(cudaGraphLaunch(graph, st));
        ctx->launches += m->launches_per_token;
        for (Layer &ly : m->layers) if (ly.cache) mk_mla_note_replay(ly.cache, 0);
        if (m->ep) mk_moe_ep_note_replay(m->ep, m->ep_steps_per_token);
        if (m->gather) mk_gather_note_replay(m->gather, m->gather_steps_per_token);
    } else if (graph_ok && m->warm >= 1) {
        // the first token ran eagerly (workspaces grown, attributes set); this one is recorded and then launched
        const int64_t l0 = ctx->launches;
        cudaGraph_t g = nullptr;
        MK_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
        rc = enqueue_token(ctx, m);
        const cudaError_t e = cudaStreamEndCapture(st, &g);
        if (rc != MK_OK || e != cudaSuccess) {
            if (g) cudaGraphDestroy(g);
            if (rc == MK_OK) { mk_set_error("mk_model_forward: graph capture failed: %s", cudaGetErrorString(e)); rc = MK_ERR_CUDA; }
            return rc;
        }
        m->launches_per_token = ctx->launches - l0;
        m->ep_steps_per_token = m->ep ? mk_moe_ep_steps(m->ep) - ep0 : 0u;
        m->gather_steps_per_token = m->gather ? mk_gather_steps(m->gather) - ga0 : 0u;
        const cudaError_t e2 = cudaGraphInstantiate(&graph, g, 0);
        cudaGraphDestroy(g);
        if (e2 != cudaSuccess) { mk_set_error("mk_model_forward: graph instantiation failed: %s", cudaGetErrorString(e2)); return MK_ERR_CUDA; }
        m->graph_ws = ctx->ws;
        m->graph_epoch = ctx->alloc_epoch;
        MK_CUDA(cudaGraphLaunch(graph, st));
    } else {
        const int64_t l0 = ctx->launches;
        rc = enqueue_token(ctx, m);
        if (rc != MK_OK) return rc;
        m->launches_per_token = ctx->launches - l0;
        m->warm++;
    }
    m->positions++;
    if (logits) MK_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToDevice, st));
    if (next) { copy_i32_kernel<<<1, 1, 0, st>>>(m->next, next); ctx->launches++; }
    MK_CUDA(cudaGetLastError());
    return MK_OK;
}

extern "C" int32_t mk_model_forward(mk_ctx *ctx, mk_model *m, int32_t token, float *logits, int32_t *next) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr, "NULL argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    int32_t rc = mk_io_reserve(ctx, 256);
    if (rc != MK_OK) return rc;
    int32_t *tdev = (int32_t *)ctx->io_dev;
    MK_CUDA(cudaMemcpyAsync(tdev, &token, 4, cudaMemcpyHostToDevice, ctx->stream));
    rc = mk_model_forward_dev(ctx, m, tdev, nullptr, nullptr);
    if (rc != MK_OK) return rc;
    if (logits) MK_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (next) MK_CUDA(cudaMemcpyAsync(next, m->next, 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}


extern "C" int32_t mk_model_prefill(mk_ctx *ctx, mk_model *m, const int32_t *tokens, int32_t n, float *logits, int32_t *next) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && tokens != nullptr && n >= 1, "bad argument");
    if (m->positions + n > m->opts.max_positions) {
        mk_set_error("mk_model_prefill: %d tokens on top of %d exceed max_positions = %d", n, m->positions, m->opts.max_positions);
        return MK_ERR_STATE;
    }
    MK_CUDA(cudaSetDevice(ctx->device));
    int32_t rc = MK_OK;
    if (m->world > 1 || m->layer_hidden) {
        // expert-parallel models and models that keep per-layer taps take the tokens one by one
        for (int i = 0; i < n && rc == MK_OK; ++i) rc = mk_model_forward(ctx, m, tokens[i], i == n - 1 ? logits : nullptr, i == n - 1 ? next : nullptr);
        return rc;
    }
    const int chunk_max = 256;
    for (int i0 = 0; i0 < n; i0 += chunk_max) {
        const int nc = std::min(chunk_max, n - i0);
        rc = ensure_prefill_buffers(ctx, m, nc);
        if (rc != MK_OK) return rc;
        MK_CUDA(cudaMemcpyAsync(m->pf_tok, tokens + i0, (size_t)nc * 4, cudaMemcpyHostToDevice, ctx->stream));
        rc = enqueue_prefill(ctx, m, nc);
        if (rc != MK_OK) return rc;
        m->positions += nc;
        MK_CUDA(cudaStreamSynchronize(ctx->stream));      // the token ids came from pageable host memory
    }
    if (logits) MK_CUDA(cudaMemcpyAsync(logits, m->logits, (size_t)m->cfg.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
    if (next) MK_CUDA(cudaMemcpyAsync(next, m->next, 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_model_generate(mk_ctx *ctx, mk_model *m, const int32_t *prompt, int32_t n_prompt, int32_t n_new, int32_t *out_tokens) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && prompt != nullptr && n_prompt >= 1 && n_new >= 0 && (n_new == 0 || out_tokens != nullptr),
                 "bad argument");
    MK_CHECK_ARG(m->positions + n_prompt + n_new - (n_new > 0 ? 1 : 0) <= m->opts.max_positions, "prompt + new tokens exceed max_positions");
    MK_CUDA(cudaSetDevice(ctx->device));
    int32_t rc = mk_io_reserve(ctx, mk_align_up((size_t)(n_prompt + n_new) * 4, 256));
    if (rc != MK_OK) return rc;
    int32_t *pdev = (int32_t *)ctx->io_dev, *odev = pdev + n_prompt;
    MK_CUDA(cudaMemcpyAsync(pdev, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (m->world == 1 && !m->layer_hidden && n_prompt > 1) {
        // the prompt layer by layer (enqueue_prefill); the pick after its last token is the first new token
        const int chunk_max = 256;
        for (int i0 = 0; i0 < n_prompt; i0 += chunk_max) {
            const int nc = std::min(chunk_max, n_prompt - i0);
            rc = ensure_prefill_buffers(ctx, m, nc);
            if (rc != MK_OK) return rc;
            MK_CUDA(cudaMemcpyAsync(m->pf_tok, pdev + i0, (size_t)nc * 4, cudaMemcpyDeviceToDevice, ctx->stream));
            rc = enqueue_prefill(ctx, m, nc);
            if (rc != MK_OK) return rc;
            m->positions += nc;
        }
        if (n_new > 0) { copy_i32_kernel<<<1, 1, 0, ctx->stream>>>(m->next, odev); ctx->launches++; }
    } else {
        // prompt tokens one by one (expert-parallel models, models that keep per-layer taps)
        for (int i = 0; i < n_prompt; ++i) {
            rc = mk_model_forward_dev(ctx, m, pdev + i, nullptr, (i == n_prompt - 1 && n_new > 0) ? odev : nullptr);
            if (rc != MK_OK) return rc;
        }
    }
    for (int i = 1; i < n_new; ++i) {
        rc = mk_model_forward_dev(ctx, m, nullptr, nullptr, odev + i);
        if (rc != MK_OK) return rc;
    }
    if (n_new > 0) MK_CUDA(cudaMemcpyAsync(out_tokens, odev, (size_t)n_new * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_model_layer_hidden(mk_ctx *ctx, mk_model *m, float *out) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && out != nullptr, "NULL argument");
    MK_CHECK_ARG(m->layer_hidden != nullptr, "the model was opened without keep_layer_hidden");
    MK_CUDA(cudaSetDevice(ctx->device));
    MK_CUDA(cudaMemcpyAsync(out, m->layer_hidden, (size_t)m->cfg.n_layers * 4 * m->cfg.d * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}

extern "C" int32_t mk_model_last_hidden(mk_ctx *ctx, mk_model *m, float *hidden) {
    MK_CHECK_ARG(ctx != nullptr && m != nullptr && hidden != nullptr, "NULL argument");
    MK_CUDA(cudaSetDevice(ctx->device));
    MK_CUDA(cudaMemcpyAsync(hidden, m->x, (size_t)m->cfg.d * 4, cudaMemcpyDeviceToHost, ctx->stream));
    MK_CUDA(cudaStreamSynchronize(ctx->stream));
    return MK_OK;
}
