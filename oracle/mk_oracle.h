/*
 * CPU oracle for the quantized decode hot path of microkimi.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * CPU arithmetic (Rust sources, cited per function as file:line relative to the
 * reference project).  It exists so the CUDA kernels can be checked against the
 * reference's own numbers and so a CPU baseline can be timed beside the GPU.
 * Nothing in the shipped product path may call into it.
 *
 * Every function keeps the reference's operation ORDER (mul then add, never a
 * fused multiply-add; fixed reduction trees) - build with -ffp-contract=off.
 */
#ifndef MK_ORACLE_H
#define MK_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- build.rs RNG (src/build.rs:21-51) ---- */
typedef struct { uint64_t s; } or_rng;
void     or_rng_for_tensor(or_rng *r, const char *name);
uint64_t or_rng_next_u64(or_rng *r);
double   or_rng_uniform(or_rng *r);
float    or_rng_gauss(or_rng *r);
void     or_rng_fill_gauss(const char *name, float sigma, float *out, size_t n);

/* ---- MXFP4 (src/mxfp4.rs) ---- */
float or_exp2_i(int e);                                   /* mxfp4.rs:10-16  */
float or_scale_from_byte(uint8_t sb);                     /* mxfp4.rs:340-346 */
void  or_mxfp4_dequant(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols, float *out); /* :19-31 */
void  or_mxfp4_quantize(const float *w, size_t rows, size_t cols, int search, uint8_t *packed, uint8_t *scales); /* :38-138 */
void  or_mxfp4_matvec_f32(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                          const float *x, float *out, int n_threads);                    /* :488-539 */
void  or_mxfp4_matvec_q8(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                         const int8_t *xq, const float *xs, float *out, int n_threads);  /* :405-443 */
void  or_mxfp4_matvec(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                      const float *x, float *out, int n_threads, int use_q8);            /* :458-539 */
void  or_mxfp4_matvec_shader_emul(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                                  const float *x, float *out, size_t lanes);             /* :357-393 */
/* model.rs:2412-2447: batched order, xt = [cols*m] transposed, out = [m*rows] */
void  or_mxfp4_matvec_nt(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols,
                         const float *xt, size_t m, float *out);

/* ---- q8_0 (src/q8.rs) ---- */
void    or_q8_quantize(const float *x, size_t n, int8_t *q, float *scales);  /* q8.rs:49-69 */
int32_t or_block_dot(const uint8_t *packed16, const int8_t *x32);            /* q8.rs:194-202 */
int32_t or_block_dot_i8(const int8_t *w32, const int8_t *x32);               /* q8.rs:119-125 */

/* ---- f32 kernels (src/model.rs) ---- */
float or_dot(const float *a, const float *b, size_t n);                      /* model.rs:63-82 */
void  or_matvec_f32(const float *w, size_t rows, size_t cols, const float *x, float *out, int n_threads); /* :199-247 */
void  or_rmsnorm(const float *x, const float *w, size_t n, float eps, float *out); /* :599-605 */
float or_sigmoid(float x);                                                   /* :607-610 */
float or_situ(float g, float u);                                             /* :617-621 */
int   or_argmax(const float *v, size_t n);                                   /* :3271-3291 (first strict maximum) */

/* ---- q8_0 lm_head (model.rs:261-348) ---- */
void or_q8head_from_f32(const float *w, size_t rows, size_t cols, int8_t *q, float *scales);
void or_q8head_matvec(const int8_t *q, const float *scales, size_t rows, size_t cols,
                      const float *x, float *out, int n_threads);
/* variant with the weight scales rounded to IEEE half before use (layout the
 * benchmark spec words as "f16 scales"; no counterpart in the reference). */
void or_q8head_from_f32_f16s(const float *w, size_t rows, size_t cols, int8_t *q, uint16_t *scales_h);
void or_q8head_matvec_f16s(const int8_t *q, const uint16_t *scales_h, size_t rows, size_t cols,
                           const float *x, float *out, int n_threads);

/* ---- routers ---- */
/* K3 noaux_tc router (model.rs:2153-2173): ids/weights in final slot order. */
void or_router_k3(const float *gate_w, const float *gate_b, size_t n_experts, size_t d, size_t top_k,
                  const float *x, int32_t *ids, float *weights, float *logits_out /* nullable */);
/* DeepSeek sqrtsoftplus gate (deepseek.rs:16-58), no hash routing. */
void or_gate_ds(const float *gate_w, const float *bias /* nullable */, size_t n_experts, size_t d, size_t top_k,
                float route_scale, const float *x, int32_t *ids, float *weights);

/* ---- experts ---- */
/* deepseek.rs:74-95 : f32 SwiGLU-clamp expert. */
void or_expert_ds_f32(const float *w1, const float *w2, const float *w3, const float *x,
                      size_t d, size_t inter, float limit, float *out);

typedef struct {
    size_t d, inter, n_experts, top_k;
    float  limit;                 /* swiglu clamp (deepseek.rs:1082) */
    int    use_q8;                /* 1: matvec_packed default path; 0: exact f32 path */
    const float   *gate_w;        /* [n_experts, d] */
    const float   *gate_b;        /* [n_experts] */
    /* routed experts: expert e, matrix m in {0:w1,1:w2,2:w3}: packed at
     * packed[(e*3+m)] (pointer table), scales likewise */
    const uint8_t *const *packed; /* [n_experts*3] */
    const uint8_t *const *scales; /* [n_experts*3] */
    /* one shared expert, MXFP4 (w1,w2,w3) */
    const uint8_t *sh_packed[3];
    const uint8_t *sh_scales[3];
} or_moe_ds_desc;
/* K3 router (model.rs:2153-2173) feeding the DeepSeek expert body
 * (deepseek.rs:1038-1108): routing weight folded into the activation before w2,
 * outputs summed in slot order, plus one unweighted shared expert. One token. */
void or_moe_ds_forward(const or_moe_ds_desc *m, const float *x, float *out,
                       int32_t *ids_out /* [top_k], nullable */, float *w_out /* nullable */, int n_threads);

/* ---- MXFP4SQ (src/mxfp4.rs:140-240): the scale byte decodes as ((q + 1) / 256)^2 * smax ---- */
float or_scale_sq(uint8_t q, float smax);
float or_mxfp4sq_quantize(const float *w, size_t rows, size_t cols, uint8_t *packed, uint8_t *scales); /* returns smax */
void  or_mxfp4sq_dequant(const uint8_t *packed, const uint8_t *scales, float smax, size_t rows, size_t cols, float *out);

/* ---- FP8 e4m3fn + ue8m0 (128 x 128 blocks) dequant (dequant.rs:10-41) ---- */
float or_e4m3_to_f32(uint8_t b);
void or_dequant_fp8(const uint8_t *w, const uint8_t *scales, size_t rows, size_t cols, float *out);

/* ---- VQ1 codebook matvec (quant.rs:313-346, lutgemv.rs:208-238) ----
 * codebook f32 [256][16]; indices u8 [rows][cols/16]: W[r, 16v + j] = codebook[idx[r][v]][j].
 * gather: out[r] = sum over v (ascending) of s_v, s_v = sum over j (ascending) of cb[idx][j] * x[16v + j],
 * every sum starting from 0 with a separate multiply and add.  lut: one table of 256 such dots per group,
 * then additions only; bit-identical to gather (lutgemv.rs:22-27). */
void or_matvec_vq_gather(const float *codebook, const uint8_t *indices, size_t rows, size_t cols, const float *x, float *out);
void or_matvec_vq_lut(const float *codebook, const uint8_t *indices, size_t rows, size_t cols, const float *x, float *out);

/* K3 latent MoE layer (model.rs:2150-2380), one token: router on x [d]; h = routed_down x;
 * per selected expert a = w1 h, u = w3 h, act = situ(a, u), o = w2 act (MXFP4 experts over
 * the latent width rh); y = sum of w_i * o_i in slot order; out = routed_up rmsnorm(y) plus
 * the f32 shared expert (SiTU MLP on x). */
typedef struct {
    size_t d, rh, inter, n_experts, top_k, shared_inter;
    float rms_eps;
    int use_q8;
    const float *gate_w;       /* [n_experts][d] */
    const float *gate_b;       /* [n_experts] */
    const float *routed_down;  /* [rh][d] */
    const float *routed_norm;  /* [rh] */
    const float *routed_up;    /* [d][rh] */
    const float *shared_gate;  /* [shared_inter][d], NULL = no shared expert */
    const float *shared_up;    /* [shared_inter][d] */
    const float *shared_down;  /* [d][shared_inter] */
    const uint8_t *const *packed; /* [n_experts*3] w1 [inter x rh], w2 [rh x inter], w3 [inter x rh] */
    const uint8_t *const *scales;
} or_moe_k3_desc;
void or_moe_k3_forward(const or_moe_k3_desc *m, const float *x, float *out,
                       int32_t *ids_out /* [top_k], nullable */, float *w_out /* nullable */);

/* ---- MLA q8_0 cache, reference per-head layout (model.rs:765-781) ---- */
typedef struct {
    size_t nh, nope, rope, vd;
    size_t n;       /* positions held */
    size_t cap;
    int8_t *kq;     /* [n][nh][nope] */
    float  *ks;     /* [n][nh][nope/32] */
    float  *kr;     /* [n][rope] */
    int8_t *vq;     /* [n][nh][vd] */
    float  *vs;     /* [n][nh][vd/32] */
} or_mla_cache;
or_mla_cache *or_mla_new(size_t nh, size_t nope, size_t rope, size_t vd, size_t cap);
void or_mla_free(or_mla_cache *c);
void or_mla_push(or_mla_cache *c, const float *k_row, const float *v_row);             /* :1583-1618 (no Hadamard) */
void or_mla_to_f32(const or_mla_cache *c, float *k, float *v);                         /* :1623-1676 */
void or_mla_attn_flash_q8(const or_mla_cache *c, const float *qh, size_t h, size_t pos, float scale, float *oh); /* :1706-1786 */
void or_mla_attn_flash_q8_mqa(const or_mla_cache *c, const float *q, size_t pos, float scale, float *attn);      /* :1804-1908 */
void or_mla_attn_ref_q8(const or_mla_cache *c, const float *qh, size_t h, size_t pos, float scale, float *oh);   /* :1914-1937 */
/* f32-cache kernels (model.rs:1353-1500) used by the reference's own A/B tests */
void or_mla_attn_ref_f32(const float *k, const float *v, size_t nh, size_t hd, size_t vd,
                         const float *qh, size_t h, size_t pos, float scale, float *oh);
void or_mla_attn_flash_f32(const float *k, const float *v, size_t nh, size_t hd, size_t vd,
                           const float *qh, size_t h, size_t pos, float scale, float *oh);

/* ---- MLA q8_0 cache, absorbed shared-latent layout (no reference function:
 *      the per-position recipe of model.rs:1833-1890 applied to ONE q8 row of
 *      width `lat` (= kv_lora + rope) shared by all heads; V = first `vd`
 *      columns of the same row). ---- */
typedef struct {
    size_t lat, vd, n, cap;
    int8_t *q;      /* [n][lat] */
    float  *s;      /* [n][lat/32] */
} or_mla_abs_cache;
or_mla_abs_cache *or_mla_abs_new(size_t lat, size_t vd, size_t cap);
void or_mla_abs_free(or_mla_abs_cache *c);
void or_mla_abs_push(or_mla_abs_cache *c, const float *row);
void or_mla_abs_attn(const or_mla_abs_cache *c, const float *q /* [nh][lat] */, size_t nh,
                     size_t pos, float scale, float *out /* [nh][vd] */);
/* f64 dense-softmax check of the same quantities (dequantized cache, f32 query). */
void or_mla_abs_attn_f64(const or_mla_abs_cache *c, const float *q, size_t nh,
                         size_t pos, float scale, double *out);

/* IEEE half helpers (round-to-nearest-even), used only by the f16-scale variant */
/* ---- KDA decode step and AttnRes (src/model.rs:1066-1177, 625-669; src/selftest.rs:48-113) ---- */
/* conv window: kconv - 1 previous raw inputs [j][proj] (oldest first); vec is replaced by silu(conv) */
void or_kda_conv_step(size_t proj, size_t kconv, const float *w_conv /* [proj][kconv] */, float *vec, float *cache_raw); /* :1070-1085 */
void or_kda_norm_head(size_t heads, size_t dim, float *vec, float scale);                                             /* :1088-1097 */
void or_kda_gate(size_t heads, size_t dim, float gate_lb, const float *a_log, const float *dt_bias, const float *g_low, float *g); /* :1100-1109 */
void or_kda_recur_step(size_t heads, size_t dim, float *s, const float *q, const float *k, const float *v, const float *g,
                       const float *beta, float *o);                                                                  /* :1114-1156 */
void or_kda_gated_onorm(size_t heads, size_t dim, float eps, float *o, const float *o_norm, const float *g2);         /* :1167-1176 */
/* kda_forward between its projections and o_proj (:1203-1228): raw q, k, v, g_low, beta, g2 in; o [heads*dim] out */
typedef struct {
    size_t heads, dim, kconv;
    float gate_lb, rms_eps;
    const float *q_conv, *k_conv, *v_conv; /* [heads*dim][kconv] */
    const float *a_log, *dt_bias, *o_norm; /* [dim], [heads*dim], [dim] */
} or_kda_desc;
void or_kda_step(const or_kda_desc *d, float *conv_q, float *conv_k, float *conv_v /* [(kconv-1)][proj] each */, float *s,
                 const float *q_raw, const float *k_raw, const float *v_raw, const float *g_low, const float *beta_raw,
                 const float *g2, float *o);
/* the selftest's standalone recurrence on raw inputs (selftest.rs:48-113): o [T][H][dim], s [H][dim][dim] (zeroed here) */
void or_kda_core(const float *q, const float *k, const float *v, const float *g, const float *beta, const float *a_log,
                 const float *dt_bias, size_t t_steps, size_t heads, size_t dim, float *o, float *s);
void or_attn_res(size_t d, float eps, const float *prefix, const float *blocks /* [b][d] */, size_t b, const float *w, float *out); /* :632-669 */

uint16_t or_f32_to_f16(float f);
float    or_f16_to_f32(uint16_t h);

/* ---- the whole decode token (mk_oracle_model.c) -------------------------------------------
 * Config (src/config.rs:8-43; explicit layer lists are not supported), the MKIM0001/2 container
 * (src/weights.rs), `microkimi build` with every tensor on its Gaussian fallback branch
 * (src/build.rs:344-576) and Model::forward (src/model.rs:2889-3031). */
typedef struct {
    uint32_t n_layers, d, vocab, n_experts, top_k, n_shared;
    uint32_t kda_heads, kda_dim, kda_conv, kda_fa;
    float    gate_lb;
    uint32_t mla_heads, mla_qa, mla_kva, mla_nope, mla_rope, mla_v;
    uint32_t routed_hidden, moe_inter, shared_inter, dense_inter, attn_res_block, first_k_dense;
    float    rms_eps;
    uint32_t eos_id, bos_id;
} or_config;
void or_config_microkimi(or_config *c);
int  or_config_is_mla(const or_config *c, uint32_t l);
int  or_config_is_moe(const or_config *c, uint32_t l);
/* writes the synthetic model file; 0 on success */
int  or_build_bin(const char *path, const or_config *c);
typedef struct or_bin or_bin;
or_bin *or_bin_open(const char *path);
void or_bin_close(or_bin *b);
const or_config *or_bin_config(const or_bin *b);
size_t or_bin_count(const or_bin *b);
/* tensor by name: data pointer (NULL if absent), dtype (0 f32, 1 mxfp4), dims2 = {rows, cols or 0}, blob size */
const void *or_bin_get(const or_bin *b, const char *name, uint8_t *dtype, uint32_t *dims2, uint64_t *size);
int or_bin_entry(const or_bin *b, size_t i, const char **name, uint8_t *dtype, uint32_t *dims2, uint64_t *off, uint64_t *size);
typedef struct or_model or_model;
or_model *or_model_open(const char *path, size_t max_positions, int n_threads);
void or_model_free(or_model *m);
void or_model_reset(or_model *m);
const or_config *or_model_config(const or_model *m);
/* one token: logits [vocab] (nullable), hidden_out [d] (nullable) = the normed state fed to the lm_head; 0 on success */
int or_model_forward(or_model *m, uint32_t token, float *logits, float *hidden_out);
/* the same, also returning per layer [attention output, residual after it, FFN output, residual after the layer]:
 * layer_out [n_layers][4][d] (nullable) */
int or_model_forward_layers(or_model *m, uint32_t token, float *logits, float *hidden_out, float *layer_out);

/* 1: exp / tanh / log taken in double precision and rounded once instead of the f32 libm calls (see mk_oracle.c) */
void or_set_cr_math(int on);
float or_m_expf(float x);
float or_m_tanhf(float x);
float or_m_logf(float x);
int or_num_threads(void);
void or_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
