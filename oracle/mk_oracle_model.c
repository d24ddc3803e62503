/*
 * CPU oracle, part 2: the whole decode token of the K3 engine.
 * TEST INFRASTRUCTURE ONLY - see mk_oracle.h.  Citations are file:line of the
 * reference project (Rust).
 *
 *   or_config_*      Config::microkimi / Config::from_json         src/config.rs:47-138
 *   or_bin_*         the MKIM0001/2 container (reader and writer)  src/weights.rs:1-64, 107-186, 390-468
 *   or_build_bin     `microkimi build`, every tensor on its Gaussian fallback branch
 *                    (no downloaded pools)                          src/build.rs:319-335, 344-576
 *   or_model_*       Model::from_bin, Model::forward and the blocks it calls
 *                    (kda_forward, mla_forward, dense_forward; moe_forward is
 *                    or_moe_k3_forward)                             src/model.rs:906-1025, 1179-1232, 1939-2022,
 *                                                                   2382-2396, 2889-3031
 */
#define _GNU_SOURCE
#include "mk_oracle.h"

#include <fcntl.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ config */
void or_config_microkimi(or_config *c) { /* config.rs:47-79 */
    memset(c, 0, sizeof(*c));
    c->n_layers = 93; c->d = 512; c->vocab = 163840; c->n_experts = 896; c->top_k = 16; c->n_shared = 2;
    c->kda_heads = 4; c->kda_dim = 128; c->kda_conv = 4; c->kda_fa = 128; c->gate_lb = -5.0f;
    c->mla_heads = 4; c->mla_qa = 128; c->mla_kva = 64; c->mla_nope = 128; c->mla_rope = 64; c->mla_v = 128;
    c->routed_hidden = 128; c->moe_inter = 64; c->shared_inter = 128; c->dense_inter = 2048;
    c->attn_res_block = 12; c->first_k_dense = 1; c->rms_eps = 1e-5f; c->eos_id = 163586; c->bos_id = 163584;
}
int or_config_is_mla(const or_config *c, uint32_t l) { return l % 4 == 3 || l == c->n_layers - 1; } /* config.rs:127-132 */
int or_config_is_moe(const or_config *c, uint32_t l) { return l >= c->first_k_dense; }               /* config.rs:133-138 */

/* Number that follows "key": anywhere in the JSON text (the config block is flat apart from "specials",
 * whose keys do not collide with the top-level ones). */
static int json_num(const char *js, size_t n, const char *key, double *out) {
    char pat[96];
    const int pl = snprintf(pat, sizeof(pat), "\"%s\"", key);
    for (size_t i = 0; i + (size_t)pl < n; ++i) {
        if (memcmp(js + i, pat, (size_t)pl) != 0) continue;
        size_t j = i + (size_t)pl;
        while (j < n && (js[j] == ' ' || js[j] == '\t' || js[j] == '\n' || js[j] == '\r')) ++j;
        if (j >= n || js[j] != ':') continue;
        ++j;
        char buf[64];
        size_t k = 0;
        while (j < n && k + 1 < sizeof(buf) && (js[j] == ' ' || js[j] == '\t')) ++j;
        while (j < n && k + 1 < sizeof(buf) && (strchr("+-0123456789.eE", js[j]) != NULL)) buf[k++] = js[j++];
        buf[k] = 0;
        if (k == 0) return 0;
        *out = strtod(buf, NULL);
        return 1;
    }
    return 0;
}
static void config_from_json(or_config *c, const char *js, size_t n) { /* config.rs:86-125 (explicit layer lists not supported) */
    or_config_microkimi(c);
    double v;
#define NUM(key, field, type) if (json_num(js, n, key, &v)) c->field = (type)v
    NUM("n_layers", n_layers, uint32_t); NUM("hidden", d, uint32_t); NUM("vocab", vocab, uint32_t);
    NUM("n_experts", n_experts, uint32_t); NUM("top_k", top_k, uint32_t); NUM("n_shared", n_shared, uint32_t);
    NUM("kda_heads", kda_heads, uint32_t); NUM("kda_dim", kda_dim, uint32_t); NUM("kda_conv", kda_conv, uint32_t);
    NUM("kda_fa_rank", kda_fa, uint32_t); NUM("gate_lower_bound", gate_lb, float);
    NUM("mla_heads", mla_heads, uint32_t); NUM("mla_q_lora", mla_qa, uint32_t); NUM("mla_kv_lora", mla_kva, uint32_t);
    NUM("mla_nope", mla_nope, uint32_t); NUM("mla_rope", mla_rope, uint32_t); NUM("mla_v", mla_v, uint32_t);
    NUM("routed_hidden", routed_hidden, uint32_t); NUM("moe_inter", moe_inter, uint32_t);
    NUM("shared_inter", shared_inter, uint32_t); NUM("dense_inter", dense_inter, uint32_t);
    NUM("attn_res_block", attn_res_block, uint32_t); NUM("first_k_dense", first_k_dense, uint32_t);
    NUM("rms_eps", rms_eps, float); NUM("end_of_msg", eos_id, uint32_t); NUM("bos", bos_id, uint32_t);
#undef NUM
}
static int config_to_json(const or_config *c, char *buf, size_t cap) {
    return snprintf(buf, cap,
        "{\"n_layers\":%u,\"hidden\":%u,\"vocab\":%u,\"n_experts\":%u,\"top_k\":%u,\"n_shared\":%u,\"kda_heads\":%u,"
        "\"kda_dim\":%u,\"kda_conv\":%u,\"kda_fa_rank\":%u,\"gate_lower_bound\":%.9g,\"mla_heads\":%u,\"mla_q_lora\":%u,"
        "\"mla_kv_lora\":%u,\"mla_nope\":%u,\"mla_rope\":%u,\"mla_v\":%u,\"routed_hidden\":%u,\"moe_inter\":%u,"
        "\"shared_inter\":%u,\"dense_inter\":%u,\"attn_res_block\":%u,\"first_k_dense\":%u,\"rms_eps\":%.9g,"
        "\"specials\":{\"end_of_msg\":%u,\"bos\":%u}}",
        c->n_layers, c->d, c->vocab, c->n_experts, c->top_k, c->n_shared, c->kda_heads, c->kda_dim, c->kda_conv, c->kda_fa,
        (double)c->gate_lb, c->mla_heads, c->mla_qa, c->mla_kva, c->mla_nope, c->mla_rope, c->mla_v, c->routed_hidden,
        c->moe_inter, c->shared_inter, c->dense_inter, c->attn_res_block, c->first_k_dense, (double)c->rms_eps, c->eos_id,
        c->bos_id);
}

/* ------------------------------------------------------------------ the container: writer (weights.rs:66-186) */
enum { DT_F32 = 0, DT_MXFP4 = 1 };
typedef struct { char name[128]; uint8_t dtype; uint8_t nd; uint32_t dims[2]; uint64_t off, size; } dir_ent;
typedef struct { dir_ent *e; size_t n, cap; } dir_list;

static uint64_t blob_size(uint8_t dtype, const uint32_t *dims, int nd) { /* weights.rs:40-64 */
    uint64_t n = 1;
    for (int i = 0; i < nd; ++i) n *= dims[i];
    if (dtype == DT_F32) return n * 4;
    return (uint64_t)dims[0] * dims[1] / 2 + (uint64_t)dims[0] * dims[1] / 32;
}
static int is_expert_tensor(const char *name) { /* weights.rs:417-419 */
    const size_t l = strlen(name);
    return strstr(name, ".block_sparse_moe.experts.") != NULL && l > 3 &&
           (strcmp(name + l - 3, ".w1") == 0 || strcmp(name + l - 3, ".w2") == 0 || strcmp(name + l - 3, ".w3") == 0);
}
static void dir_add(dir_list *d, const char *name, uint8_t dtype, uint32_t d0, uint32_t d1) {
    if (d->n == d->cap) {
        d->cap = d->cap ? d->cap * 2 : 1024;
        d->e = (dir_ent *)realloc(d->e, d->cap * sizeof(dir_ent));
    }
    dir_ent *e = &d->e[d->n++];
    memset(e, 0, sizeof(*e));
    snprintf(e->name, sizeof(e->name), "%.127s", name);
    e->dtype = dtype;
    e->nd = d1 ? 2 : 1;
    e->dims[0] = d0; e->dims[1] = d1;
    e->size = blob_size(dtype, e->dims, e->nd);
}
static void dir_layout(dir_list *d, uint64_t prefix) { /* weights.rs:107-131 */
    uint64_t dir_size = 0;
    for (size_t i = 0; i < d->n; ++i) dir_size += 2 + strlen(d->e[i].name) + 1 + 1 + 4 * (uint64_t)d->e[i].nd + 8 + 8;
    uint64_t pos = prefix + 4 + dir_size;
    for (size_t i = 0; i < d->n; ++i) {
        const uint64_t align = is_expert_tensor(d->e[i].name) ? 4096 : 64;
        pos = (pos + align - 1) / align * align;
        d->e[i].off = pos;
        pos += d->e[i].size;
    }
}
static const dir_ent *dir_find_linear(const dir_list *d, const char *name) {
    for (size_t i = 0; i < d->n; ++i) if (strcmp(d->e[i].name, name) == 0) return &d->e[i];
    return NULL;
}

/* ------------------------------------------------------------------ `microkimi build`, Gaussian fallback branch */
#define SIGMA 0.02f /* build.rs:17 */
static void put_f32(uint8_t *base, const dir_list *d, const char *name, const float *v, size_t n) {
    const dir_ent *e = dir_find_linear(d, name);
    if (e && e->size == n * 4) memcpy(base + e->off, v, n * 4);
}
static void put_gauss(uint8_t *base, const dir_list *d, const char *tensor, const char *seed, size_t n, float sigma) {
    float *v = (float *)malloc(n * 4);
    or_rng_fill_gauss(seed, sigma, v, n); /* build.rs:318-335: rng.gauss() * SIGMA with an empty pool */
    put_f32(base, d, tensor, v, n);
    free(v);
}
static void put_ones(uint8_t *base, const dir_list *d, const char *tensor, size_t n, float val) {
    float *v = (float *)malloc(n * 4);
    for (size_t i = 0; i < n; ++i) v[i] = val;
    put_f32(base, d, tensor, v, n);
    free(v);
}

int or_build_bin(const char *path, const or_config *c) {
    dir_list dl = {0};
    char nm[160], sd[160];
    const uint32_t d = c->d, proj = c->kda_heads * c->kda_dim, qh = c->mla_nope + c->mla_rope;
    const uint32_t qb = c->mla_heads * qh, kvb = c->mla_heads * (c->mla_nope + c->mla_v), cdim = c->mla_kva + c->mla_rope;
    const uint32_t hv = c->mla_heads * c->mla_v;
    /* registration order = write order (build.rs:350-420) */
    dir_add(&dl, "embed_tokens.weight", DT_F32, c->vocab, d);
    dir_add(&dl, "lm_head.weight", DT_F32, c->vocab, d);
    dir_add(&dl, "norm.weight", DT_F32, d, 0);
    dir_add(&dl, "output_attn_res_norm.weight", DT_F32, d, 0);
    dir_add(&dl, "output_attn_res_proj.weight", DT_F32, d, 0);
    for (uint32_t l = 0; l < c->n_layers; ++l) {
#define ADD(suffix, d0, d1) do { snprintf(nm, sizeof(nm), "layers.%u.%s", l, suffix); dir_add(&dl, nm, DT_F32, d0, d1); } while (0)
        ADD("input_layernorm.weight", d, 0); ADD("post_attention_layernorm.weight", d, 0);
        ADD("self_attention_res_norm.weight", d, 0); ADD("self_attention_res_proj.weight", d, 0);
        ADD("mlp_res_norm.weight", d, 0); ADD("mlp_res_proj.weight", d, 0);
        if (or_config_is_mla(c, l)) {
            ADD("self_attn.q_a_proj.weight", c->mla_qa, d); ADD("self_attn.q_a_layernorm.weight", c->mla_qa, 0);
            ADD("self_attn.q_b_proj.weight", qb, c->mla_qa); ADD("self_attn.kv_a_proj_with_mqa.weight", cdim, d);
            ADD("self_attn.kv_a_layernorm.weight", c->mla_kva, 0); ADD("self_attn.kv_b_proj.weight", kvb, c->mla_kva);
            ADD("self_attn.g_proj.weight", hv, d); ADD("self_attn.o_proj.weight", d, hv);
        } else {
            ADD("self_attn.q_proj.weight", proj, d); ADD("self_attn.k_proj.weight", proj, d); ADD("self_attn.v_proj.weight", proj, d);
            ADD("self_attn.g_proj.weight", proj, d); ADD("self_attn.o_proj.weight", d, proj);
            ADD("self_attn.q_conv1d.weight", proj, c->kda_conv); ADD("self_attn.k_conv1d.weight", proj, c->kda_conv);
            ADD("self_attn.v_conv1d.weight", proj, c->kda_conv);
            ADD("self_attn.f_a_proj.weight", c->kda_fa, d); ADD("self_attn.f_b_proj.weight", proj, c->kda_fa);
            ADD("self_attn.A_log", c->kda_dim, 0); ADD("self_attn.dt_bias", proj, 0);
            ADD("self_attn.b_proj.weight", c->kda_heads, d); ADD("self_attn.o_norm.weight", c->kda_dim, 0);
        }
        if (or_config_is_moe(c, l)) {
            ADD("block_sparse_moe.gate.weight", c->n_experts, d); ADD("block_sparse_moe.gate.e_score_correction_bias", c->n_experts, 0);
            ADD("block_sparse_moe.routed_expert_down_proj.weight", c->routed_hidden, d);
            ADD("block_sparse_moe.routed_expert_up_proj.weight", d, c->routed_hidden);
            ADD("block_sparse_moe.routed_expert_norm.weight", c->routed_hidden, 0);
            ADD("block_sparse_moe.shared_experts.gate_proj.weight", c->shared_inter, d);
            ADD("block_sparse_moe.shared_experts.up_proj.weight", c->shared_inter, d);
            ADD("block_sparse_moe.shared_experts.down_proj.weight", d, c->shared_inter);
        } else {
            ADD("mlp.gate_proj.weight", c->dense_inter, d); ADD("mlp.up_proj.weight", c->dense_inter, d);
            ADD("mlp.down_proj.weight", d, c->dense_inter);
        }
#undef ADD
    }
    const size_t first_expert = dl.n;
    for (uint32_t l = 0; l < c->n_layers; ++l) {
        if (!or_config_is_moe(c, l)) continue;
        for (uint32_t e = 0; e < c->n_experts; ++e) {
            snprintf(nm, sizeof(nm), "layers.%u.block_sparse_moe.experts.%u.w1", l, e);
            dir_add(&dl, nm, DT_MXFP4, c->moe_inter, c->routed_hidden);
            snprintf(nm, sizeof(nm), "layers.%u.block_sparse_moe.experts.%u.w2", l, e);
            dir_add(&dl, nm, DT_MXFP4, c->routed_hidden, c->moe_inter);
            snprintf(nm, sizeof(nm), "layers.%u.block_sparse_moe.experts.%u.w3", l, e);
            dir_add(&dl, nm, DT_MXFP4, c->moe_inter, c->routed_hidden);
        }
    }
    /* header: MKIM0001 for the historical micro configuration, MKIM0002 + JSON otherwise (weights.rs:142-160) */
    or_config micro;
    or_config_microkimi(&micro);
    const int v2 = memcmp(&micro, c, sizeof(micro)) != 0;
    char js[2048];
    const int jl = v2 ? config_to_json(c, js, sizeof(js)) : 0;
    const uint64_t prefix = v2 ? 8 + 4 + (uint64_t)jl : 8;
    dir_layout(&dl, prefix);
    const uint64_t total = dl.e[dl.n - 1].off + dl.e[dl.n - 1].size;

    int fd = open(path, O_RDWR | O_CREAT | O_TRUNC, 0644);
    if (fd < 0) { free(dl.e); return -1; }
    if (ftruncate(fd, (off_t)total) != 0) { close(fd); free(dl.e); return -2; }
    uint8_t *base = (uint8_t *)mmap(NULL, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (base == MAP_FAILED) { close(fd); free(dl.e); return -3; }
    uint8_t *p = base;
    memcpy(p, v2 ? "MKIM0002" : "MKIM0001", 8); p += 8;
    if (v2) { const uint32_t u = (uint32_t)jl; memcpy(p, &u, 4); p += 4; memcpy(p, js, (size_t)jl); p += jl; }
    { const uint32_t u = (uint32_t)dl.n; memcpy(p, &u, 4); p += 4; }
    for (size_t i = 0; i < dl.n; ++i) { /* weights.rs:133-147 */
        const dir_ent *e = &dl.e[i];
        const uint16_t nl = (uint16_t)strlen(e->name);
        memcpy(p, &nl, 2); p += 2; memcpy(p, e->name, nl); p += nl;
        *p++ = e->dtype; *p++ = e->nd;
        for (int k = 0; k < e->nd; ++k) { memcpy(p, &e->dims[k], 4); p += 4; }
        memcpy(p, &e->off, 8); p += 8; memcpy(p, &e->size, 8); p += 8;
    }

    /* f32 tensors.  The builder takes embed_tokens / lm_head rows from a downloaded checkpoint and fails
     * without it (build.rs:252-253, 431-441); here every row is Gaussian (seeds "embed_all" / "lm_head_all"). */
    put_gauss(base, &dl, "embed_tokens.weight", "embed_all", (size_t)c->vocab * d, SIGMA);
    put_gauss(base, &dl, "lm_head.weight", "lm_head_all", (size_t)c->vocab * d, SIGMA);
    put_ones(base, &dl, "norm.weight", d, 1.0f);
    put_ones(base, &dl, "output_attn_res_norm.weight", d, 1.0f);
    put_gauss(base, &dl, "output_attn_res_proj.weight", "oar_proj_fb", d, SIGMA);
#pragma omp parallel for schedule(dynamic, 1) private(nm, sd)
    for (uint32_t l = 0; l < c->n_layers; ++l) { /* build.rs:448-526 */
        char pf[32];
        snprintf(pf, sizeof(pf), "layers.%u.", l);
#define T(suffix) (snprintf(nm, sizeof(nm), "%s%s", pf, suffix), nm)
#define S1(fmt, ...) (snprintf(sd, sizeof(sd), fmt, __VA_ARGS__), sd)
        put_ones(base, &dl, T("input_layernorm.weight"), d, 1.0f);
        put_ones(base, &dl, T("post_attention_layernorm.weight"), d, 1.0f);
        put_ones(base, &dl, T("self_attention_res_norm.weight"), d, 1.0f);
        put_gauss(base, &dl, T("self_attention_res_proj.weight"), S1("sar%u", l), d, SIGMA);
        put_ones(base, &dl, T("mlp_res_norm.weight"), d, 1.0f);
        put_gauss(base, &dl, T("mlp_res_proj.weight"), S1("mlpres%u", l), d, SIGMA);
        if (or_config_is_mla(c, l)) {
            put_gauss(base, &dl, T("self_attn.q_a_proj.weight"), S1("%sqa", pf), (size_t)c->mla_qa * d, SIGMA);
            put_ones(base, &dl, T("self_attn.q_a_layernorm.weight"), c->mla_qa, 1.0f);
            put_gauss(base, &dl, T("self_attn.q_b_proj.weight"), S1("%sqb", pf), (size_t)qb * c->mla_qa, SIGMA);
            put_gauss(base, &dl, T("self_attn.kv_a_proj_with_mqa.weight"), S1("%skva", pf), (size_t)cdim * d, SIGMA);
            put_ones(base, &dl, T("self_attn.kv_a_layernorm.weight"), c->mla_kva, 1.0f);
            put_gauss(base, &dl, T("self_attn.kv_b_proj.weight"), S1("%skvb", pf), (size_t)kvb * c->mla_kva, SIGMA);
            put_gauss(base, &dl, T("self_attn.g_proj.weight"), S1("%sg", pf), (size_t)hv * d, SIGMA);
            put_gauss(base, &dl, T("self_attn.o_proj.weight"), S1("%so", pf), (size_t)d * hv, SIGMA);
        } else {
            static const char *const five[5] = {"q_proj", "k_proj", "v_proj", "g_proj", "o_proj"};
            for (int k = 0; k < 5; ++k) {
                char t2[64];
                snprintf(t2, sizeof(t2), "self_attn.%s.weight", five[k]);
                put_gauss(base, &dl, T(t2), S1("%s%s", pf, five[k]), (size_t)proj * d, SIGMA);
            }
            static const char *const conv[3] = {"q_conv1d", "k_conv1d", "v_conv1d"};
            for (int k = 0; k < 3; ++k) {
                char t2[64];
                snprintf(t2, sizeof(t2), "self_attn.%s.weight", conv[k]);
                put_gauss(base, &dl, T(t2), S1("%s%s", pf, conv[k]), (size_t)proj * c->kda_conv, SIGMA);
            }
            put_gauss(base, &dl, T("self_attn.f_a_proj.weight"), S1("%sfa", pf), (size_t)c->kda_fa * d, SIGMA);
            put_gauss(base, &dl, T("self_attn.f_b_proj.weight"), S1("%sfb", pf), (size_t)proj * c->kda_fa, SIGMA);
            { /* A_log = ln(uniform(1, 16)) (build.rs:489-496) */
                or_rng r;
                or_rng_for_tensor(&r, S1("%salog", pf));
                float *v = (float *)malloc(c->kda_dim * 4);
                for (uint32_t i = 0; i < c->kda_dim; ++i) v[i] = (float)log(1.0 + or_rng_uniform(&r) * 15.0);
                put_f32(base, &dl, T("self_attn.A_log"), v, c->kda_dim);
                free(v);
            }
            put_gauss(base, &dl, T("self_attn.dt_bias"), S1("%sdt", pf), proj, SIGMA);
            put_gauss(base, &dl, T("self_attn.b_proj.weight"), S1("%sb", pf), (size_t)c->kda_heads * d, SIGMA);
            put_ones(base, &dl, T("self_attn.o_norm.weight"), c->kda_dim, 1.0f);
        }
        if (or_config_is_moe(c, l)) {
            put_gauss(base, &dl, T("block_sparse_moe.gate.weight"), S1("%sgate", pf), (size_t)c->n_experts * d, SIGMA);
            put_ones(base, &dl, T("block_sparse_moe.gate.e_score_correction_bias"), c->n_experts, 0.0f);
            put_gauss(base, &dl, T("block_sparse_moe.routed_expert_down_proj.weight"), S1("%srd", pf), (size_t)c->routed_hidden * d, SIGMA);
            put_gauss(base, &dl, T("block_sparse_moe.routed_expert_up_proj.weight"), S1("%sru", pf), (size_t)d * c->routed_hidden, SIGMA);
            put_ones(base, &dl, T("block_sparse_moe.routed_expert_norm.weight"), c->routed_hidden, 1.0f);
            put_gauss(base, &dl, T("block_sparse_moe.shared_experts.gate_proj.weight"), S1("%ssg", pf), (size_t)c->shared_inter * d, SIGMA);
            put_gauss(base, &dl, T("block_sparse_moe.shared_experts.up_proj.weight"), S1("%ssu", pf), (size_t)c->shared_inter * d, SIGMA);
            put_gauss(base, &dl, T("block_sparse_moe.shared_experts.down_proj.weight"), S1("%ssd", pf), (size_t)d * c->shared_inter, SIGMA);
        } else {
            put_gauss(base, &dl, T("mlp.gate_proj.weight"), S1("%sdg", pf), (size_t)c->dense_inter * d, SIGMA);
            put_gauss(base, &dl, T("mlp.up_proj.weight"), S1("%sdu", pf), (size_t)c->dense_inter * d, SIGMA);
            put_gauss(base, &dl, T("mlp.down_proj.weight"), S1("%sdd", pf), (size_t)d * c->dense_inter, SIGMA);
        }
#undef T
#undef S1
    }
    /* MXFP4 experts: values seeded by the tensor's own name, quantized with the searched rule (build.rs:553-571).
     * The expert entries were appended in order, so they are addressed by index, not looked up by name. */
    const long n_exp_t = (long)(dl.n - first_expert);
#pragma omp parallel
    {
        const size_t ne = (size_t)c->moe_inter * c->routed_hidden;
        float *vals = (float *)malloc(ne * 4);
#pragma omp for schedule(static)
        for (long i = 0; i < n_exp_t; ++i) {
            const dir_ent *e = &dl.e[first_expert + (size_t)i];
            or_rng_fill_gauss(e->name, SIGMA, vals, ne);
            uint8_t *blob = base + e->off;
            or_mxfp4_quantize(vals, e->dims[0], e->dims[1], 1, blob, blob + ne / 2);
        }
        free(vals);
    }
    munmap(base, total);
    close(fd);
    free(dl.e);
    return 0;
}

/* ------------------------------------------------------------------ the container: reader (weights.rs:421-468) */
struct or_bin {
    uint8_t *base;
    uint64_t bytes;
    or_config cfg;
    dir_ent *e;
    size_t n;
    uint32_t *table; /* open-addressing hash over names -> index + 1 */
    size_t tcap;
};
static uint64_t fnv(const char *s) {
    uint64_t h = 0xcbf29ce484222325ULL;
    for (; *s; ++s) { h ^= (uint8_t)*s; h *= 0x00000100000001b3ULL; }
    return h;
}
or_bin *or_bin_open(const char *path) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return NULL;
    struct stat st;
    if (fstat(fd, &st) != 0) { close(fd); return NULL; }
    uint8_t *base = (uint8_t *)mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (base == MAP_FAILED) return NULL;
    or_bin *b = (or_bin *)calloc(1, sizeof(or_bin));
    b->base = base; b->bytes = (uint64_t)st.st_size;
    const uint8_t *p = base + 8;
    if (memcmp(base, "MKIM0001", 8) == 0) {
        or_config_microkimi(&b->cfg);
    } else if (memcmp(base, "MKIM0002", 8) == 0) {
        uint32_t cl;
        memcpy(&cl, p, 4); p += 4;
        config_from_json(&b->cfg, (const char *)p, cl);
        p += cl;
    } else {
        munmap(base, b->bytes); free(b); return NULL;
    }
    uint32_t n;
    memcpy(&n, p, 4); p += 4;
    b->n = n;
    b->e = (dir_ent *)calloc(n, sizeof(dir_ent));
    b->tcap = 1;
    while (b->tcap < (size_t)n * 2 + 16) b->tcap <<= 1;
    b->table = (uint32_t *)calloc(b->tcap, sizeof(uint32_t));
    for (uint32_t i = 0; i < n; ++i) {
        dir_ent *e = &b->e[i];
        uint16_t nl;
        memcpy(&nl, p, 2); p += 2;
        const size_t cp = nl < sizeof(e->name) - 1 ? nl : sizeof(e->name) - 1;
        memcpy(e->name, p, cp); p += nl;
        e->dtype = *p++; e->nd = *p++;
        for (int k = 0; k < e->nd; ++k) { uint32_t dv; memcpy(&dv, p, 4); p += 4; if (k < 2) e->dims[k] = dv; }
        memcpy(&e->off, p, 8); p += 8; memcpy(&e->size, p, 8); p += 8;
        size_t h = (size_t)fnv(e->name) & (b->tcap - 1);
        while (b->table[h]) h = (h + 1) & (b->tcap - 1);
        b->table[h] = i + 1;
    }
    return b;
}
void or_bin_close(or_bin *b) {
    if (!b) return;
    munmap(b->base, b->bytes);
    free(b->e); free(b->table); free(b);
}
const or_config *or_bin_config(const or_bin *b) { return &b->cfg; }
size_t or_bin_count(const or_bin *b) { return b->n; }
const void *or_bin_get(const or_bin *b, const char *name, uint8_t *dtype, uint32_t *dims2, uint64_t *size) {
    size_t h = (size_t)fnv(name) & (b->tcap - 1);
    while (b->table[h]) {
        const dir_ent *e = &b->e[b->table[h] - 1];
        if (strcmp(e->name, name) == 0) {
            if (dtype) *dtype = e->dtype;
            if (dims2) { dims2[0] = e->dims[0]; dims2[1] = e->nd > 1 ? e->dims[1] : 0; }
            if (size) *size = e->size;
            return b->base + e->off;
        }
        h = (h + 1) & (b->tcap - 1);
    }
    return NULL;
}
int or_bin_entry(const or_bin *b, size_t i, const char **name, uint8_t *dtype, uint32_t *dims2, uint64_t *off, uint64_t *size) {
    if (i >= b->n) return -1;
    const dir_ent *e = &b->e[i];
    if (name) *name = e->name;
    if (dtype) *dtype = e->dtype;
    if (dims2) { dims2[0] = e->dims[0]; dims2[1] = e->nd > 1 ? e->dims[1] : 0; }
    if (off) *off = e->off;
    if (size) *size = e->size;
    return 0;
}

/* ------------------------------------------------------------------ the model (model.rs:906-1025) */
typedef struct {
    int is_mla, is_moe;
    const float *input_ln, *post_ln;
    float *sa_res_w, *mlp_res_w; /* norm * proj, combined at load (model.rs:911-915) */
    /* KDA (model.rs:982-1000) */
    const float *q_proj, *k_proj, *v_proj, *g_proj, *o_proj, *f_a, *f_b, *b_proj;
    or_kda_desc kda;
    float *conv_q, *conv_k, *conv_v, *s;
    /* MLA (model.rs:959-969) */
    const float *q_a, *q_a_ln, *q_b, *kv_a, *kv_a_ln, *kv_b, *mg_proj, *mo_proj;
    or_mla_cache *cache;
    /* FFN */
    or_moe_k3_desc moe;
    const uint8_t **packed, **scales;
    const float *dg, *du, *dd;
} or_layer;
struct or_model {
    or_bin *bin;
    or_config cfg;
    int n_threads;
    size_t max_pos;
    const float *embed, *lm_head, *norm_f;
    float *out_res_w;
    int8_t *hq;   /* Q8Head::from_f32 of lm_head (model.rs:921-925) */
    float *hs;
    or_layer *layers;
    float *blocks; /* [n_layers / attn_res_block + 2][d] */
};

static const float *need_f32(or_bin *b, const char *name, uint64_t count, int *bad) {
    uint8_t dt; uint64_t sz;
    const void *p = or_bin_get(b, name, &dt, NULL, &sz);
    if (!p || dt != DT_F32 || sz != count * 4) { fprintf(stderr, "or_model_open: tensor %s missing or of the wrong size\n", name); *bad = 1; return NULL; }
    return (const float *)p;
}
static float *combine(const float *a, const float *b, size_t n) {
    float *o = (float *)malloc(n * 4);
    for (size_t i = 0; i < n; ++i) o[i] = (a && b) ? a[i] * b[i] : 0.0f;
    return o;
}

or_model *or_model_open(const char *path, size_t max_positions, int n_threads) {
    or_bin *b = or_bin_open(path);
    if (!b) return NULL;
    or_model *m = (or_model *)calloc(1, sizeof(or_model));
    m->bin = b; m->cfg = b->cfg; m->n_threads = n_threads < 1 ? 1 : n_threads; m->max_pos = max_positions;
    const or_config *c = &m->cfg;
    const size_t d = c->d, proj = (size_t)c->kda_heads * c->kda_dim, qh = c->mla_nope + c->mla_rope;
    const size_t qb = c->mla_heads * qh, kvb = (size_t)c->mla_heads * (c->mla_nope + c->mla_v), cdim = c->mla_kva + c->mla_rope;
    const size_t hv = (size_t)c->mla_heads * c->mla_v;
    int bad = 0;
    char nm[160];
    m->embed = need_f32(b, "embed_tokens.weight", (uint64_t)c->vocab * d, &bad);
    m->lm_head = need_f32(b, "lm_head.weight", (uint64_t)c->vocab * d, &bad);
    m->norm_f = need_f32(b, "norm.weight", d, &bad);
    m->out_res_w = combine(need_f32(b, "output_attn_res_norm.weight", d, &bad), need_f32(b, "output_attn_res_proj.weight", d, &bad), d);
    m->layers = (or_layer *)calloc(c->n_layers, sizeof(or_layer));
    m->blocks = (float *)calloc((size_t)(c->n_layers / c->attn_res_block + 2) * d, 4);
    for (uint32_t l = 0; l < c->n_layers && !bad; ++l) {
        or_layer *L = &m->layers[l];
#define G(suffix, count) (snprintf(nm, sizeof(nm), "layers.%u.%s", l, suffix), need_f32(b, nm, (uint64_t)(count), &bad))
        L->input_ln = G("input_layernorm.weight", d);
        L->post_ln = G("post_attention_layernorm.weight", d);
        L->sa_res_w = combine(G("self_attention_res_norm.weight", d), G("self_attention_res_proj.weight", d), d);
        L->mlp_res_w = combine(G("mlp_res_norm.weight", d), G("mlp_res_proj.weight", d), d);
        L->is_mla = or_config_is_mla(c, l);
        L->is_moe = or_config_is_moe(c, l);
        if (L->is_mla) {
            L->q_a = G("self_attn.q_a_proj.weight", c->mla_qa * d); L->q_a_ln = G("self_attn.q_a_layernorm.weight", c->mla_qa);
            L->q_b = G("self_attn.q_b_proj.weight", qb * c->mla_qa); L->kv_a = G("self_attn.kv_a_proj_with_mqa.weight", cdim * d);
            L->kv_a_ln = G("self_attn.kv_a_layernorm.weight", c->mla_kva); L->kv_b = G("self_attn.kv_b_proj.weight", kvb * c->mla_kva);
            L->mg_proj = G("self_attn.g_proj.weight", hv * d); L->mo_proj = G("self_attn.o_proj.weight", d * hv);
            L->cache = or_mla_new(c->mla_heads, c->mla_nope, c->mla_rope, c->mla_v, max_positions);
        } else {
            L->q_proj = G("self_attn.q_proj.weight", proj * d); L->k_proj = G("self_attn.k_proj.weight", proj * d);
            L->v_proj = G("self_attn.v_proj.weight", proj * d); L->g_proj = G("self_attn.g_proj.weight", proj * d);
            L->o_proj = G("self_attn.o_proj.weight", d * proj); L->f_a = G("self_attn.f_a_proj.weight", c->kda_fa * d);
            L->f_b = G("self_attn.f_b_proj.weight", proj * c->kda_fa); L->b_proj = G("self_attn.b_proj.weight", c->kda_heads * d);
            L->kda.heads = c->kda_heads; L->kda.dim = c->kda_dim; L->kda.kconv = c->kda_conv;
            L->kda.gate_lb = c->gate_lb; L->kda.rms_eps = c->rms_eps;
            L->kda.q_conv = G("self_attn.q_conv1d.weight", proj * c->kda_conv); L->kda.k_conv = G("self_attn.k_conv1d.weight", proj * c->kda_conv);
            L->kda.v_conv = G("self_attn.v_conv1d.weight", proj * c->kda_conv); L->kda.a_log = G("self_attn.A_log", c->kda_dim);
            L->kda.dt_bias = G("self_attn.dt_bias", proj); L->kda.o_norm = G("self_attn.o_norm.weight", c->kda_dim);
            L->conv_q = (float *)calloc((c->kda_conv - 1) * proj, 4); L->conv_k = (float *)calloc((c->kda_conv - 1) * proj, 4);
            L->conv_v = (float *)calloc((c->kda_conv - 1) * proj, 4); L->s = (float *)calloc((size_t)c->kda_heads * c->kda_dim * c->kda_dim, 4);
        }
        if (L->is_moe) {
            or_moe_k3_desc *q = &L->moe;
            q->d = d; q->rh = c->routed_hidden; q->inter = c->moe_inter; q->n_experts = c->n_experts; q->top_k = c->top_k;
            q->shared_inter = c->shared_inter; q->rms_eps = c->rms_eps; q->use_q8 = 1;
            q->gate_w = G("block_sparse_moe.gate.weight", c->n_experts * d);
            q->gate_b = G("block_sparse_moe.gate.e_score_correction_bias", c->n_experts);
            q->routed_down = G("block_sparse_moe.routed_expert_down_proj.weight", c->routed_hidden * d);
            q->routed_up = G("block_sparse_moe.routed_expert_up_proj.weight", d * c->routed_hidden);
            q->routed_norm = G("block_sparse_moe.routed_expert_norm.weight", c->routed_hidden);
            q->shared_gate = G("block_sparse_moe.shared_experts.gate_proj.weight", c->shared_inter * d);
            q->shared_up = G("block_sparse_moe.shared_experts.up_proj.weight", c->shared_inter * d);
            q->shared_down = G("block_sparse_moe.shared_experts.down_proj.weight", d * c->shared_inter);
            L->packed = (const uint8_t **)calloc((size_t)c->n_experts * 3, sizeof(void *));
            L->scales = (const uint8_t **)calloc((size_t)c->n_experts * 3, sizeof(void *));
            static const char *const wn[3] = {"w1", "w2", "w3"};
            const size_t half = (size_t)c->moe_inter * c->routed_hidden / 2;
            for (uint32_t e = 0; e < c->n_experts && !bad; ++e)
                for (int k = 0; k < 3; ++k) {
                    snprintf(nm, sizeof(nm), "layers.%u.block_sparse_moe.experts.%u.%s", l, e, wn[k]);
                    uint8_t dt; uint64_t sz;
                    const uint8_t *p = (const uint8_t *)or_bin_get(b, nm, &dt, NULL, &sz);
                    if (!p || dt != DT_MXFP4 || sz != half + half / 16) { fprintf(stderr, "or_model_open: expert %s missing\n", nm); bad = 1; break; }
                    L->packed[e * 3 + k] = p;
                    L->scales[e * 3 + k] = p + half;
                }
            q->packed = L->packed; q->scales = L->scales;
        } else {
            L->dg = G("mlp.gate_proj.weight", c->dense_inter * d); L->du = G("mlp.up_proj.weight", c->dense_inter * d);
            L->dd = G("mlp.down_proj.weight", d * c->dense_inter);
        }
#undef G
    }
    if (bad) { or_model_free(m); return NULL; }
    m->hq = (int8_t *)malloc((size_t)c->vocab * d);
    m->hs = (float *)malloc((size_t)c->vocab * (d / 32) * 4);
    or_q8head_from_f32(m->lm_head, c->vocab, d, m->hq, m->hs);
    return m;
}
void or_model_free(or_model *m) {
    if (!m) return;
    for (uint32_t l = 0; m->layers && l < m->cfg.n_layers; ++l) {
        or_layer *L = &m->layers[l];
        free(L->sa_res_w); free(L->mlp_res_w); free(L->conv_q); free(L->conv_k); free(L->conv_v); free(L->s);
        if (L->cache) or_mla_free(L->cache);
        free((void *)L->packed); free((void *)L->scales);
    }
    free(m->layers); free(m->blocks); free(m->out_res_w); free(m->hq); free(m->hs);
    or_bin_close(m->bin);
    free(m);
}
const or_config *or_model_config(const or_model *m) { return &m->cfg; }
void or_model_reset(or_model *m) { /* fresh caches: KdaCache zeros, MlaCache::new (model.rs:956, 971-977) */
    const or_config *c = &m->cfg;
    const size_t proj = (size_t)c->kda_heads * c->kda_dim;
    for (uint32_t l = 0; l < c->n_layers; ++l) {
        or_layer *L = &m->layers[l];
        if (L->is_mla) { L->cache->n = 0; continue; }
        memset(L->conv_q, 0, (c->kda_conv - 1) * proj * 4); memset(L->conv_k, 0, (c->kda_conv - 1) * proj * 4);
        memset(L->conv_v, 0, (c->kda_conv - 1) * proj * 4); memset(L->s, 0, (size_t)c->kda_heads * c->kda_dim * c->kda_dim * 4);
    }
}

static void kda_forward(or_model *m, or_layer *L, const float *x, float *out) { /* model.rs:1179-1232 */
    const or_config *c = &m->cfg;
    const size_t d = c->d, proj = (size_t)c->kda_heads * c->kda_dim;
    const int nt = m->n_threads;
    float *buf = (float *)malloc((6 * proj + c->kda_fa + c->kda_heads) * 4);
    float *q = buf, *k = q + proj, *v = k + proj, *g_low = v + proj, *g2 = g_low + proj, *o = g2 + proj, *fa = o + proj, *beta = fa + c->kda_fa;
    or_matvec_f32(L->q_proj, proj, d, x, q, nt);
    or_matvec_f32(L->k_proj, proj, d, x, k, nt);
    or_matvec_f32(L->v_proj, proj, d, x, v, nt);
    or_matvec_f32(L->f_a, c->kda_fa, d, x, fa, nt);
    or_matvec_f32(L->f_b, proj, c->kda_fa, fa, g_low, nt);
    or_matvec_f32(L->b_proj, c->kda_heads, d, x, beta, nt);   /* the sigmoid is applied inside or_kda_step */
    or_matvec_f32(L->g_proj, proj, d, x, g2, nt);
    or_kda_step(&L->kda, L->conv_q, L->conv_k, L->conv_v, L->s, q, k, v, g_low, beta, g2, o);
    or_matvec_f32(L->o_proj, d, proj, o, out, nt);
    free(buf);
}
static void mla_forward(or_model *m, or_layer *L, const float *x, float *out) { /* model.rs:1939-2022, q8 cache, MQA kernel */
    const or_config *c = &m->cfg;
    const size_t d = c->d, H = c->mla_heads, nope = c->mla_nope, rope = c->mla_rope, vd = c->mla_v, qh = nope + rope;
    const size_t qa_n = c->mla_qa, kva = c->mla_kva, cdim = kva + rope, hv = H * vd;
    const int nt = m->n_threads;
    float *buf = (float *)malloc((2 * qa_n + H * qh + cdim + kva + H * (nope + vd) + H * qh + hv + hv + hv) * 4);
    float *qa = buf, *qan = qa + qa_n, *q = qan + qa_n, *cc = q + H * qh, *kpn = cc + cdim, *kb = kpn + kva;
    float *k_new = kb + H * (nope + vd), *v_new = k_new + H * qh, *attn = v_new + hv, *g = attn + hv;
    or_matvec_f32(L->q_a, qa_n, d, x, qa, nt);
    or_rmsnorm(qa, L->q_a_ln, qa_n, c->rms_eps, qan);
    or_matvec_f32(L->q_b, H * qh, qa_n, qan, q, nt);
    or_matvec_f32(L->kv_a, cdim, d, x, cc, nt);
    or_rmsnorm(cc, L->kv_a_ln, kva, c->rms_eps, kpn);
    or_matvec_f32(L->kv_b, H * (nope + vd), kva, kpn, kb, nt);
    for (size_t h = 0; h < H; ++h) { /* :1964-1973 */
        memcpy(k_new + h * qh, kb + h * (nope + vd), nope * 4);
        memcpy(k_new + h * qh + nope, cc + kva, rope * 4);
        memcpy(v_new + h * vd, kb + h * (nope + vd) + nope, vd * 4);
    }
    or_mla_push(L->cache, k_new, v_new);
    const size_t pos = L->cache->n - 1;
    const float scale = powf((float)qh, -0.5f); /* :1977 */
    or_mla_attn_flash_q8_mqa(L->cache, q, pos, scale, attn);
    or_matvec_f32(L->mg_proj, hv, d, x, g, nt);
    for (size_t i = 0; i < hv; ++i) attn[i] *= or_sigmoid(g[i]); /* :2017-2019 */
    or_matvec_f32(L->mo_proj, d, hv, attn, out, nt);
    free(buf);
}
static void dense_forward(or_model *m, or_layer *L, const float *x, float *out) { /* model.rs:2382-2396 */
    const or_config *c = &m->cfg;
    const size_t di = c->dense_inter;
    float *a = (float *)malloc(3 * di * 4), *u = a + di, *act = u + di;
    or_matvec_f32(L->dg, di, c->d, x, a, m->n_threads);
    or_matvec_f32(L->du, di, c->d, x, u, m->n_threads);
    for (size_t j = 0; j < di; ++j) act[j] = or_situ(a[j], u[j]);
    or_matvec_f32(L->dd, c->d, di, act, out, m->n_threads);
    free(a);
}

/* Model::forward (model.rs:2889-3031): one token through every layer; logits [vocab]; `hidden_out` (optional, [d])
 * receives the final normed hidden state (the input of logits_project). */
int or_model_forward_layers(or_model *m, uint32_t token, float *logits, float *hidden_out, float *layer_out);
int or_model_forward(or_model *m, uint32_t token, float *logits, float *hidden_out) {
    return or_model_forward_layers(m, token, logits, hidden_out, NULL);
}
/* layer_out (optional, [n_layers][4][d]): per layer the attention block's output, the residual stream after it, the FFN's
 * output and the residual stream after the layer (the engine's parity dumps record the last, model.rs:2760) */
int or_model_forward_layers(or_model *m, uint32_t token, float *logits, float *hidden_out, float *layer_out) {
    const or_config *c = &m->cfg;
    const size_t d = c->d;
    if (token >= c->vocab) return -1;
    float *hidden = (float *)malloc(6 * d * 4), *prefix = hidden + d, *x = prefix + d, *attn_out = x + d, *prefix2 = attn_out + d, *mlp_out = prefix2 + d;
    memcpy(hidden, m->embed + (size_t)token * d, d * 4);
    size_t nb = 0;
    for (uint32_t l = 0; l < c->n_layers; ++l) {
        or_layer *L = &m->layers[l];
        memcpy(prefix, hidden, d * 4);
        if (nb > 0) or_attn_res(d, c->rms_eps, prefix, m->blocks, nb, L->sa_res_w, hidden);
        int have_prefix = 1;
        if (l % c->attn_res_block == 0) { memcpy(m->blocks + nb * d, prefix, d * 4); ++nb; have_prefix = 0; }
        or_rmsnorm(hidden, L->input_ln, d, c->rms_eps, x);
        if (L->is_mla) {
            if (L->cache->n >= L->cache->cap) { free(hidden); return -2; }
            mla_forward(m, L, x, attn_out);
        } else {
            kda_forward(m, L, x, attn_out);
        }
        if (have_prefix) for (size_t j = 0; j < d; ++j) prefix2[j] = prefix[j] + attn_out[j];
        else memcpy(prefix2, attn_out, d * 4);
        or_attn_res(d, c->rms_eps, prefix2, m->blocks, nb, L->mlp_res_w, hidden);
        or_rmsnorm(hidden, L->post_ln, d, c->rms_eps, x);
        if (L->is_moe) or_moe_k3_forward(&L->moe, x, mlp_out, NULL, NULL);
        else dense_forward(m, L, x, mlp_out);
        for (size_t j = 0; j < d; ++j) hidden[j] = prefix2[j] + mlp_out[j];
        if (layer_out) {
            float *lo = layer_out + (size_t)l * 4 * d;
            memcpy(lo, attn_out, d * 4); memcpy(lo + d, prefix2, d * 4); memcpy(lo + 2 * d, mlp_out, d * 4); memcpy(lo + 3 * d, hidden, d * 4);
        }
    }
    memcpy(prefix, hidden, d * 4);
    or_attn_res(d, c->rms_eps, prefix, m->blocks, nb, m->out_res_w, hidden);
    or_rmsnorm(hidden, m->norm_f, d, c->rms_eps, x);
    if (hidden_out) memcpy(hidden_out, x, d * 4);
    if (logits) or_q8head_matvec(m->hq, m->hs, c->vocab, d, x, logits, m->n_threads); /* logits_project, q8 head (model.rs:867-872) */
    free(hidden);
    return 0;
}
