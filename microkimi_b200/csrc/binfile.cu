// The engine's weight container (MKIM0001 / MKIM0002, src/weights.rs:1-64): reader (BinFile::open,
// src/weights.rs:421-590) and writer (BinWriter, src/weights.rs:66-186) behind the C ABI.  Host code only.
//
//   magic "MKIM0001"                          -> the historical micro configuration (src/config.rs:47-79)
//   magic "MKIM0002" | u32 len | JSON config  -> explicit configuration (src/config.rs:86-125)
//   u32 n | n x { u16 name_len | name | u8 dtype | u8 n_dims | u32 dims[] | u64 offset | u64 size } | blobs
// Blobs start on 64-byte boundaries, routed-expert matrices on 4096-byte ones (src/weights.rs:107-131).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <new>
#include <string>
#include <unordered_map>
#include <vector>

#include "mk_common.cuh"

struct mk_bin_entry_rec {
    std::string name;
    uint8_t dtype, nd;
    uint32_t dims[4];
    uint64_t off, size;
};
struct mk_bin {
    uint8_t *base;
    uint64_t bytes;
    mk_model_config cfg;
    std::vector<mk_bin_entry_rec> entries;
    std::unordered_map<std::string, size_t> index;
};
struct mk_bin_writer {
    bool v2;
    mk_model_config cfg;
    std::vector<mk_bin_entry_rec> entries;
    std::unordered_map<std::string, size_t> index;
    int fd;
    uint64_t total;
};

extern "C" void mk_model_config_default(mk_model_config *c) {  // Config::microkimi (src/config.rs:47-79)
    if (!c) return;
    memset(c, 0, sizeof(*c));
    c->n_layers = 93; c->d = 512; c->vocab = 163840; c->n_experts = 896; c->top_k = 16; c->n_shared = 2;
    c->kda_heads = 4; c->kda_dim = 128; c->kda_conv = 4; c->kda_fa = 128; c->gate_lb = -5.0f;
    c->mla_heads = 4; c->mla_qa = 128; c->mla_kva = 64; c->mla_nope = 128; c->mla_rope = 64; c->mla_v = 128;
    c->routed_hidden = 128; c->moe_inter = 64; c->shared_inter = 128; c->dense_inter = 2048;
    c->attn_res_block = 12; c->first_k_dense = 1; c->rms_eps = 1e-5f; c->eos_id = 163586; c->bos_id = 163584;
}

static uint64_t blob_size(uint8_t dtype, const uint32_t *dims, int nd, bool *ok) {  // src/weights.rs:40-64
    uint64_t n = 1;
    for (int i = 0; i < nd; ++i) n *= dims[i];
    *ok = true;
    switch (dtype) {
    case MK_DTYPE_F32: case MK_DTYPE_I32: return n * 4;
    case MK_DTYPE_MXFP4: if (nd != 2) break; return (uint64_t)dims[0] * dims[1] / 2 + (uint64_t)dims[0] * dims[1] / 32;
    case MK_DTYPE_VQ1: if (nd != 2) break; return (uint64_t)dims[0] * dims[1] / 16;
    case MK_DTYPE_MXFP4SQ: if (nd != 2) break; return (uint64_t)dims[0] * dims[1] / 2 + (uint64_t)dims[0] * dims[1] / 32 + 4;
    default: break;
    }
    *ok = false;
    return 0;
}
static bool is_expert_tensor(const std::string &n) {  // src/weights.rs:417-419
    if (n.find(".block_sparse_moe.experts.") == std::string::npos || n.size() < 3) return false;
    const std::string t = n.substr(n.size() - 3);
    return t == ".w1" || t == ".w2" || t == ".w3";
}

// ---------------------------------------------------------------- the JSON config block (numbers only)
// Finds "key" followed by ':' anywhere in the text and parses the number after it.  The block the engine writes
// is flat apart from "specials", whose keys (end_of_msg, bos) do not collide with the top-level ones.
static bool json_num(const char *js, size_t n, const char *key, double *out) {
    const std::string pat = std::string("\"") + key + "\"";
    for (size_t i = 0; i + pat.size() < n; ++i) {
        if (memcmp(js + i, pat.data(), pat.size()) != 0) continue;
        size_t j = i + pat.size();
        while (j < n && (js[j] == ' ' || js[j] == '\t' || js[j] == '\n' || js[j] == '\r')) ++j;
        if (j >= n || js[j] != ':') continue;
        ++j;
        while (j < n && (js[j] == ' ' || js[j] == '\t' || js[j] == '\n' || js[j] == '\r')) ++j;
        char buf[64];
        size_t k = 0;
        while (j < n && k + 1 < sizeof(buf) && strchr("+-0123456789.eE", js[j]) != nullptr) buf[k++] = js[j++];
        buf[k] = 0;
        if (k == 0) return false;
        *out = strtod(buf, nullptr);
        return true;
    }
    return false;
}
static bool json_has_array(const char *js, size_t n, const char *key) {
    const std::string pat = std::string("\"") + key + "\"";
    for (size_t i = 0; i + pat.size() < n; ++i) {
        if (memcmp(js + i, pat.data(), pat.size()) != 0) continue;
        size_t j = i + pat.size();
        while (j < n && (js[j] == ' ' || js[j] == ':' || js[j] == '\t' || js[j] == '\n')) ++j;
        if (j < n && js[j] == '[') return true;
    }
    return false;
}
static void config_from_json(mk_model_config *c, const char *js, size_t n) {  // Config::from_json (src/config.rs:86-125)
    mk_model_config_default(c);
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
    // explicit per-layer type lists (written by the engine's slicer after layer pruning) and the DeepSeek
    // architecture are recorded, not interpreted: a model that carries them is refused at mk_model_open
    c->has_layer_lists = json_has_array(js, n, "mla_layers") || json_has_array(js, n, "dense_layers");
    c->is_deepseek = strstr(std::string(js, n).c_str(), "deepseek_v4") != nullptr;
}
static std::string config_to_json(const mk_model_config *c) {
    char buf[2048];
    snprintf(buf, sizeof(buf),
             "{\"n_layers\":%u,\"hidden\":%u,\"vocab\":%u,\"n_experts\":%u,\"top_k\":%u,\"n_shared\":%u,\"kda_heads\":%u,"
             "\"kda_dim\":%u,\"kda_conv\":%u,\"kda_fa_rank\":%u,\"gate_lower_bound\":%.9g,\"mla_heads\":%u,\"mla_q_lora\":%u,"
             "\"mla_kv_lora\":%u,\"mla_nope\":%u,\"mla_rope\":%u,\"mla_v\":%u,\"routed_hidden\":%u,\"moe_inter\":%u,"
             "\"shared_inter\":%u,\"dense_inter\":%u,\"attn_res_block\":%u,\"first_k_dense\":%u,\"rms_eps\":%.9g,"
             "\"specials\":{\"end_of_msg\":%u,\"bos\":%u}}",
             c->n_layers, c->d, c->vocab, c->n_experts, c->top_k, c->n_shared, c->kda_heads, c->kda_dim, c->kda_conv, c->kda_fa,
             (double)c->gate_lb, c->mla_heads, c->mla_qa, c->mla_kva, c->mla_nope, c->mla_rope, c->mla_v, c->routed_hidden,
             c->moe_inter, c->shared_inter, c->dense_inter, c->attn_res_block, c->first_k_dense, (double)c->rms_eps, c->eos_id,
             c->bos_id);
    return buf;
}

// ---------------------------------------------------------------- reader
extern "C" int32_t mk_bin_open(const char *path, mk_bin **out) {
    MK_CHECK_ARG(path != nullptr && out != nullptr, "NULL argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) { mk_set_error("mk_bin_open: %s unreadable", path); return MK_ERR_ARG; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 12) { close(fd); mk_set_error("mk_bin_open: %s is too short", path); return MK_ERR_ARG; }
    uint8_t *base = (uint8_t *)mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (base == MAP_FAILED) { mk_set_error("mk_bin_open: mmap of %s failed", path); return MK_ERR_STATE; }
    mk_bin *b = new (std::nothrow) mk_bin();
    if (!b) { munmap(base, (size_t)st.st_size); return MK_ERR_OOM; }
    b->base = base;
    b->bytes = (uint64_t)st.st_size;
    const uint8_t *p = base + 8, *end = base + b->bytes;
    auto fail = [&](const char *why) {
        mk_set_error("mk_bin_open: %s: %s", path, why);
        munmap(base, (size_t)b->bytes);
        delete b;
        return MK_ERR_ARG;
    };
    if (memcmp(base, "MKIM0001", 8) == 0) {
        mk_model_config_default(&b->cfg);
    } else if (memcmp(base, "MKIM0002", 8) == 0) {
        uint32_t cl;
        memcpy(&cl, p, 4); p += 4;
        if (p + cl + 4 > end) return fail("config block runs past the end of the file");
        config_from_json(&b->cfg, (const char *)p, cl);
        p += cl;
    } else {
        return fail("bad magic (expected MKIM0001 or MKIM0002)");
    }
    if (p + 4 > end) return fail("truncated directory");
    uint32_t n;
    memcpy(&n, p, 4); p += 4;
    b->entries.reserve(n);
    b->index.reserve((size_t)n * 2);
    for (uint32_t i = 0; i < n; ++i) {
        if (p + 2 > end) return fail("truncated directory");
        uint16_t nl;
        memcpy(&nl, p, 2); p += 2;
        if (p + nl + 2 > end) return fail("truncated directory");
        mk_bin_entry_rec e;
        e.name.assign((const char *)p, nl); p += nl;
        e.dtype = *p++; e.nd = *p++;
        if (e.nd > 4 || p + 4 * e.nd + 16 > end) return fail("directory entry with more than 4 dims or truncated");
        memset(e.dims, 0, sizeof(e.dims));
        for (int k = 0; k < e.nd; ++k) { memcpy(&e.dims[k], p, 4); p += 4; }
        memcpy(&e.off, p, 8); p += 8;
        memcpy(&e.size, p, 8); p += 8;
        if (e.off > b->bytes || e.size > b->bytes - e.off) return fail("a blob runs past the end of the file (truncated weight file)");
        b->index.emplace(e.name, b->entries.size());
        b->entries.push_back(std::move(e));
    }
    *out = b;
    return MK_OK;
}
extern "C" int32_t mk_bin_close(mk_bin *b) {
    if (!b) return MK_OK;
    munmap(b->base, (size_t)b->bytes);
    delete b;
    return MK_OK;
}
extern "C" int32_t mk_bin_config(const mk_bin *b, mk_model_config *out) {
    MK_CHECK_ARG(b != nullptr && out != nullptr, "NULL argument");
    *out = b->cfg;
    return MK_OK;
}
extern "C" int64_t mk_bin_count(const mk_bin *b) { return b ? (int64_t)b->entries.size() : -1; }
static int32_t entry_out(const mk_bin *b, const mk_bin_entry_rec &e, const char **name, int32_t *dtype, int32_t *ndims, uint32_t *dims,
                         const void **data, uint64_t *size) {
    if (name) *name = e.name.c_str();
    if (dtype) *dtype = e.dtype;
    if (ndims) *ndims = e.nd;
    if (dims) memcpy(dims, e.dims, sizeof(e.dims));
    if (data) *data = b->base + e.off;
    if (size) *size = e.size;
    return MK_OK;
}
extern "C" int32_t mk_bin_find(const mk_bin *b, const char *name, int32_t *dtype, int32_t *ndims, uint32_t *dims, const void **data,
                               uint64_t *size) {
    MK_CHECK_ARG(b != nullptr && name != nullptr, "NULL argument");
    auto it = b->index.find(name);
    if (it == b->index.end()) { mk_set_error("mk_bin_find: no tensor named %s", name); return MK_ERR_ARG; }
    return entry_out(b, b->entries[it->second], nullptr, dtype, ndims, dims, data, size);
}
extern "C" int32_t mk_bin_entry(const mk_bin *b, int64_t i, const char **name, int32_t *dtype, int32_t *ndims, uint32_t *dims,
                                const void **data, uint64_t *size) {
    MK_CHECK_ARG(b != nullptr && i >= 0 && i < (int64_t)b->entries.size(), "no such entry");
    return entry_out(b, b->entries[(size_t)i], name, dtype, ndims, dims, data, size);
}

// ---------------------------------------------------------------- writer
extern "C" int32_t mk_bin_writer_create(const mk_model_config *cfg, mk_bin_writer **out) {
    MK_CHECK_ARG(out != nullptr, "out is NULL");
    mk_bin_writer *w = new (std::nothrow) mk_bin_writer();
    if (!w) return MK_ERR_OOM;
    w->v2 = cfg != nullptr;
    if (cfg) w->cfg = *cfg; else mk_model_config_default(&w->cfg);
    w->fd = -1;
    w->total = 0;
    *out = w;
    return MK_OK;
}
extern "C" int32_t mk_bin_writer_add(mk_bin_writer *w, const char *name, int32_t dtype, int32_t ndims, const uint32_t *dims) {
    MK_CHECK_ARG(w != nullptr && name != nullptr && dims != nullptr && ndims >= 1 && ndims <= 4, "bad argument");
    MK_CHECK_ARG(w->fd < 0, "the directory is closed once mk_bin_writer_begin has run");
    MK_CHECK_ARG(strlen(name) < 65536 && w->index.find(name) == w->index.end(), "name too long or already added");
    mk_bin_entry_rec e;
    e.name = name;
    e.dtype = (uint8_t)dtype;
    e.nd = (uint8_t)ndims;
    memset(e.dims, 0, sizeof(e.dims));
    for (int k = 0; k < ndims; ++k) e.dims[k] = dims[k];
    bool ok;
    e.size = blob_size(e.dtype, e.dims, e.nd, &ok);
    MK_CHECK_ARG(ok, "unknown dtype or wrong number of dims for it");
    e.off = 0;
    w->index.emplace(e.name, w->entries.size());
    w->entries.push_back(std::move(e));
    return MK_OK;
}
static bool write_all(int fd, const void *p, size_t n, uint64_t off) {
    const char *c = (const char *)p;
    while (n > 0) {
        const ssize_t k = pwrite(fd, c, n, (off_t)off);
        if (k <= 0) return false;
        c += k; n -= (size_t)k; off += (uint64_t)k;
    }
    return true;
}
extern "C" int32_t mk_bin_writer_begin(mk_bin_writer *w, const char *path) {
    MK_CHECK_ARG(w != nullptr && path != nullptr && w->fd < 0 && !w->entries.empty(), "bad argument or nothing to write");
    const std::string js = w->v2 ? config_to_json(&w->cfg) : std::string();
    const uint64_t prefix = w->v2 ? 8 + 4 + js.size() : 8;
    uint64_t dir_size = 0;
    for (const auto &e : w->entries) dir_size += 2 + e.name.size() + 1 + 1 + 4 * (uint64_t)e.nd + 8 + 8;
    uint64_t pos = prefix + 4 + dir_size;
    for (auto &e : w->entries) {
        const uint64_t align = is_expert_tensor(e.name) ? 4096 : 64;
        pos = (pos + align - 1) / align * align;
        e.off = pos;
        pos += e.size;
    }
    w->total = pos;
    std::vector<uint8_t> head;
    head.reserve((size_t)(prefix + 4 + dir_size));
    auto put = [&](const void *p, size_t n) { head.insert(head.end(), (const uint8_t *)p, (const uint8_t *)p + n); };
    put(w->v2 ? "MKIM0002" : "MKIM0001", 8);
    if (w->v2) { const uint32_t cl = (uint32_t)js.size(); put(&cl, 4); put(js.data(), js.size()); }
    const uint32_t n = (uint32_t)w->entries.size();
    put(&n, 4);
    for (const auto &e : w->entries) {
        const uint16_t nl = (uint16_t)e.name.size();
        put(&nl, 2); put(e.name.data(), nl); put(&e.dtype, 1); put(&e.nd, 1);
        for (int k = 0; k < e.nd; ++k) put(&e.dims[k], 4);
        put(&e.off, 8); put(&e.size, 8);
    }
    w->fd = open(path, O_RDWR | O_CREAT | O_TRUNC, 0644);
    if (w->fd < 0) { mk_set_error("mk_bin_writer_begin: cannot create %s", path); return MK_ERR_ARG; }
    if (ftruncate(w->fd, (off_t)w->total) != 0 || !write_all(w->fd, head.data(), head.size(), 0)) {
        mk_set_error("mk_bin_writer_begin: cannot write %s (%llu bytes)", path, (unsigned long long)w->total);
        close(w->fd); w->fd = -1;
        return MK_ERR_STATE;
    }
    return MK_OK;
}
extern "C" int32_t mk_bin_writer_put(mk_bin_writer *w, const char *name, const void *data, uint64_t size) {
    MK_CHECK_ARG(w != nullptr && name != nullptr && data != nullptr, "NULL argument");
    MK_CHECK_ARG(w->fd >= 0, "call mk_bin_writer_begin first");
    auto it = w->index.find(name);
    if (it == w->index.end()) { mk_set_error("mk_bin_writer_put: no tensor named %s was added", name); return MK_ERR_ARG; }
    const mk_bin_entry_rec &e = w->entries[it->second];
    if (e.size != size) {
        mk_set_error("mk_bin_writer_put: %s holds %llu bytes, got %llu", name, (unsigned long long)e.size, (unsigned long long)size);
        return MK_ERR_ARG;
    }
    if (!write_all(w->fd, data, (size_t)size, e.off)) { mk_set_error("mk_bin_writer_put: write failed"); return MK_ERR_STATE; }
    return MK_OK;
}
extern "C" int32_t mk_bin_writer_finish(mk_bin_writer *w) {
    if (!w) return MK_OK;
    if (w->fd >= 0) close(w->fd);
    delete w;
    return MK_OK;
}
