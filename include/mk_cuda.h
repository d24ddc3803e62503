/*
 * mk_cuda.h - C ABI of libmk_b200.so: the quantized decode hot path of the
 * microkimi engine as hand-written CUDA for NVIDIA B200 (sm_100a).
 *
 * This is the surface a `src/cuda.rs` `extern "C"` block binds.  It takes the
 * place of the engine's Metal hook (src/metal.rs) and of the CPU operators that
 * hook stands in for; each entry point names the reference interface it
 * replaces (file:line within the reference project).
 *
 * Conventions
 *  - every function returns an int32 status: MK_OK (0) or a negative MK_ERR_*;
 *    nothing throws, aborts or falls back to a CPU path.  mk_last_error()
 *    gives a thread-local message for the last failure on this thread.
 *  - plain pointers and sizes only.  `_dev` variants take DEVICE pointers of the
 *    context's GPU and enqueue on the context's stream without synchronizing;
 *    the others take HOST pointers, copy in, run, copy out and synchronize, like
 *    metal::gpu_matvec_fp4 does (src/metal.rs:943-1018).
 *  - a context is bound to one GPU and is thread-compatible, not re-entrant:
 *    concurrent callers must serialize, as the Metal path does on its io mutex
 *    (src/metal.rs:432-437).
 *  - weights are uploaded (and re-tiled for the tensor-core fragment order)
 *    ONCE at registration, like the Metal weight cache (src/metal.rs:387-396);
 *    the caller keeps ownership of the host bytes.  Values are unchanged:
 *    mk_weight_export() returns the registered bytes in their original layout.
 */
#ifndef MK_CUDA_H
#define MK_CUDA_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MK_OK            0
#define MK_ERR_ARG      -1   /* bad pointer, size or handle                     */
#define MK_ERR_CUDA     -2   /* a CUDA runtime call failed                      */
#define MK_ERR_OOM      -3   /* device allocation failed                        */
#define MK_ERR_STATE    -4   /* call not valid in the object's current state    */
#define MK_ERR_TIMEOUT  -5   /* a bounded device-side wait ran out              */
#define MK_ERR_UNSUPPORTED -6

typedef struct mk_ctx    mk_ctx;
typedef struct mk_weight mk_weight;
typedef struct mk_moe    mk_moe;
typedef struct mk_mla    mk_mla;

/* How the f32 activation enters the integer block dot.
 * MK_ACT_Q8   : q8_0, one int8 per element - the engine's default path
 *               (src/mxfp4.rs:480-487 -> src/q8.rs:49-69).
 * MK_ACT_Q8X2 : two int8 limbs per element (15-bit activation), for callers
 *               that want to stay close to the exact-f32 path
 *               (src/mxfp4.rs:488-539) at the same memory traffic. */
#define MK_ACT_Q8    0
#define MK_ACT_Q8X2  1
/* MoE layer only (mk_moe_desc.act_mode): calls of 4 or more token rows run the experts as block-scaled tensor-core
 * products (tcgen05.mma kind::mxf4, both operands packed FP4): E2M1 weights with their ue8m0 scales as registered, the
 * activations as six E2M1 limbs with power-of-two block scales (every limb takes the remainder down by a factor of 4;
 * what is left after six is at most 1/12288 of the block's largest element).  Results track the engine's exact-f32
 * path (src/mxfp4.rs:488-539) to ~1e-5 of max |y|.  The experts' input width and inter must be multiples of 256
 * (mk_moe_create refuses the mode otherwise).
 * A layer created in this mode keeps a second copy of its experts on the device (blocked into the 16 KB boxes a step
 * loads): twice the expert memory.  Calls of fewer than 4 rows, and the expert-parallel step, run the ordinary q8 kernels. */
#define MK_ACT_FP4X6 2
/* OR into act_mode: accumulate the per-block terms of every output strictly in
 * ascending block order with separate multiply and add, reproducing the CPU
 * result of src/mxfp4.rs:409-418 / src/model.rs:337-347 bit for bit (slower). */
#define MK_ACT_STRICT 0x100

/* q8_0 scale storage.  F32 is the engine's layout (src/q8.rs:26-29,
 * src/model.rs:261-266); F16 halves the scale stream. */
#define MK_SCALE_F32 0
#define MK_SCALE_F16 1

/* ---- context ---------------------------------------------------------- */
/* Replaces metal::gpu_available / init_ctx (src/metal.rs:445-452): binds GPU
 * `device`; fails (no fallback) when it is not an sm_100 part. */
int32_t mk_init(int32_t device, mk_ctx **out);
int32_t mk_shutdown(mk_ctx *ctx);
const char *mk_last_error(void);
/* Stream used by every later call on this context (a cudaStream_t; NULL is the
 * CUDA legacy default stream).  Until this is called the context runs on a
 * non-blocking stream of its own. */
int32_t mk_set_stream(mk_ctx *ctx, void *cuda_stream);
int32_t mk_sync(mk_ctx *ctx);
/* Device-to-device copy on the context's stream (for results the library hands out as device
 * pointers, e.g. the gathered logits). */
int32_t mk_memcpy_dev(mk_ctx *ctx, void *dst, const void *src, uint64_t bytes);
/* Number of kernels this context has launched since mk_init. */
int64_t mk_launch_count(mk_ctx *ctx);
int32_t mk_device_info(mk_ctx *ctx, int32_t *sm_count, int32_t *cc_major, int32_t *cc_minor, uint64_t *mem_bytes);
/* Device-side status word: 0, or the first MK_ERR_* a kernel recorded (bounded
 * waits, range checks).  Reading it synchronizes the stream and clears the word. */
int32_t mk_status_word(mk_ctx *ctx, int32_t *out);

/* Tuning knobs, for measurement only (defaults are chosen per shape):
 *   "force_ks" : K split of the matvec kernels, one of 0 (auto), 1, 2, 4, 8.
 *   "pdl": 1 (default) = the one-token matvec is launched behind its activation quantizer with programmatic stream
 *             serialization: its first weight loads run while the quantizer still does, it waits (griddepcontrol.wait)
 *             before its first read of the quantized activations.  0 = ordinary launch order (same results).
 *   "moe_no_fuse": 1 = small-batch MoE calls use the separate router / top-k / plan /
 *                quantize launches of large batches instead of the fused router kernel.
 *   "mla_max_split": upper bound on the KV splits of an attention call, 0 = automatic
 *                (fewer splits = more tiles per CTA; used by the tests).
 *   "kda_smem": 1 = the KDA step stages S in shared memory (short loops) also for kda_dim 64 and 128,
 *                where the default keeps each column in registers (fully unrolled); same bits.
 *   "mla_no_t5": 1 = absorbed-layout attention on the mma.sync kernel instead of the
 *                tcgen05 (tensor-memory) kernel.
 *   "mla_strict": 1 = per-head-layout attention on a one-warp-per-head kernel that forms every sum in the CPU's
 *                order (64-position tiles, src/model.rs:1804-1908): for parity runs, not for speed.
 *   "mla_no_tc": 1 = run attention on the generic one-warp-per-head CUDA-core kernel
 *                instead of the specialised ones (tensor-core kernel of the absorbed
 *                layout, 8-heads-per-CTA kernel of the per-head layout at vd = 128). */
int32_t mk_set_option(mk_ctx *ctx, const char *name, int64_t value);

/* Per-category kernel timing with CUDA events on the context's stream, the
 * counterpart of the engine's Prof accumulators (src/model.rs:791-835).
 * Categories: MK_PROF_*.  mk_prof_read synchronizes the stream, then returns the
 * number of timed launches and their summed device time since the last enable. */
#define MK_PROF_MATVEC_MXFP4 0
#define MK_PROF_LM_HEAD      1
#define MK_PROF_ROUTER       2
#define MK_PROF_EXPERTS      3
#define MK_PROF_MLA          4
#define MK_PROF_OTHER        5
#define MK_PROF_NCAT         6
int32_t mk_prof_enable(mk_ctx *ctx, int32_t on);
int32_t mk_prof_read(mk_ctx *ctx, int32_t category, int64_t *launches, double *total_ms);

/* ---- weights ---------------------------------------------------------- */
/* MXFP4 matrix: packed u8 [rows, cols/2] (low nibble = even column) and ue8m0
 * scales u8 [rows, cols/32] - BinFile::mxfp4_parts (src/weights.rs:619-626),
 * the arguments of mxfp4::matvec_packed (src/mxfp4.rs:458).  cols % 32 == 0.
 * src_on_device != 0: the pointers are device pointers (copied, not adopted). */
int32_t mk_weight_mxfp4(mk_ctx *ctx, const uint8_t *packed, const uint8_t *scales,
                        int64_t rows, int64_t cols, int32_t src_on_device, mk_weight **out);
/* Row-wise q8_0 copy of an f32 matrix, built on the GPU, bit-identical to
 * Q8Head::from_f32 (src/model.rs:274-286) for MK_SCALE_F32. */
int32_t mk_weight_q8_from_f32(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols,
                              int32_t scale_type, int32_t src_on_device, mk_weight **out);
/* Already-quantized q8_0 rows: q i8 [rows, cols], scales [rows, cols/32]
 * (f32 or IEEE half according to scale_type). */
int32_t mk_weight_q8(mk_ctx *ctx, const int8_t *q, const void *scales, int64_t rows, int64_t cols,
                     int32_t scale_type, int32_t src_on_device, mk_weight **out);
/* A dense f32 matrix [rows, cols] (row-major), as the engine's matvec consumes it
 * (src/model.rs:199; the Metal seam uploads the same bytes, src/metal.rs:750). */
int32_t mk_weight_f32(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols, int32_t src_on_device, mk_weight **out);
/* A VQ1 matrix (src/quant.rs:17-18, 313-346): codebook f32 [256, 16] and one index byte per 16
 * weights, indices u8 [rows, cols/16]; W[r, 16 v + j] = codebook[indices[r, v]][j]. */
int32_t mk_weight_vq1(mk_ctx *ctx, const float *codebook, const uint8_t *indices, int64_t rows, int64_t cols,
                      int32_t src_on_device, mk_weight **out);
int32_t mk_weight_free(mk_ctx *ctx, mk_weight *w);
/* Bytes held on the device for this weight (values + scales). */
int64_t mk_weight_bytes(const mk_weight *w);
/* Copies the registered bytes back to HOST memory in their original layout
 * (packed/q first, then scales); either pointer may be NULL. */
int32_t mk_weight_export(mk_ctx *ctx, const mk_weight *w, void *values, void *scales);
/* mxfp4::dequant (src/mxfp4.rs:19-31) on the GPU: f32 [rows, cols] to HOST. */
int32_t mk_dequant_mxfp4(mk_ctx *ctx, const mk_weight *w, float *out);

/* dequant::dequant_fp8 (src/dequant.rs:12-41) on the GPU: e4m3fn bytes w [rows, cols] with one ue8m0
 * scale byte per 128 x 128 block (scales [ceil(rows/128), ceil(cols/128)]) -> f32 [rows, cols].
 * HOST in / HOST out; bit-identical (the DeepSeek spine weights, src/dequant.rs). */
int32_t mk_dequant_fp8(mk_ctx *ctx, const uint8_t *w, const uint8_t *scales, int64_t rows, int64_t cols, float *out);

/* mxfp4::dequant_any (src/mxfp4.rs:228-240) on the GPU: a raw blob of either MXFP4 flavour as it sits in a model file
 * (MK_DTYPE_MXFP4: packed || scales; MK_DTYPE_MXFP4SQ: packed || scales || smax, scale = ((q + 1) / 256)^2 * smax,
 * src/mxfp4.rs:140-158) -> f32 [rows, cols].  HOST in / HOST out; bit-identical. */
int32_t mk_dequant_mxfp4_blob(mk_ctx *ctx, int32_t dtype, const uint8_t *blob, int64_t rows, int64_t cols, float *out);

/* ---- activations ------------------------------------------------------ */
/* q8::quantize_q8_into (src/q8.rs:49-69) on the GPU, HOST in / HOST out:
 * x f32 [n] (n % 32 == 0) -> q i8 [n], scales f32 [n/32].  Bit-identical. */
int32_t mk_quantize_q8(mk_ctx *ctx, const float *x, int64_t n, int8_t *q, float *scales);

/* ---- matrix x vector -------------------------------------------------- */
/* mxfp4::matvec_packed / metal::gpu_matvec_fp4 (src/mxfp4.rs:458-539,
 * src/metal.rs:943-1018): y[b, r] = sum_c W[r, c] * x[b, c] for b < batch.
 * x f32 [batch, cols], y f32 [batch, rows]. */
int32_t mk_matvec_mxfp4(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode);
int32_t mk_matvec_mxfp4_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode);
/* No counterpart in the reference.  Same result as mk_matvec_mxfp4_dev, for hosts that
 * must not allocate device memory once they are running: an engine that has handed
 * all of HBM to its own weight and KV-cache pools (a late workspace cudaMalloc can
 * fail there), or a decode loop that cannot afford the device-wide synchronization a
 * cudaMalloc implies.  The quantized activations go to a fixed 144 KiB array inside
 * the library's device image instead of a grown workspace; the call makes no
 * cudaMalloc/cudaFree.  Limits: padded cols <= 16384 and batch <= 8 (<= 4 with
 * MK_ACT_Q8X2); larger calls return MK_ERR_ARG.  The first call on a device looks the
 * array's device address up, so make that call before any stream capture.  All
 * calls share the array: two calls that overlap on the GPU (different streams or
 * contexts of one process) race; calls on one stream are ordered and safe. */
int32_t mk_matvec_mxfp4_noalloc_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch, int32_t act_mode);
/* Q8Head::matvec + the greedy pick of top_k_probs (src/model.rs:290-335,
 * 3271-3291): y f32 [batch, rows]; argmax (optional, int32 [batch]) = first
 * index attaining the maximum of each row of y. */
int32_t mk_matvec_q8(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch,
                     int32_t act_mode, int32_t *argmax);
int32_t mk_matvec_q8_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch,
                         int32_t act_mode, int32_t *argmax);

/* model::matvec / metal::gpu_matvec (src/model.rs:199-247, src/metal.rs:750): dense
 * f32 y[b, r] = dot(W[r], x[b]) with the engine's dot() order (src/model.rs:63-82:
 * 8 accumulators, separate multiply and add), i.e. the CPU's bits.
 * x f32 [batch, cols], y f32 [batch, rows]. */
int32_t mk_matvec_f32(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch);
int32_t mk_matvec_f32_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch);
/* quant::matvec_vq / lutgemv::matvec_vq_lut (src/quant.rs:340-346, src/lutgemv.rs:208-238): the VQ1
 * matvec by lookup table, bit-identical to both of the engine's paths (table entries and rows
 * accumulate in the engine's ascending order). x f32 [batch, cols], y f32 [batch, rows]. */
int32_t mk_matvec_vq1(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch);
int32_t mk_matvec_vq1_dev(mk_ctx *ctx, const mk_weight *w, const float *x, float *y, int32_t batch);
/* rmsnorm (src/model.rs:599-605) on DEVICE rows: out[i] = (x[i] * inv) * w[i] with
 * inv = 1 / sqrt(dot(x, x) / len + eps); x, out f32 [n, len], w f32 [len].  Bit-identical. */
int32_t mk_rmsnorm_dev(mk_ctx *ctx, const float *x, const float *w, int32_t n, int32_t len, float eps, float *out);
/* a[i] *= sigmoid(g[i]) on DEVICE vectors: the output gate of mla_forward (src/model.rs:2015-2019). */
int32_t mk_sigmoid_gate_dev(mk_ctx *ctx, float *a, const float *g, int64_t count);

/* ---- KDA decode step (src/model.rs:1066-1228) ----------------------------
 * The part of kda_forward between its projections and o_proj, one token per call, with the
 * layer's state resident on the device: the conv windows of q, k, v (kconv - 1 previous raw
 * inputs each, src/model.rs:1070-1085) and the matrix S [heads][dim][dim] (:1114-1156).
 * mk_kda_create copies the HOST parameter arrays and zeroes the state (a new sequence). */
typedef struct mk_kda mk_kda;
typedef struct {
    int32_t heads, dim, kconv;                /* cfg.kda_heads, kda_dim (<= 1024), kda_conv (4; 2..16) */
    float gate_lb, rms_eps;                   /* cfg.gate_lb (-5), cfg.rms_eps */
    const float *q_conv, *k_conv, *v_conv;    /* [heads * dim][kconv], weight kconv - 1 on the current input */
    const float *a_log, *dt_bias, *o_norm;    /* [dim], [heads * dim], [dim] */
} mk_kda_desc;
int32_t mk_kda_create(mk_ctx *ctx, const mk_kda_desc *desc, mk_kda **out);
void    mk_kda_free(mk_ctx *ctx, mk_kda *kda);
int32_t mk_kda_reset(mk_ctx *ctx, mk_kda *kda);   /* zero state: KdaCache::new */
/* DEVICE f32 inputs: the raw projections q, k, v [heads * dim], g_low = f_b(f_a(x)) [heads * dim],
 * beta_raw = b_proj(x) [heads] (before the sigmoid), g2 = g_proj(x) [heads * dim].  Does, in the
 * engine's order: conv + SiLU of q, k, v and the window shift; per-head L2 norm of q (times
 * dim^-0.5) and k; gate = gate_lb * sigmoid(exp(A_log) * (g_low + dt_bias)); the recurrence
 * (decay, delta = v - k^T S, S += (beta k) (x) delta, o = q^T S); the gated per-head RMS norm.
 * o f32 [heads * dim] is the input of o_proj.  Sums keep the engine's order; exp is rounded once
 * from double precision, so results equal the CPU's except where two correctly-rounded-in-
 * practice expf differ (tests hold it to 1e-6 relative). */
int32_t mk_kda_step_dev(mk_ctx *ctx, mk_kda *kda, const float *q_raw, const float *k_raw, const float *v_raw,
                        const float *g_low, const float *beta_raw, const float *g2, float *o);
/* n_tok consecutive positions in one call (the engine's kda_prefill loop, src/model.rs:1281-1300): token t reads its
 * q / k / v / g2 / beta rows t * ld_x floats after the given pointers, its g_low row t * ld_g floats on, and writes its
 * output row t * ld_o floats on.  Bit-identical to n_tok calls of mk_kda_step_dev; the state is read and written once.
 * From 4 positions on (widths 64 and 128) the work that does not depend on the previous position runs for all positions
 * side by side and only the recurrence walks them (three launches); that form keeps its intermediates in the
 * context's workspace, which may grow on the first call of a size (an allocation: not inside stream capture). */
int32_t mk_kda_steps_dev(mk_ctx *ctx, mk_kda *kda, int32_t n_tok, const float *q_raw, const float *k_raw, const float *v_raw,
                         const float *g_low, const float *beta_raw, const float *g2, float *o, int64_t ld_x, int64_t ld_g, int64_t ld_o);
/* State to / from HOST memory (cache snapshots for speculative rollback, src/spec.rs:214, 294-299;
 * .mkmem files): s [heads][dim][dim]; conv [3 (q, k, v)][kconv - 1][heads * dim], oldest input first
 * (the layout of KdaCache::conv_q / conv_k / conv_v). */
int32_t mk_kda_export(mk_ctx *ctx, mk_kda *kda, float *s, float *conv);
int32_t mk_kda_import(mk_ctx *ctx, mk_kda *kda, const float *s, const float *conv);
/* attn_res (src/model.rs:625-669) on DEVICE rows: softmax over the RMS-normed scores of b block
 * rows (blocks + i * ld, i < b) and the prefix row, output = the probability-weighted sum of the
 * RAW rows; w = norm.weight * proj.weight; all f32 [d].  Same sum orders as the engine. */
int32_t mk_attn_res_dev(mk_ctx *ctx, const float *prefix, const float *blocks, int64_t ld, int32_t b, const float *w,
                        int32_t d, float eps, float *out);

/* ---- vocabulary-sharded lm_head over the GPUs of one node ---------------
 * No counterpart in the reference (a single-process engine).  Rank r registers rows
 * [row0, row0 + rows) of the lm_head (mk_weight_q8_from_f32 on its slice); one call then
 * computes the shard's logits into this rank's gather buffer and one exchange kernel
 * pushes them into the gather buffers of all other ranks over NVLink (peer memory, plain
 * stores; no collective library call on the path), sends this rank's (maximum, index)
 * pair along, waits - bounded, MK_ERR_TIMEOUT in the status word if a rank never arrives -
 * until every rank has delivered, and picks the token: the complete f32 logits
 * [batch, vocab] are then in this rank's buffer.
 * The result is bit-identical to one GPU computing the whole matrix.
 *   mk_gather_create : allocates this rank's buffer, returns a 64-byte handle for it
 *   mk_gather_connect: opens the other ranks' buffers from their handles ([world][64] by
 *                      rank; exchange them with any host-side means).  An all-zero handle
 *                      stands for a rank that never joined: its share is written to a local
 *                      stand-in buffer, its flag never arrives, and every call reports
 *                      MK_ERR_TIMEOUT in the status word after the bounded wait (about half
 *                      a second) instead of hanging
 * world <= 8, max_batch <= 2 (decode).  Every rank must make the same sequence of calls.
 * After a timeout: the two-buffer rule (a rank is at most one step ahead of a peer that still reads) holds only while
 * no wait runs out.  A rank whose wait ran out goes on and could, two steps later, overwrite a buffer that a merely
 * slow peer still reads - and only the rank that timed out sees MK_ERR_TIMEOUT.  So every rank reads mk_status_word
 * after each step (or each token); on MK_ERR_TIMEOUT on any rank, all ranks stop calling, free the gather objects
 * (mk_gather_free) and build new ones.  The same holds for mk_moe_ep below. */
typedef struct mk_gather mk_gather;
int32_t mk_gather_create(mk_ctx *ctx, int32_t rank, int32_t world, int64_t vocab, int32_t max_batch, mk_gather **out,
                         uint8_t *handle);
int32_t mk_gather_connect(mk_ctx *ctx, mk_gather *g, const uint8_t *handles);
int32_t mk_gather_free(mk_ctx *ctx, mk_gather *g);
/* x f32 [batch, cols] on the DEVICE (the same on every rank); *logits receives a DEVICE pointer to the
 * complete [batch, vocab] logits (valid until the call after next); argmax (optional, DEVICE int32
 * [batch]) = first index of the maximum over the whole vocabulary. */
int32_t mk_matvec_q8_gather_dev(mk_ctx *ctx, const mk_weight *w, mk_gather *g, const float *x, int32_t batch, int64_t row0,
                                const float **logits, int32_t *argmax);
/* The token-only step of greedy decode (the pick of src/model.rs:3277-3290 needs the token, not the other shards'
 * logits): the ranks exchange only their (maximum, index) pairs, 16 bytes per rank and token.  argmax (required,
 * DEVICE int32 [batch]) is the same on every rank; *local_rows (optional) receives a DEVICE pointer to this
 * rank's rows of the logits, [batch] rows of w->rows floats, `vocab` floats apart (valid until the call after
 * next).  All ranks must make the same kind of call in a step. */
int32_t mk_matvec_q8_gather_token_dev(mk_ctx *ctx, const mk_weight *w, mk_gather *g, const float *x, int32_t batch, int64_t row0,
                                      const float **local_rows, int32_t *argmax);

/* ---- MoE layer ---------------------------------------------------------
 * One call per layer instead of 3 matvecs per selected expert: replaces
 * moe_forward / ds_moe wholesale (src/model.rs:2150-2380, src/deepseek.rs:1038-1108).
 *   router     : logits = gate_w x in the engine's dot() order (bit-exact); bias for
 *                selection only; top-k by (key desc, index asc)
 *     MK_ROUTER_SIGMOID      : score = sigmoid(logit), weights = score / (sum + 1e-20)
 *                              (K3 noaux_tc, src/model.rs:2153-2173)
 *     MK_ROUTER_SQRT_SOFTPLUS: score = sqrt(softplus(logit)), weights = score / sum * route_scale
 *                              (DeepSeek gate_forward, src/deepseek.rs:16-58; its hash layers,
 *                              which read the ids from a table, go through mk_moe_experts_dev)
 *   experts    : MXFP4 w1/w3 -> act -> w2 through the q8 integer path
 *     MK_MOE_SWIGLU_CLAMP: act = (wgt * silu(min(g, limit))) * clamp(u, +-limit), the routing
 *                weight folded in BEFORE w2, outputs summed in slot order, plus one
 *                unweighted MXFP4 shared expert `shared`      (src/deepseek.rs:1083-1106)
 *     MK_MOE_SITU: the K3 body (src/model.rs:2202-2380): act = situ(g, u), y = sum of
 *                wgt_i * o_i in slot order.  With `latent` > 0 the experts work on
 *                h = routed_down x (w1, w3: [inter, latent], w2: [latent, inter]) and the
 *                layer returns routed_up rmsnorm(y, routed_norm, rms_eps); the f32 shared
 *                expert `shared_f32` (SiTU MLP on the layer input) is added to the result.
 * Expert index n_experts names the MXFP4 shared expert. */
#define MK_MOE_SWIGLU_CLAMP 0
#define MK_MOE_SITU         1
#define MK_ROUTER_SIGMOID       0
#define MK_ROUTER_SQRT_SOFTPLUS 1
typedef struct {
    int32_t n_experts, top_k, d, inter;
    float   swiglu_limit;
    int32_t activation;              /* MK_MOE_* */
    const float *gate_w;             /* HOST f32 [n_experts, d]; NULL: no router (experts only) */
    const float *gate_b;             /* HOST f32 [n_experts]; NULL = zeros */
    const mk_weight *const *experts; /* [n_experts * 3] = w1 [inter,d], w2 [d,inter], w3 [inter,d] per expert;
                                        NULL entries = expert not resident on this GPU (expert parallel) */
    const mk_weight *shared[3];      /* MXFP4 shared expert w1, w2, w3; all NULL = none here */
    int32_t router;                  /* MK_ROUTER_* */
    float   route_scale;             /* MK_ROUTER_SQRT_SOFTPLUS only; 0 is read as 1 */
    int32_t latent;                  /* MK_MOE_SITU: routed_hidden, the width the experts work on; 0 = d */
    float   rms_eps;
    const mk_weight *routed_down;    /* f32 [latent, d]   (mk_weight_f32) */
    const mk_weight *routed_up;      /* f32 [d, latent] */
    const float *routed_norm;        /* HOST f32 [latent] */
    const mk_weight *shared_f32[3];  /* f32 shared expert: gate [si, d], down [d, si], up [si, d]; all NULL = none */
    int32_t act_mode;                /* MK_ACT_Q8 (0); MK_ACT_FP4X6 (see above); or MK_ACT_Q8 | MK_ACT_STRICT: the expert matvecs add their block terms in the
                                        CPU's order (src/mxfp4.rs:409-418), so no q8 rounding of an activation can differ from the
                                        CPU's; slower on wide experts (no K split) */
} mk_moe_desc;
int32_t mk_moe_create(mk_ctx *ctx, const mk_moe_desc *desc, mk_moe **out);
int32_t mk_moe_free(mk_ctx *ctx, mk_moe *moe);
/* Router only: ids int32 [n, top_k] and weights f32 [n, top_k] in slot order;
 * logits (optional) f32 [n, n_experts]. */
int32_t mk_moe_route(mk_ctx *ctx, mk_moe *moe, const float *x, int32_t n_tokens, int32_t *ids, float *weights, float *logits);
int32_t mk_moe_route_dev(mk_ctx *ctx, mk_moe *moe, const float *x, int32_t n_tokens, int32_t *ids, float *weights, float *logits);
/* Whole layer for n_tokens rows x f32 [n, d] -> out f32 [n, d]; ids / weights optional outputs. */
int32_t mk_moe_forward(mk_ctx *ctx, mk_moe *moe, const float *x, int32_t n_tokens, float *out, int32_t *ids, float *weights);
int32_t mk_moe_forward_dev(mk_ctx *ctx, mk_moe *moe, const float *x, int32_t n_tokens, float *out, int32_t *ids, float *weights);
/* Grouped experts on an explicit list of (row of x, expert, routing weight) pairs -
 * the piece that runs on the expert's owner under expert parallelism:
 * outs f32 [n_pairs, d] = expert(pair_expert[p]) applied to x[pair_row[p]].  DEVICE pointers. */
int32_t mk_moe_experts_dev(mk_ctx *ctx, mk_moe *moe, const float *x, int32_t n_rows, const int32_t *pair_row,
                           const int32_t *pair_expert, const float *pair_weight, int32_t n_pairs, float *outs);
/* out[t] = sum over slots (in slot order) of outs[t * slots + s]: the fixed-order
 * combination after the expert jobs (src/deepseek.rs:1095-1106).  DEVICE pointers. */
int32_t mk_moe_combine_dev(mk_ctx *ctx, const float *outs, int32_t n_tokens, int32_t slots, int32_t d, float *out);

/* ---- expert-parallel MoE over the GPUs of one node (decode) ----------------
 * No counterpart in the reference (a single-process engine).  Token rows are replicated on
 * every rank (<= 16 rows); the layer object of a rank holds only that rank's routed experts
 * (NULL entries for the others) plus the shared expert.  One call routes all rows on every
 * rank (identical ids), runs the (row, expert) pairs whose expert is resident - the shared
 * expert of row t on rank t % world -, pushes their output rows into the (row, slot) table
 * of every other rank over NVLink (peer memory, no collective library call), waits -
 * bounded, MK_ERR_TIMEOUT in the status word otherwise - for the other ranks' rows and sums
 * the table in slot order: the result is bit-identical to one GPU holding all experts.
 * Create / connect work like mk_gather_create / mk_gather_connect (64-byte handles). */
typedef struct mk_moe_ep mk_moe_ep;
int32_t mk_moe_ep_create(mk_ctx *ctx, const mk_moe *moe, int32_t rank, int32_t world, int32_t max_tokens, mk_moe_ep **out,
                         uint8_t *handle);
int32_t mk_moe_ep_connect(mk_ctx *ctx, mk_moe_ep *ep, const uint8_t *handles);
int32_t mk_moe_ep_free(mk_ctx *ctx, mk_moe_ep *ep);
/* Arguments as mk_moe_forward_dev; every rank passes the same x and must make the same sequence of calls. */
int32_t mk_moe_forward_ep_dev(mk_ctx *ctx, mk_moe *moe, mk_moe_ep *ep, const float *x, int32_t n_tokens, float *out, int32_t *ids,
                              float *weights);

/* ---- q8_0 MLA KV cache and decode attention ------------------------------
 * Replaces MlaCache::push and mla_attn_flash_q8_mqa (src/model.rs:1583-1618,
 * 1804-1908).  One object holds n_seqs independent caches of max_positions each.
 *
 * MK_MLA_PER_HEAD (the engine's layout, src/model.rs:765-781): per position the
 *   nope part of K and all of V are q8_0 per head (int8 + one f32 scale per 32),
 *   the rope part of K is kept f32 and stored once (from head 0).
 *   append: k_row f32 [n_heads, nope+rope], v_row f32 [n_heads, vd]
 *   attend: q f32 [n_heads, nope+rope] -> out f32 [n_heads, vd]
 * MK_MLA_ABSORBED (no counterpart in the engine): one shared q8_0 latent row of
 *   width nope (= kv_lora_rank + rope dim, all quantized; `rope` must be 0) per
 *   position; every head attends to the same rows and V is the first vd columns.
 *   append: k_row f32 [nope], v_row ignored
 *   attend: q f32 [n_heads, nope] (already absorbed) -> out f32 [n_heads, vd]
 * Attention follows the engine's recipe: the query's nope part is quantized to
 * q8_0, score = (rope dot + sum_g (qs*ks)*idot) * scale, softmax over positions
 * 0..=pos, V dequantized as int8 * scale. */
#define MK_MLA_PER_HEAD 0
#define MK_MLA_ABSORBED 1
typedef struct {
    int32_t layout;         /* MK_MLA_* */
    int32_t n_heads, nope, rope, vd;
    int32_t max_positions;  /* per sequence */
    int32_t n_seqs;
} mk_mla_desc;
int32_t mk_mla_create(mk_ctx *ctx, const mk_mla_desc *desc, mk_mla **out);
int32_t mk_mla_free(mk_ctx *ctx, mk_mla *mla);
int32_t mk_mla_reset(mk_ctx *ctx, mk_mla *mla, int32_t seq);            /* forget the positions of one sequence (-1: all) */
int32_t mk_mla_positions(mk_ctx *ctx, const mk_mla *mla, int32_t seq);  /* positions held, or a negative status */
/* MlaCache::push for n consecutive positions of one sequence (rows concatenated). */
int32_t mk_mla_append(mk_ctx *ctx, mk_mla *mla, int32_t seq, const float *k_rows, const float *v_rows, int32_t n);
int32_t mk_mla_append_dev(mk_ctx *ctx, mk_mla *mla, int32_t seq, const float *k_rows, const float *v_rows, int32_t n);
/* mla_attn_flash_q8_mqa over positions 0..=pos of sequence seq (pos < positions held). */
int32_t mk_mla_attend(mk_ctx *ctx, mk_mla *mla, int32_t seq, const float *q, int32_t pos, float scale, float *out);
/* All sequences at once, each over all the positions it holds: q f32 [n_seqs, n_heads, qdim],
 * out f32 [n_seqs, n_heads, vd].  DEVICE pointers. */
int32_t mk_mla_attend_batch_dev(mk_ctx *ctx, mk_mla *mla, const float *q, float scale, float *out);
/* One decode step of one sequence as launches whose shape does not depend on the position, so that a CUDA graph
 * holding them can be replayed token after token: MlaCache::push of one position at the sequence's device-side
 * count, then mla_attn_flash_q8_mqa over everything held (grids sized for max_positions; a full cache is
 * MK_ERR_STATE from the call, or in the status word when replayed).  DEVICE pointers, shapes as mk_mla_append /
 * mk_mla_attend.  A caller that replays a captured step must make no other append to that sequence in between. */
int32_t mk_mla_decode_step_dev(mk_ctx *ctx, mk_mla *mla, int32_t seq, const float *k_row, const float *v_row, const float *q,
                               float scale, float *out);
/* n consecutive positions of one sequence in one go - the cache and attention part of mla_prefill
 * (src/model.rs:2033-2115): k_rows / v_rows [n] rows as mk_mla_append takes them are appended at the sequence's
 * device-side count, then query row b (q_rows [n][n_heads][nope + rope]) attends to the positions up to its own;
 * out [n][n_heads * vd].  Per (row, head) the arithmetic of n calls of mk_mla_decode_step_dev - the same bits in
 * the strict attention mode - with the launches shared.  DEVICE pointers.  May grow the object's scratch buffers
 * (allocates; not for stream capture). */
int32_t mk_mla_prefill_dev(mk_ctx *ctx, mk_mla *mla, int32_t seq, const float *k_rows, const float *v_rows, const float *q_rows,
                           int32_t n, float scale, float *out);
/* Cache contents of one sequence back to HOST memory in the engine's layout
 * (src/model.rs:765-781), any pointer may be NULL:
 *  PER_HEAD: kq i8 [n, H, nope], ks f32 [n, H, nope/32], kr f32 [n, rope], vq i8 [n, H, vd], vs f32 [n, H, vd/32]
 *  ABSORBED: kq i8 [n, nope], ks f32 [n, nope/32]; the others are not written. */
int32_t mk_mla_export(mk_ctx *ctx, const mk_mla *mla, int32_t seq, int8_t *kq, float *ks, float *kr, int8_t *vq, float *vs);

/* ---- the engine's weight file (MKIM0001 / MKIM0002) -------------------------
 * BinFile::open / read_config / BinWriter (src/weights.rs:1-64, 66-186, 390-590): magic, optional JSON
 * configuration block, a directory of (name, dtype, dims, offset, size) and the blobs (64-byte aligned,
 * routed-expert matrices 4096-byte aligned).  The reader maps the file read-only; pointers it hands out
 * stay valid until mk_bin_close.  MKIM0001 files carry the historical micro configuration. */
#define MK_DTYPE_F32     0
#define MK_DTYPE_MXFP4   1   /* blob = packed [r, c/2] then ue8m0 scales [r, c/32] */
#define MK_DTYPE_I32     2
#define MK_DTYPE_VQ1     3
#define MK_DTYPE_MXFP4SQ 4
/* Config (src/config.rs:8-43).  has_layer_lists / is_deepseek are set by the reader when the file's
 * configuration names explicit per-layer type lists or the DeepSeek architecture; mk_model_open
 * refuses such files (MK_ERR_UNSUPPORTED). */
typedef struct {
    uint32_t n_layers, d, vocab, n_experts, top_k, n_shared;
    uint32_t kda_heads, kda_dim, kda_conv, kda_fa;
    float    gate_lb;
    uint32_t mla_heads, mla_qa, mla_kva, mla_nope, mla_rope, mla_v;
    uint32_t routed_hidden, moe_inter, shared_inter, dense_inter, attn_res_block, first_k_dense;
    float    rms_eps;
    uint32_t eos_id, bos_id;
    uint32_t has_layer_lists, is_deepseek;
} mk_model_config;
void mk_model_config_default(mk_model_config *c);     /* Config::microkimi (src/config.rs:47-79) */
typedef struct mk_bin mk_bin;
typedef struct mk_bin_writer mk_bin_writer;
int32_t mk_bin_open(const char *path, mk_bin **out);  /* a truncated or malformed file is MK_ERR_ARG, never a crash */
int32_t mk_bin_close(mk_bin *b);
int32_t mk_bin_config(const mk_bin *b, mk_model_config *out);
int64_t mk_bin_count(const mk_bin *b);
/* Tensor by name / by directory position: dtype, number of dims, dims[4], HOST pointer to the blob, its size.
 * Any output pointer may be NULL. */
int32_t mk_bin_find(const mk_bin *b, const char *name, int32_t *dtype, int32_t *ndims, uint32_t *dims, const void **data,
                    uint64_t *size);
int32_t mk_bin_entry(const mk_bin *b, int64_t i, const char **name, int32_t *dtype, int32_t *ndims, uint32_t *dims,
                     const void **data, uint64_t *size);
/* Writer: add every tensor (directory order = call order), begin (lays the file out and writes header and
 * directory), put each blob, finish.  cfg == NULL writes MKIM0001, otherwise MKIM0002 with the JSON block. */
int32_t mk_bin_writer_create(const mk_model_config *cfg, mk_bin_writer **out);
int32_t mk_bin_writer_add(mk_bin_writer *w, const char *name, int32_t dtype, int32_t ndims, const uint32_t *dims);
int32_t mk_bin_writer_begin(mk_bin_writer *w, const char *path);
int32_t mk_bin_writer_put(mk_bin_writer *w, const char *name, const void *data, uint64_t size);
int32_t mk_bin_writer_finish(mk_bin_writer *w);       /* closes the file and frees the writer */

/* mxfp4::quantize (src/mxfp4.rs:38-138) on the GPU, DEVICE pointers: w f32 [rows, cols] -> packed u8
 * [rows, cols/2] + ue8m0 scales u8 [rows, cols/32].  search != 0: the three-candidate scale search
 * (the engine's default), 0: quantize_naive.  Bytes equal the CPU quantizer's. */
int32_t mk_quantize_mxfp4_dev(mk_ctx *ctx, const float *w, int64_t rows, int64_t cols, int32_t search, uint8_t *packed,
                              uint8_t *scales);

/* ---- the whole decode token ---------------------------------------------------
 * Model::from_bin + Model::forward (src/model.rs:906-1025, 2889-3031) for the K3 architecture with the
 * engine's defaults: q8_0 lm_head built at load, q8_0 MLA cache, MXFP4 experts through the q8 integer
 * path.  All weights and all layer state (KDA conv windows and S, MLA caches, AttnRes block rows) live
 * on the GPU; a token is a fixed sequence of launches that reads its position counters on the device,
 * so with use_graph the library captures it once as a CUDA graph and replays it per token. */
typedef struct mk_model mk_model;
typedef struct {
    int32_t max_positions;   /* tokens a sequence may hold (prompt + generated): capacity of every MLA cache */
    int32_t use_graph;       /* 1: replay the token as a CUDA graph from the third call on (the first call runs eagerly, the
                                second is recorded).  Needs a real stream: on the legacy default stream (mk_set_stream(NULL))
                                and while mk_prof_enable is on the token is launched kernel by kernel */
    int32_t strict;          /* 1: MoE experts and lm_head in MK_ACT_STRICT order (results closest to the CPU token) */
    int32_t keep_layer_hidden; /* 1: keep per-layer taps of the last token for mk_model_layer_hidden (the engine's
                                --dump-hidden / parity dumps, src/model.rs:2749-2823) */
    int32_t rank, world;     /* expert parallel + vocabulary-sharded lm_head over `world` GPUs (0 or 1: one GPU):
                                this rank keeps routed experts [rank E/world, (rank+1) E/world) of every MoE
                                layer and the same share of the lm_head rows; the rest of the model is replicated */
} mk_model_opts;
int32_t mk_model_open(mk_ctx *ctx, const mk_bin *bin, const mk_model_opts *opts, mk_model **out);
int32_t mk_model_free(mk_ctx *ctx, mk_model *m);
int32_t mk_model_reset(mk_ctx *ctx, mk_model *m);              /* new sequence: fresh caches, position 0 */
int32_t mk_model_positions(mk_ctx *ctx, const mk_model *m);    /* tokens consumed so far, or a negative status */
int64_t mk_model_weight_bytes(const mk_model *m);              /* device bytes held by weights */
int64_t mk_model_launches_per_token(const mk_model *m);        /* kernels in one token (as last enqueued) */
/* world > 1: handles [2][64] of this rank's exchange buffers (expert rows, logits), then connect with the
 * handles of all ranks [world][2][64] (as mk_gather_connect / mk_moe_ep_connect). */
int32_t mk_model_ep_handles(mk_ctx *ctx, mk_model *m, uint8_t *handles);
int32_t mk_model_ep_connect(mk_ctx *ctx, mk_model *m, const uint8_t *all_handles);
/* One token, enqueued on the context's stream without synchronizing.  token: DEVICE int32 (NULL = the
 * greedy pick of the previous call, which stays on the device); logits (optional): DEVICE f32 [vocab];
 * next (optional): DEVICE int32 = first index of the maximum logit (src/model.rs:3277-3290). */
int32_t mk_model_forward_dev(mk_ctx *ctx, mk_model *m, const int32_t *token, float *logits, int32_t *next);
/* HOST variant: copies the token in, runs, copies logits [vocab] (optional) and the pick (optional) out, synchronizes. */
int32_t mk_model_forward(mk_ctx *ctx, mk_model *m, int32_t token, float *logits, int32_t *next);
/* The greedy loop of run_turn (src/model.rs:3586-3593): n_prompt prompt tokens one by one, then n_new picks, each
 * fed back as the next token on the device; out_tokens HOST int32 [n_new]; one synchronization at the end. */
/* Layer-major prefill of n prompt tokens (Model::prefill, src/model.rs:3043-3260): per layer the projections, the
 * FFN and the AttnRes glue run once for all tokens, the KDA step and the MLA append + attention position by position
 * (the engine's sequential kda_prefill branch, src/model.rs:1291-1300: bit-identical to n single-token calls, and
 * so is this).  tokens: HOST int32 [n]; logits (optional, HOST f32 [vocab]) and next (optional, HOST) belong to the
 * LAST token.  Continues the sequence like mk_model_forward; any n, processed in pieces of 256 tokens. */
int32_t mk_model_prefill(mk_ctx *ctx, mk_model *m, const int32_t *tokens, int32_t n, float *logits, int32_t *next);
int32_t mk_model_generate(mk_ctx *ctx, mk_model *m, const int32_t *prompt, int32_t n_prompt, int32_t n_new, int32_t *out_tokens);
/* Per-layer taps of the last token, HOST f32 [n_layers][4][d] (needs opts.keep_layer_hidden): the attention block's
 * output, the residual stream after it, the FFN's output, the residual stream after the layer. */
int32_t mk_model_layer_hidden(mk_ctx *ctx, mk_model *m, float *out);
/* The final normed hidden state of the last token (the input of the lm_head), HOST f32 [d]: for parity checks. */
int32_t mk_model_last_hidden(mk_ctx *ctx, mk_model *m, float *hidden);

/* MlaCache::to_f32 / assign_f32 (src/model.rs:1620-1692): the cache of one sequence as f32 rows to HOST memory, and back
 * (state snapshots, .mkmem files, src/mkmem.rs:1-61).  PER_HEAD: k [n, H, nope + rope] (dequantized nope part, then the
 * shared rope row), v [n, H, vd]; ABSORBED: k [n, nope], v ignored.  Import empties the sequence and pushes the rows
 * again: a cache exported and imported lands on the same q8_0 grid (bytes and scales unchanged). */
int32_t mk_mla_export_f32(mk_ctx *ctx, const mk_mla *mla, int32_t seq, float *k, float *v);
int32_t mk_mla_import_f32(mk_ctx *ctx, mk_mla *mla, int32_t seq, const float *k, const float *v, int32_t n);

#ifdef __cplusplus
}
#endif
#endif
