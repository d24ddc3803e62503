"""The engine's weight container and the whole decode token, on top of the C ABI.

    BinFile(path)                 BinFile::open            src/weights.rs:471-590
    BinWriter(cfg)                BinWriter                src/weights.rs:66-186
    quantize_mxfp4(w)             mxfp4::quantize          src/mxfp4.rs:38-138 (on the GPU)
    Model(path, max_positions)    Model::load / ::forward  src/model.rs:874-1025, 2889-3031
    build_synthetic_bin(...)      `microkimi build` with every tensor on its Gaussian fallback branch
                                  (src/build.rs:344-576), values drawn on the GPU

Token ids and logits cross the boundary as plain integers / arrays; everything else stays on the GPU.
"""
import ctypes as C

import numpy as np

from . import lib as _l
from .ops import Context, _is_torch_cuda

DTYPES = {"f32": 0, "mxfp4": 1, "i32": 2, "vq1": 3, "mxfp4sq": 4}


def default_config(**over):
    """Config::microkimi (src/config.rs:47-79) with fields overridden by keyword."""
    c = _l.ModelConfig()
    _l.load().mk_model_config_default(C.byref(c))
    for k, v in over.items():
        assert hasattr(c, k), f"no config field {k}"
        setattr(c, k, v)
    return c


def config_dict(c):
    return {n: getattr(c, n) for n, _ in c._fields_}


class BinFile:
    """A model file opened read-only (memory-mapped).  Arrays returned by get() are views of the mapping and must
    not outlive the object."""

    def __init__(self, path):
        self._L = _l.load()
        h = C.c_void_p()
        _l.check(self._L.mk_bin_open(str(path).encode(), C.byref(h)))
        self._h = h
        self.path = str(path)
        self.config = _l.ModelConfig()
        _l.check(self._L.mk_bin_config(self._h, C.byref(self.config)))

    def __len__(self):
        return int(self._L.mk_bin_count(self._h))

    def _unpack(self, dt, nd, dims, data, size):
        shape = tuple(dims[i] for i in range(nd.value))
        raw = np.ctypeslib.as_array((C.c_uint8 * size.value).from_address(data.value))
        return dt.value, shape, raw

    def entry(self, i):
        """(name, dtype code, shape, raw uint8 view of the blob) of directory entry i."""
        name, dt, nd, dims, data, size = C.c_char_p(), C.c_int32(), C.c_int32(), (C.c_uint32 * 4)(), C.c_void_p(), C.c_uint64()
        _l.check(self._L.mk_bin_entry(self._h, i, C.byref(name), C.byref(dt), C.byref(nd), dims, C.byref(data), C.byref(size)))
        return (name.value.decode(),) + self._unpack(dt, nd, dims, data, size)

    def names(self):
        return [self.entry(i)[0] for i in range(len(self))]

    def get(self, name):
        """f32 / i32: an array of the directory's shape; mxfp4: (packed u8 [r, c/2], scales u8 [r, c/32]) as
        BinFile::mxfp4_parts (src/weights.rs:619-626) returns them; other dtypes: the raw bytes."""
        dt, nd, dims, data, size = C.c_int32(), C.c_int32(), (C.c_uint32 * 4)(), C.c_void_p(), C.c_uint64()
        _l.check(self._L.mk_bin_find(self._h, name.encode(), C.byref(dt), C.byref(nd), dims, C.byref(data), C.byref(size)))
        code, shape, raw = self._unpack(dt, nd, dims, data, size)
        if code == DTYPES["f32"]:
            return raw.view(np.float32).reshape(shape)
        if code == DTYPES["i32"]:
            return raw.view(np.int32).reshape(shape)
        if code == DTYPES["mxfp4"]:
            r, c = shape
            return raw[:r * c // 2].reshape(r, c // 2), raw[r * c // 2:].reshape(r, c // 32)
        return raw

    def close(self):
        if getattr(self, "_h", None):
            self._L.mk_bin_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class BinWriter:
    """Writes a model file: add() every tensor, begin(path), put() every blob, finish().  cfg None writes the
    MKIM0001 form (historical micro configuration), a ModelConfig the MKIM0002 form with its JSON block."""

    def __init__(self, cfg=None):
        self._L = _l.load()
        h = C.c_void_p()
        _l.check(self._L.mk_bin_writer_create(C.byref(cfg) if cfg is not None else None, C.byref(h)))
        self._h = h

    def add(self, name, dtype, shape):
        dims = (C.c_uint32 * 4)(*shape)
        _l.check(self._L.mk_bin_writer_add(self._h, name.encode(), DTYPES[dtype], len(shape), dims))

    def begin(self, path):
        _l.check(self._L.mk_bin_writer_begin(self._h, str(path).encode()))

    def put(self, name, data):
        a = np.ascontiguousarray(data)
        _l.check(self._L.mk_bin_writer_put(self._h, name.encode(), a.ctypes.data_as(C.c_void_p), a.nbytes))

    def finish(self):
        if getattr(self, "_h", None):
            self._L.mk_bin_writer_finish(self._h)
            self._h = None

    def __del__(self):
        try:
            self.finish()
        except Exception:
            pass


def quantize_mxfp4(w, search=True, ctx=None):
    """mxfp4::quantize (search=False: quantize_naive) of a torch CUDA f32 matrix [rows, cols] on the GPU ->
    (packed u8 [rows, cols/2], scales u8 [rows, cols/32]) torch CUDA tensors; bytes equal the CPU quantizer's."""
    import torch
    ctx = ctx or Context.default()
    assert _is_torch_cuda(w) and w.dtype == torch.float32 and w.is_contiguous() and w.dim() == 2 and w.shape[1] % 32 == 0
    ctx._follow_torch()
    rows, cols = w.shape
    packed = torch.empty((rows, cols // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((rows, cols // 32), dtype=torch.uint8, device=w.device)
    _l.check(ctx._L.mk_quantize_mxfp4_dev(ctx._h, C.c_void_p(w.data_ptr()), rows, cols, int(bool(search)),
                                          C.c_void_p(packed.data_ptr()), C.c_void_p(scales.data_ptr())))
    return packed, scales


class Model:
    """The K3 model resident on one GPU (or this rank's share of it): Model::load + Model::forward with the
    engine's defaults (q8_0 lm_head, q8_0 MLA cache, MXFP4 experts through the q8 integer path)."""

    def __init__(self, path, max_positions, use_graph=True, rank=0, world=1, strict=False, keep_layer_hidden=False, ctx=None):
        self.ctx = ctx or Context.default()
        self.bin = path if isinstance(path, BinFile) else BinFile(path)
        self.config = self.bin.config
        opts = _l.ModelOpts(int(max_positions), int(bool(use_graph)), int(bool(strict)), int(bool(keep_layer_hidden)), int(rank), int(world))
        h = C.c_void_p()
        _l.check(self.ctx._L.mk_model_open(self.ctx._h, self.bin._h, C.byref(opts), C.byref(h)))
        self._h = h
        self.world, self.rank = int(world), int(rank)

    # -- expert parallel / sharded lm_head over the ranks of a process group
    def connect(self, group=None):
        """world > 1: exchanges the ranks' buffer handles over the process group and opens them."""
        import torch
        import torch.distributed as dist
        mine = (C.c_uint8 * 128)()
        _l.check(self.ctx._L.mk_model_ep_handles(self.ctx._h, self._h, mine))
        dev = torch.device("cuda", self.ctx.device)
        t = torch.tensor(list(mine), dtype=torch.uint8, device=dev)
        allh = torch.empty((self.world, 128), dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allh.view(-1), t, group=group)
        buf = (C.c_uint8 * (128 * self.world)).from_buffer_copy(bytes(allh.cpu().numpy().tobytes()))
        ok = torch.ones(1, dtype=torch.int32, device=dev)
        err = None
        try:
            _l.check(self.ctx._L.mk_model_ep_connect(self.ctx._h, self._h, buf))
        except Exception as exc:
            err = exc
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)   # every rank raises, or none does
        if int(ok.item()) == 0:
            raise RuntimeError(f"peer exchange buffers could not be connected on every rank ({err})")

    def forward(self, token, want_logits=True):
        """One token (host int) -> (logits float32 [vocab] or None, greedy pick)."""
        logits = np.empty(self.config.vocab, np.float32) if want_logits else None
        nxt = C.c_int32()
        _l.check(self.ctx._L.mk_model_forward(self.ctx._h, self._h, int(token),
                                              logits.ctypes.data_as(C.c_void_p) if want_logits else None, C.byref(nxt)))
        return logits, nxt.value

    def forward_dev(self, token=None, logits=None, next_out=None):
        """One token enqueued on torch's current stream: `token` a torch CUDA int32 [1] (None = the previous pick),
        `logits` an optional torch CUDA float32 [vocab] to fill, `next_out` an optional torch CUDA int32 [1]."""
        self.ctx._follow_torch()
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
        _l.check(self.ctx._L.mk_model_forward_dev(self.ctx._h, self._h, p(token), p(logits), p(next_out)))

    def prefill(self, tokens, want_logits=True):
        """A run of prompt tokens, layer by layer (Model::prefill, src/model.rs:3043-3260): the caches end as after one
        forward() per token - bit for bit - and the logits and greedy pick of the LAST token come back."""
        tk = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty(self.config.vocab, np.float32) if want_logits else None
        nxt = C.c_int32()
        _l.check(self.ctx._L.mk_model_prefill(self.ctx._h, self._h, tk.ctypes.data_as(C.c_void_p), tk.size,
                                              logits.ctypes.data_as(C.c_void_p) if want_logits else None, C.byref(nxt)))
        return logits, nxt.value

    def generate(self, prompt, n_new):
        """The greedy loop: prompt tokens one by one, then n_new picks (the first one follows the last prompt
        token), each fed back on the device.  Returns int32 [n_new]."""
        pr = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(int(n_new), np.int32)
        _l.check(self.ctx._L.mk_model_generate(self.ctx._h, self._h, pr.ctypes.data_as(C.c_void_p), pr.size, int(n_new),
                                               out.ctypes.data_as(C.c_void_p)))
        return out

    def last_hidden(self):
        h = np.empty(self.config.d, np.float32)
        _l.check(self.ctx._L.mk_model_last_hidden(self.ctx._h, self._h, h.ctypes.data_as(C.c_void_p)))
        return h

    def layer_hidden(self):
        """Per-layer taps of the last token [n_layers, 4, d] (keep_layer_hidden=True): the attention block's output, the
        residual stream after it, the FFN's output, the residual stream after the layer."""
        h = np.empty((self.config.n_layers, 4, self.config.d), np.float32)
        _l.check(self.ctx._L.mk_model_layer_hidden(self.ctx._h, self._h, h.ctypes.data_as(C.c_void_p)))
        return h

    def reset(self):
        _l.check(self.ctx._L.mk_model_reset(self.ctx._h, self._h))

    @property
    def positions(self):
        return int(self.ctx._L.mk_model_positions(self.ctx._h, self._h))

    @property
    def weight_bytes(self):
        return int(self.ctx._L.mk_model_weight_bytes(self._h))

    @property
    def launches_per_token(self):
        return int(self.ctx._L.mk_model_launches_per_token(self._h))

    def free(self):
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._L.mk_model_free(self.ctx._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _is_mla(cfg, l):
    return l % 4 == 3 or l == cfg.n_layers - 1      # Config::is_mla (src/config.rs:127-132)


def _is_moe(cfg, l):
    return l >= cfg.first_k_dense                   # Config::is_moe (src/config.rs:133-138)


def model_tensors(cfg):
    """The tensor list of a model file in the builder's registration order (src/build.rs:350-420): (name, dtype, shape)."""
    d, proj = cfg.d, cfg.kda_heads * cfg.kda_dim
    qb, kvb = cfg.mla_heads * (cfg.mla_nope + cfg.mla_rope), cfg.mla_heads * (cfg.mla_nope + cfg.mla_v)
    cdim, hv = cfg.mla_kva + cfg.mla_rope, cfg.mla_heads * cfg.mla_v
    t = [("embed_tokens.weight", "f32", (cfg.vocab, d)), ("lm_head.weight", "f32", (cfg.vocab, d)), ("norm.weight", "f32", (d,)),
         ("output_attn_res_norm.weight", "f32", (d,)), ("output_attn_res_proj.weight", "f32", (d,))]
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        t += [(p + n, "f32", (d,)) for n in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attention_res_norm.weight",
                                             "self_attention_res_proj.weight", "mlp_res_norm.weight", "mlp_res_proj.weight")]
        a = p + "self_attn."
        if _is_mla(cfg, l):
            t += [(a + "q_a_proj.weight", "f32", (cfg.mla_qa, d)), (a + "q_a_layernorm.weight", "f32", (cfg.mla_qa,)),
                  (a + "q_b_proj.weight", "f32", (qb, cfg.mla_qa)), (a + "kv_a_proj_with_mqa.weight", "f32", (cdim, d)),
                  (a + "kv_a_layernorm.weight", "f32", (cfg.mla_kva,)), (a + "kv_b_proj.weight", "f32", (kvb, cfg.mla_kva)),
                  (a + "g_proj.weight", "f32", (hv, d)), (a + "o_proj.weight", "f32", (d, hv))]
        else:
            t += [(a + f"{n}.weight", "f32", (proj, d)) for n in ("q_proj", "k_proj", "v_proj", "g_proj")]
            t += [(a + "o_proj.weight", "f32", (d, proj))]
            t += [(a + f"{n}.weight", "f32", (proj, cfg.kda_conv)) for n in ("q_conv1d", "k_conv1d", "v_conv1d")]
            t += [(a + "f_a_proj.weight", "f32", (cfg.kda_fa, d)), (a + "f_b_proj.weight", "f32", (proj, cfg.kda_fa)),
                  (a + "A_log", "f32", (cfg.kda_dim,)), (a + "dt_bias", "f32", (proj,)), (a + "b_proj.weight", "f32", (cfg.kda_heads, d)),
                  (a + "o_norm.weight", "f32", (cfg.kda_dim,))]
        if _is_moe(cfg, l):
            q = p + "block_sparse_moe."
            t += [(q + "gate.weight", "f32", (cfg.n_experts, d)), (q + "gate.e_score_correction_bias", "f32", (cfg.n_experts,)),
                  (q + "routed_expert_down_proj.weight", "f32", (cfg.routed_hidden, d)),
                  (q + "routed_expert_up_proj.weight", "f32", (d, cfg.routed_hidden)),
                  (q + "routed_expert_norm.weight", "f32", (cfg.routed_hidden,)),
                  (q + "shared_experts.gate_proj.weight", "f32", (cfg.shared_inter, d)),
                  (q + "shared_experts.up_proj.weight", "f32", (cfg.shared_inter, d)),
                  (q + "shared_experts.down_proj.weight", "f32", (d, cfg.shared_inter))]
        else:
            t += [(p + "mlp.gate_proj.weight", "f32", (cfg.dense_inter, d)), (p + "mlp.up_proj.weight", "f32", (cfg.dense_inter, d)),
                  (p + "mlp.down_proj.weight", "f32", (d, cfg.dense_inter))]
    for l in range(cfg.n_layers):
        if _is_moe(cfg, l):
            for e in range(cfg.n_experts):
                q = f"layers.{l}.block_sparse_moe.experts.{e}."
                t += [(q + "w1", "mxfp4", (cfg.moe_inter, cfg.routed_hidden)), (q + "w2", "mxfp4", (cfg.routed_hidden, cfg.moe_inter)),
                      (q + "w3", "mxfp4", (cfg.moe_inter, cfg.routed_hidden))]
    return t


def build_synthetic_bin(path, cfg=None, seed=0, ctx=None, sigma=0.02):
    """Writes a model file of the given configuration (None: the historical micro configuration, 93 layers, MKIM0001)
    whose tensors follow the builder's Gaussian fallback branch (src/build.rs:444-571): projections, routers and
    embeddings N(0, sigma), norm weights 1, router bias 0, A_log = ln(U(1, 16)), experts N(0, sigma) through
    mxfp4::quantize.  The values are drawn with torch's CUDA generator (one stream per file, seeded by `seed`) and the
    experts are quantized by the library's GPU quantizer, so the whole file takes seconds; it is a stand-in for the
    builder's output with the same shapes and distributions, not the same bits."""
    import torch
    ctx = ctx or Context.default()
    ctx._follow_torch()
    micro = cfg is None
    cfg = cfg if cfg is not None else default_config()
    dev = torch.device("cuda", ctx.device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(int(seed))
    tensors = model_tensors(cfg)
    w = BinWriter(None if micro else cfg)
    for name, dt, shape in tensors:
        w.add(name, dt, shape)
    w.begin(path)
    ones = ("layernorm.weight", "_res_norm.weight", "norm.weight", "routed_expert_norm.weight", "o_norm.weight")
    i, n = 0, len(tensors)
    while i < n:
        name, dt, shape = tensors[i]
        if dt == "mxfp4":
            # all experts of one layer in one go: [E * 3, inter * hidden] values -> quantize per matrix shape
            j = i
            prefix = name.rsplit("experts.", 1)[0]
            while j < n and tensors[j][0].startswith(prefix):
                j += 1
            rows, cols = cfg.moe_inter, cfg.routed_hidden
            vals = torch.empty((j - i, rows * cols), dtype=torch.float32, device=dev)
            vals.normal_(0.0, sigma, generator=gen)
            blobs = {}
            for k, (r, c) in ((0, (rows, cols)), (1, (cols, rows)), (2, (rows, cols))):
                sel = vals[k::3].reshape(-1, c).contiguous()             # matrices of this kind stacked by rows
                pk, sc = quantize_mxfp4(sel, ctx=ctx)
                m = sel.shape[0] // r
                blobs[k] = (pk.reshape(m, r * c // 2).cpu().numpy(), sc.reshape(m, r * c // 32).cpu().numpy())
            for t in range(i, j):
                k, e = (t - i) % 3, (t - i) // 3
                w.put(tensors[t][0], np.concatenate([blobs[k][0][e], blobs[k][1][e]]))
            i = j
            continue
        count = int(np.prod(shape))
        if name.endswith(ones):
            a = np.ones(count, np.float32)
        elif name.endswith("e_score_correction_bias"):
            a = np.zeros(count, np.float32)
        elif name.endswith("A_log"):
            a = torch.log(1.0 + 15.0 * torch.rand(count, device=dev, generator=gen)).cpu().numpy()
        else:
            t = torch.empty(count, dtype=torch.float32, device=dev)
            t.normal_(0.0, sigma, generator=gen)
            a = t.cpu().numpy()
        w.put(name, a.astype(np.float32))
        i += 1
    w.finish()
    return path
