"""ctypes loader for the CPU oracle (libmk_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark.  The product package never imports it.
Each wrapper takes and returns numpy arrays; the C function it calls cites the
reference source lines it restates (see mk_oracle.h / mk_oracle.c).
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmk_oracle.so")


def build(force=False):
    deps = [os.path.join(_HERE, f) for f in ("mk_oracle.c", "mk_oracle_model.c", "mk_oracle.h", "Makefile")]
    if (not force and os.path.exists(_SO)
            and os.path.getmtime(_SO) >= max(os.path.getmtime(p) for p in deps)):
        return _SO
    subprocess.check_call(["make", "-C", _HERE, "-B", "libmk_oracle.so"], stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()          # no-op unless the sources are newer than the library
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_u16p = C.POINTER(C.c_uint16)
_i32p = C.POINTER(C.c_int32)
_sz = C.c_size_t


class _MoeDesc(C.Structure):
    _fields_ = [("d", _sz), ("inter", _sz), ("n_experts", _sz), ("top_k", _sz),
                ("limit", C.c_float), ("use_q8", C.c_int),
                ("gate_w", _f32p), ("gate_b", _f32p),
                ("packed", C.POINTER(_u8p)), ("scales", C.POINTER(_u8p)),
                ("sh_packed", _u8p * 3), ("sh_scales", _u8p * 3)]


class _KdaDesc(C.Structure):
    _fields_ = [("heads", _sz), ("dim", _sz), ("kconv", _sz), ("gate_lb", C.c_float), ("rms_eps", C.c_float),
                ("q_conv", _f32p), ("k_conv", _f32p), ("v_conv", _f32p), ("a_log", _f32p), ("dt_bias", _f32p), ("o_norm", _f32p)]


class _MoeK3Desc(C.Structure):
    _fields_ = [("d", _sz), ("rh", _sz), ("inter", _sz), ("n_experts", _sz), ("top_k", _sz), ("shared_inter", _sz),
                ("rms_eps", C.c_float), ("use_q8", C.c_int),
                ("gate_w", _f32p), ("gate_b", _f32p), ("routed_down", _f32p), ("routed_norm", _f32p), ("routed_up", _f32p),
                ("shared_gate", _f32p), ("shared_up", _f32p), ("shared_down", _f32p),
                ("packed", C.POINTER(_u8p)), ("scales", C.POINTER(_u8p))]


def _declare(L):
    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)
    sig("or_num_threads", C.c_int)
    sig("or_rng_fill_gauss", None, C.c_char_p, C.c_float, _f32p, _sz)
    sig("or_exp2_i", C.c_float, C.c_int)
    sig("or_scale_from_byte", C.c_float, C.c_uint8)
    sig("or_mxfp4_dequant", None, _u8p, _u8p, _sz, _sz, _f32p)
    sig("or_mxfp4_quantize", None, _f32p, _sz, _sz, C.c_int, _u8p, _u8p)
    sig("or_mxfp4_matvec_f32", None, _u8p, _u8p, _sz, _sz, _f32p, _f32p, C.c_int)
    sig("or_mxfp4_matvec_q8", None, _u8p, _u8p, _sz, _sz, _i8p, _f32p, _f32p, C.c_int)
    sig("or_mxfp4_matvec", None, _u8p, _u8p, _sz, _sz, _f32p, _f32p, C.c_int, C.c_int)
    sig("or_mxfp4_matvec_shader_emul", None, _u8p, _u8p, _sz, _sz, _f32p, _f32p, _sz)
    sig("or_mxfp4_matvec_nt", None, _u8p, _u8p, _sz, _sz, _f32p, _sz, _f32p)
    sig("or_q8_quantize", None, _f32p, _sz, _i8p, _f32p)
    sig("or_block_dot", C.c_int32, _u8p, _i8p)
    sig("or_block_dot_i8", C.c_int32, _i8p, _i8p)
    sig("or_dot", C.c_float, _f32p, _f32p, _sz)
    sig("or_matvec_f32", None, _f32p, _sz, _sz, _f32p, _f32p, C.c_int)
    sig("or_rmsnorm", None, _f32p, _f32p, _sz, C.c_float, _f32p)
    sig("or_sigmoid", C.c_float, C.c_float)
    sig("or_situ", C.c_float, C.c_float, C.c_float)
    sig("or_argmax", C.c_int, _f32p, _sz)
    sig("or_q8head_from_f32", None, _f32p, _sz, _sz, _i8p, _f32p)
    sig("or_q8head_matvec", None, _i8p, _f32p, _sz, _sz, _f32p, _f32p, C.c_int)
    sig("or_q8head_from_f32_f16s", None, _f32p, _sz, _sz, _i8p, _u16p)
    sig("or_q8head_matvec_f16s", None, _i8p, _u16p, _sz, _sz, _f32p, _f32p, C.c_int)
    sig("or_router_k3", None, _f32p, _f32p, _sz, _sz, _sz, _f32p, _i32p, _f32p, _f32p)
    sig("or_gate_ds", None, _f32p, _f32p, _sz, _sz, _sz, C.c_float, _f32p, _i32p, _f32p)
    sig("or_expert_ds_f32", None, _f32p, _f32p, _f32p, _f32p, _sz, _sz, C.c_float, _f32p)
    sig("or_moe_ds_forward", None, C.POINTER(_MoeDesc), _f32p, _f32p, _i32p, _f32p, C.c_int)
    sig("or_dequant_fp8", None, _u8p, _u8p, _sz, _sz, _f32p)
    sig("or_matvec_vq_gather", None, _f32p, _u8p, _sz, _sz, _f32p, _f32p)
    sig("or_matvec_vq_lut", None, _f32p, _u8p, _sz, _sz, _f32p, _f32p)
    sig("or_moe_k3_forward", None, C.POINTER(_MoeK3Desc), _f32p, _f32p, _i32p, _f32p)
    sig("or_kda_step", None, C.POINTER(_KdaDesc), _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p)
    sig("or_kda_core", None, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _sz, _sz, _sz, _f32p, _f32p)
    sig("or_kda_recur_step", None, _sz, _sz, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p)
    sig("or_kda_norm_head", None, _sz, _sz, _f32p, C.c_float)
    sig("or_kda_gate", None, _sz, _sz, C.c_float, _f32p, _f32p, _f32p, _f32p)
    sig("or_attn_res", None, _sz, C.c_float, _f32p, _f32p, _sz, _f32p, _f32p)
    sig("or_mla_new", C.c_void_p, _sz, _sz, _sz, _sz, _sz)
    sig("or_mla_free", None, C.c_void_p)
    sig("or_mla_push", None, C.c_void_p, _f32p, _f32p)
    sig("or_mla_to_f32", None, C.c_void_p, _f32p, _f32p)
    sig("or_mla_attn_flash_q8", None, C.c_void_p, _f32p, _sz, _sz, C.c_float, _f32p)
    sig("or_mla_attn_flash_q8_mqa", None, C.c_void_p, _f32p, _sz, C.c_float, _f32p)
    sig("or_mla_attn_ref_q8", None, C.c_void_p, _f32p, _sz, _sz, C.c_float, _f32p)
    sig("or_mla_attn_ref_f32", None, _f32p, _f32p, _sz, _sz, _sz, _f32p, _sz, _sz, C.c_float, _f32p)
    sig("or_mla_attn_flash_f32", None, _f32p, _f32p, _sz, _sz, _sz, _f32p, _sz, _sz, C.c_float, _f32p)
    sig("or_mla_abs_new", C.c_void_p, _sz, _sz, _sz)
    sig("or_mla_abs_free", None, C.c_void_p)
    sig("or_mla_abs_push", None, C.c_void_p, _f32p)
    sig("or_mla_abs_attn", None, C.c_void_p, _f32p, _sz, _sz, C.c_float, _f32p)
    sig("or_mla_abs_attn_f64", None, C.c_void_p, _f32p, _sz, _sz, C.c_float, _f64p)
    sig("or_set_num_threads", None, C.c_int)
    sig("or_set_cr_math", None, C.c_int)
    sig("or_mxfp4sq_quantize", C.c_float, _f32p, _sz, _sz, _u8p, _u8p)
    sig("or_mxfp4sq_dequant", None, _u8p, _u8p, C.c_float, _sz, _sz, _f32p)
    sig("or_config_microkimi", None, C.c_void_p)
    sig("or_config_is_mla", C.c_int, C.c_void_p, C.c_uint32)
    sig("or_config_is_moe", C.c_int, C.c_void_p, C.c_uint32)
    sig("or_build_bin", C.c_int, C.c_char_p, C.c_void_p)
    sig("or_bin_open", C.c_void_p, C.c_char_p)
    sig("or_bin_close", None, C.c_void_p)
    sig("or_bin_config", C.c_void_p, C.c_void_p)
    sig("or_bin_count", C.c_size_t, C.c_void_p)
    sig("or_bin_get", C.c_void_p, C.c_void_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p)
    sig("or_bin_entry", C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p)
    sig("or_model_open", C.c_void_p, C.c_char_p, C.c_size_t, C.c_int)
    sig("or_model_free", None, C.c_void_p)
    sig("or_model_reset", None, C.c_void_p)
    sig("or_model_config", C.c_void_p, C.c_void_p)
    sig("or_model_forward", C.c_int, C.c_void_p, C.c_uint32, _f32p, _f32p)
    sig("or_model_forward_layers", C.c_int, C.c_void_p, C.c_uint32, _f32p, _f32p, _f32p)
    sig("or_f32_to_f16", C.c_uint16, C.c_float)
    sig("or_f16_to_f32", C.c_float, C.c_uint16)


class Config(C.Structure):
    """or_config: the engine's Config (src/config.rs:8-43), micro defaults from Config::microkimi."""
    _fields_ = ([(n, C.c_uint32) for n in ("n_layers", "d", "vocab", "n_experts", "top_k", "n_shared", "kda_heads", "kda_dim",
                                          "kda_conv", "kda_fa")] + [("gate_lb", C.c_float)] +
                [(n, C.c_uint32) for n in ("mla_heads", "mla_qa", "mla_kva", "mla_nope", "mla_rope", "mla_v", "routed_hidden",
                                          "moe_inter", "shared_inter", "dense_inter", "attn_res_block", "first_k_dense")] +
                [("rms_eps", C.c_float), ("eos_id", C.c_uint32), ("bos_id", C.c_uint32)])

    @classmethod
    def microkimi(cls, **over):
        c = cls()
        lib().or_config_microkimi(C.byref(c))
        for k, v in over.items():
            assert hasattr(c, k), k
            setattr(c, k, v)
        return c

    def is_mla(self, l):
        return bool(lib().or_config_is_mla(C.byref(self), l))

    def is_moe(self, l):
        return bool(lib().or_config_is_moe(C.byref(self), l))

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


def build_bin(path, cfg):
    """`microkimi build` on the Gaussian fallback branch of every tensor (src/build.rs:344-576): writes the model file."""
    rc = lib().or_build_bin(str(path).encode(), C.byref(cfg))
    if rc != 0:
        raise OSError(f"or_build_bin({path}) failed: {rc}")


class BinFile:
    """The MKIM0001/2 container (src/weights.rs:421-468), read-only."""

    def __init__(self, path):
        self._h = lib().or_bin_open(str(path).encode())
        if not self._h:
            raise OSError(f"cannot open {path}")
        self.config = Config.from_buffer_copy(C.string_at(lib().or_bin_config(self._h), C.sizeof(Config)))

    def __len__(self):
        return int(lib().or_bin_count(self._h))

    def entry(self, i):
        name, dt, dims, off, size = C.c_char_p(), C.c_uint8(), (C.c_uint32 * 2)(), C.c_uint64(), C.c_uint64()
        if lib().or_bin_entry(self._h, i, C.byref(name), C.byref(dt), dims, C.byref(off), C.byref(size)) != 0:
            raise IndexError(i)
        return name.value.decode(), dt.value, (dims[0], dims[1]), off.value, size.value

    def get(self, name):
        """f32 tensors: float32 array of the directory's shape; mxfp4: (packed [r, c/2], scales [r, c/32]) uint8 arrays."""
        dt, dims, size = C.c_uint8(), (C.c_uint32 * 2)(), C.c_uint64()
        p = lib().or_bin_get(self._h, name.encode(), C.byref(dt), dims, C.byref(size))
        if not p:
            raise KeyError(name)
        raw = np.frombuffer(C.string_at(p, size.value), dtype=np.uint8)
        r, c = dims[0], dims[1]
        if dt.value == 0:
            a = raw.view(np.float32)
            return a.reshape(r, c) if c else a
        return raw[:r * c // 2].reshape(r, c // 2), raw[r * c // 2:].reshape(r, c // 32)

    def close(self):
        if getattr(self, "_h", None):
            lib().or_bin_close(self._h)
            self._h = None

    def __del__(self):
        self.close()


class Model:
    """Model::from_bin + Model::forward (src/model.rs:906-1025, 2889-3031): q8_0 lm_head, q8_0 MLA cache, MXFP4 experts
    through the q8 integer path - the engine's defaults."""

    def __init__(self, path, max_positions, n_threads=1):
        self._h = lib().or_model_open(str(path).encode(), int(max_positions), int(n_threads))
        if not self._h:
            raise OSError(f"cannot load {path}")
        self.config = Config.from_buffer_copy(C.string_at(lib().or_model_config(self._h), C.sizeof(Config)))

    def forward(self, token, want_hidden=False):
        """One token -> logits [vocab] (and the final normed hidden state [d])."""
        logits = np.empty(self.config.vocab, np.float32)
        hid = np.empty(self.config.d, np.float32)
        rc = lib().or_model_forward(self._h, int(token), _p(logits, _f32p), _p(hid, _f32p))
        if rc != 0:
            raise ValueError(f"or_model_forward failed: {rc}")
        return (logits, hid) if want_hidden else logits

    def forward_layers(self, token):
        """One token -> (logits, final normed hidden state, taps [n_layers, 4, d]: per layer the attention block's output,
        the residual stream after it, the FFN's output, the residual stream after the layer)."""
        logits = np.empty(self.config.vocab, np.float32)
        hid = np.empty(self.config.d, np.float32)
        layers = np.empty((self.config.n_layers, 4, self.config.d), np.float32)
        rc = lib().or_model_forward_layers(self._h, int(token), _p(logits, _f32p), _p(hid, _f32p), _p(layers, _f32p))
        if rc != 0:
            raise ValueError(f"or_model_forward failed: {rc}")
        return logits, hid, layers

    def reset(self):
        lib().or_model_reset(self._h)

    def close(self):
        if getattr(self, "_h", None):
            lib().or_model_free(self._h)
            self._h = None

    def __del__(self):
        self.close()


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads():
    return int(lib().or_num_threads())


def host_threads():
    """The cores this process may run on.  Unlike num_threads() this does not follow OMP_NUM_THREADS,
    which launchers such as torchrun set to 1 for their children."""
    import os
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def set_num_threads(n):
    lib().or_set_num_threads(int(n))


def set_cr_math(on):
    """True: the oracle takes exp / tanh / log in double precision and rounds once (correctly rounded in practice, and
    what the CUDA kernels compute) instead of calling the f32 libm functions, whose last bit is the platform's."""
    lib().or_set_cr_math(int(bool(on)))


# ---------------------------------------------------------------- RNG
def fill_gauss(name, sigma, n):
    out = np.empty(n, np.float32)
    lib().or_rng_fill_gauss(name.encode(), float(sigma), _p(out, _f32p), n)
    return out


# ---------------------------------------------------------------- MXFP4
def mxfp4_dequant(packed, scales, rows, cols):
    packed, scales = _c(packed, np.uint8), _c(scales, np.uint8)
    out = np.empty((rows, cols), np.float32)
    lib().or_mxfp4_dequant(_p(packed, _u8p), _p(scales, _u8p), rows, cols, _p(out, _f32p))
    return out


def mxfp4_quantize(w, search=True):
    w = _c(w, np.float32)
    rows, cols = w.shape
    packed = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 32), np.uint8)
    lib().or_mxfp4_quantize(_p(w, _f32p), rows, cols, int(search), _p(packed, _u8p), _p(scales, _u8p))
    return packed, scales


def mxfp4sq_quantize(w):
    """mxfp4::quantize_sq: (packed, scales, smax)."""
    w = _c(w, np.float32)
    rows, cols = w.shape
    packed = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 32), np.uint8)
    smax = lib().or_mxfp4sq_quantize(_p(w, _f32p), rows, cols, _p(packed, _u8p), _p(scales, _u8p))
    return packed, scales, np.float32(smax)


def mxfp4sq_dequant(packed, scales, smax, rows, cols):
    packed, scales = _c(packed, np.uint8), _c(scales, np.uint8)
    out = np.empty((rows, cols), np.float32)
    lib().or_mxfp4sq_dequant(_p(packed, _u8p), _p(scales, _u8p), float(smax), rows, cols, _p(out, _f32p))
    return out


def mxfp4_matvec(packed, scales, x, use_q8, n_threads=1):
    packed, scales, x = _c(packed, np.uint8), _c(scales, np.uint8), _c(x, np.float32)
    rows, cols = packed.shape[0], packed.shape[1] * 2
    out = np.empty(rows, np.float32)
    lib().or_mxfp4_matvec(_p(packed, _u8p), _p(scales, _u8p), rows, cols, _p(x, _f32p), _p(out, _f32p),
                          n_threads, int(use_q8))
    return out


def mxfp4_matvec_shader_emul(packed, scales, x, lanes=256):
    packed, scales, x = _c(packed, np.uint8), _c(scales, np.uint8), _c(x, np.float32)
    rows, cols = packed.shape[0], packed.shape[1] * 2
    out = np.empty(rows, np.float32)
    lib().or_mxfp4_matvec_shader_emul(_p(packed, _u8p), _p(scales, _u8p), rows, cols, _p(x, _f32p),
                                      _p(out, _f32p), lanes)
    return out


def mxfp4_matvec_nt(packed, scales, xs):
    """xs: [m, cols] (m % 8 == 0). Returns [m, rows] in the batched order of model.rs:2412."""
    packed, scales = _c(packed, np.uint8), _c(scales, np.uint8)
    xs = _c(xs, np.float32)
    m, cols = xs.shape
    rows = packed.shape[0]
    xt = np.ascontiguousarray(xs.T)
    out = np.empty((m, rows), np.float32)
    lib().or_mxfp4_matvec_nt(_p(packed, _u8p), _p(scales, _u8p), rows, cols, _p(xt, _f32p), m, _p(out, _f32p))
    return out


# ---------------------------------------------------------------- q8_0
def q8_quantize(x):
    x = _c(x, np.float32).ravel()
    q = np.empty(x.size, np.int8)
    s = np.empty(x.size // 32, np.float32)
    lib().or_q8_quantize(_p(x, _f32p), x.size, _p(q, _i8p), _p(s, _f32p))
    return q, s


def block_dot(packed16, x32):
    return int(lib().or_block_dot(_p(_c(packed16, np.uint8), _u8p), _p(_c(x32, np.int8), _i8p)))


def block_dot_i8(w32, x32):
    return int(lib().or_block_dot_i8(_p(_c(w32, np.int8), _i8p), _p(_c(x32, np.int8), _i8p)))


def dot(a, b):
    a, b = _c(a, np.float32), _c(b, np.float32)
    return float(np.float32(lib().or_dot(_p(a, _f32p), _p(b, _f32p), a.size)))


def matvec_f32(w, x, n_threads=1):
    w, x = _c(w, np.float32), _c(x, np.float32)
    out = np.empty(w.shape[0], np.float32)
    lib().or_matvec_f32(_p(w, _f32p), w.shape[0], w.shape[1], _p(x, _f32p), _p(out, _f32p), n_threads)
    return out


def dequant_fp8(w, scales, rows, cols):
    """dequant::dequant_fp8 (dequant.rs:27-41): e4m3fn bytes [rows, cols] + ue8m0 scale per 128 x 128 block."""
    w, scales = _c(w, np.uint8), _c(scales, np.uint8)
    out = np.empty((rows, cols), np.float32)
    lib().or_dequant_fp8(_p(w, _u8p), _p(scales, _u8p), rows, cols, _p(out, _f32p))
    return out


def matvec_vq(codebook, indices, x, lut=True):
    """VQ1 matvec (quant.rs:340-346): codebook f32 [256, 16], indices u8 [rows, cols/16]."""
    cb, idx, x = _c(codebook, np.float32), _c(indices, np.uint8), _c(x, np.float32)
    rows, vpr = idx.shape
    out = np.empty(rows, np.float32)
    fn = lib().or_matvec_vq_lut if lut else lib().or_matvec_vq_gather
    fn(_p(cb, _f32p), _p(idx, _u8p), rows, vpr * 16, _p(x, _f32p), _p(out, _f32p))
    return out


def rmsnorm(x, w, eps):
    x, w = _c(x, np.float32), _c(w, np.float32)
    out = np.empty_like(x)
    lib().or_rmsnorm(_p(x, _f32p), _p(w, _f32p), x.size, float(eps), _p(out, _f32p))
    return out


def argmax(v):
    v = _c(v, np.float32)
    return int(lib().or_argmax(_p(v, _f32p), v.size))


def q8head_from_f32(w):
    w = _c(w, np.float32)
    rows, cols = w.shape
    q = np.empty((rows, cols), np.int8)
    s = np.empty((rows, cols // 32), np.float32)
    lib().or_q8head_from_f32(_p(w, _f32p), rows, cols, _p(q, _i8p), _p(s, _f32p))
    return q, s


def q8head_matvec(q, s, x, n_threads=1):
    q, s, x = _c(q, np.int8), _c(s, np.float32), _c(x, np.float32)
    out = np.empty(q.shape[0], np.float32)
    lib().or_q8head_matvec(_p(q, _i8p), _p(s, _f32p), q.shape[0], q.shape[1], _p(x, _f32p), _p(out, _f32p), n_threads)
    return out


def q8head_from_f32_f16s(w):
    w = _c(w, np.float32)
    rows, cols = w.shape
    q = np.empty((rows, cols), np.int8)
    s = np.empty((rows, cols // 32), np.uint16)
    lib().or_q8head_from_f32_f16s(_p(w, _f32p), rows, cols, _p(q, _i8p), _p(s, _u16p))
    return q, s


def q8head_matvec_f16s(q, s, x, n_threads=1):
    q, s, x = _c(q, np.int8), _c(s, np.uint16), _c(x, np.float32)
    out = np.empty(q.shape[0], np.float32)
    lib().or_q8head_matvec_f16s(_p(q, _i8p), _p(s, _u16p), q.shape[0], q.shape[1], _p(x, _f32p), _p(out, _f32p),
                                n_threads)
    return out


# ---------------------------------------------------------------- routers / experts
def router_k3(gate_w, gate_b, x, top_k):
    gate_w, gate_b, x = _c(gate_w, np.float32), _c(gate_b, np.float32), _c(x, np.float32)
    n, d = gate_w.shape
    ids = np.empty(top_k, np.int32)
    w = np.empty(top_k, np.float32)
    logits = np.empty(n, np.float32)
    lib().or_router_k3(_p(gate_w, _f32p), _p(gate_b, _f32p), n, d, top_k, _p(x, _f32p), _p(ids, _i32p),
                       _p(w, _f32p), _p(logits, _f32p))
    return ids, w, logits


def gate_ds(gate_w, bias, x, top_k, route_scale):
    gate_w, x = _c(gate_w, np.float32), _c(x, np.float32)
    n, d = gate_w.shape
    ids = np.empty(top_k, np.int32)
    w = np.empty(top_k, np.float32)
    bp = _p(_c(bias, np.float32), _f32p) if bias is not None else None
    lib().or_gate_ds(_p(gate_w, _f32p), bp, n, d, top_k, float(route_scale), _p(x, _f32p), _p(ids, _i32p), _p(w, _f32p))
    return ids, w


def expert_ds_f32(w1, w2, w3, x, limit):
    w1, w2, w3, x = (_c(a, np.float32) for a in (w1, w2, w3, x))
    inter, d = w1.shape
    out = np.empty(d, np.float32)
    lib().or_expert_ds_f32(_p(w1, _f32p), _p(w2, _f32p), _p(w3, _f32p), _p(x, _f32p), d, inter, float(limit),
                           _p(out, _f32p))
    return out


class MoeDs:
    """K3 router + DeepSeek expert body over MXFP4 experts (one token at a time).

    experts: list of (w1, w2, w3) with each = (packed, scales) uint8 arrays;
    shared: one such triple.
    """

    def __init__(self, gate_w, gate_b, experts, shared, top_k, limit=10.0):
        self.gate_w = _c(gate_w, np.float32)
        self.gate_b = _c(gate_b, np.float32)
        self.n_experts, self.d = self.gate_w.shape
        self.top_k = top_k
        self.limit = float(limit)
        self._keep = []
        n = self.n_experts
        self._pp = (_u8p * (3 * n))()
        self._sp = (_u8p * (3 * n))()
        for e, tri in enumerate(experts):
            for j, (p, s) in enumerate(tri):
                p, s = _c(p, np.uint8), _c(s, np.uint8)
                self._keep += [p, s]
                self._pp[3 * e + j] = _p(p, _u8p)
                self._sp[3 * e + j] = _p(s, _u8p)
        self.inter = experts[0][0][0].shape[0]
        self._sh = []
        for (p, s) in shared:
            p, s = _c(p, np.uint8), _c(s, np.uint8)
            self._sh.append((p, s))

    def forward(self, x, use_q8=True, n_threads=1):
        x = _c(x, np.float32)
        d = _MoeDesc()
        d.d, d.inter, d.n_experts, d.top_k = self.d, self.inter, self.n_experts, self.top_k
        d.limit, d.use_q8 = self.limit, int(use_q8)
        d.gate_w, d.gate_b = _p(self.gate_w, _f32p), _p(self.gate_b, _f32p)
        d.packed = C.cast(self._pp, C.POINTER(_u8p))
        d.scales = C.cast(self._sp, C.POINTER(_u8p))
        for j in range(3):
            d.sh_packed[j] = _p(self._sh[j][0], _u8p)
            d.sh_scales[j] = _p(self._sh[j][1], _u8p)
        out = np.empty(self.d, np.float32)
        ids = np.empty(self.top_k, np.int32)
        w = np.empty(self.top_k, np.float32)
        lib().or_moe_ds_forward(C.byref(d), _p(x, _f32p), _p(out, _f32p), _p(ids, _i32p), _p(w, _f32p), n_threads)
        return out, ids, w


class KdaLayer:
    """The KDA decode step between the projections and o_proj (model.rs:1203-1228): holds the conv windows
    (kconv - 1 previous raw inputs of q, k, v) and the recurrent state S [heads, dim, dim]."""

    def __init__(self, heads, dim, q_conv, k_conv, v_conv, a_log, dt_bias, o_norm, kconv=4, gate_lb=-5.0, rms_eps=1e-6):
        self.heads, self.dim, self.kconv, self.gate_lb, self.rms_eps = heads, dim, kconv, float(gate_lb), float(rms_eps)
        self.w = [_c(a, np.float32) for a in (q_conv, k_conv, v_conv, a_log, dt_bias, o_norm)]
        proj = heads * dim
        self.conv = [np.zeros((kconv - 1, proj), np.float32) for _ in range(3)]
        self.s = np.zeros((heads, dim, dim), np.float32)

    def step(self, q_raw, k_raw, v_raw, g_low, beta_raw, g2):
        d = _KdaDesc()
        d.heads, d.dim, d.kconv, d.gate_lb, d.rms_eps = self.heads, self.dim, self.kconv, self.gate_lb, self.rms_eps
        d.q_conv, d.k_conv, d.v_conv, d.a_log, d.dt_bias, d.o_norm = (_p(a, _f32p) for a in self.w)
        ins = [_c(a, np.float32) for a in (q_raw, k_raw, v_raw, g_low, beta_raw, g2)]
        o = np.empty(self.heads * self.dim, np.float32)
        lib().or_kda_step(C.byref(d), *(_p(c, _f32p) for c in self.conv), _p(self.s, _f32p), *(_p(a, _f32p) for a in ins),
                          _p(o, _f32p))
        return o


def kda_core(q, k, v, g, beta, a_log, dt_bias, t_steps, heads, dim):
    """The selftest's standalone recurrence (selftest.rs:48-113): (o [T*H*dim], S [H*dim*dim])."""
    a = [_c(x, np.float32) for x in (q, k, v, g, beta, a_log, dt_bias)]
    o = np.empty(t_steps * heads * dim, np.float32)
    s = np.empty(heads * dim * dim, np.float32)
    lib().or_kda_core(*(_p(x, _f32p) for x in a), t_steps, heads, dim, _p(o, _f32p), _p(s, _f32p))
    return o, s


def kda_model_recurrence(q, k, v, g, beta, a_log, dt_bias, t_steps, heads, dim, gate_lb=-5.0):
    """The same raw inputs through the engine's own pieces: kda_norm_head, kda_gate, sigmoid(beta) and
    kda_recur_step (model.rs:1088-1156)."""
    L = lib()
    proj = heads * dim
    s = np.zeros(heads * dim * dim, np.float32)
    o = np.empty((t_steps, proj), np.float32)
    a_log, dt_bias = _c(a_log, np.float32), _c(dt_bias, np.float32)
    for t in range(t_steps):
        qt = _c(np.asarray(q, np.float32).reshape(t_steps, proj)[t].copy(), np.float32)
        kt = _c(np.asarray(k, np.float32).reshape(t_steps, proj)[t].copy(), np.float32)
        vt = _c(np.asarray(v, np.float32).reshape(t_steps, proj)[t], np.float32)
        gl = _c(np.asarray(g, np.float32).reshape(t_steps, proj)[t], np.float32)
        bt = np.array([L.or_sigmoid(float(b)) for b in np.asarray(beta, np.float32).reshape(t_steps, heads)[t]], np.float32)
        L.or_kda_norm_head(heads, dim, _p(qt, _f32p), float(np.float32(dim) ** np.float32(-0.5)))
        L.or_kda_norm_head(heads, dim, _p(kt, _f32p), 1.0)
        gg = np.empty(proj, np.float32)
        L.or_kda_gate(heads, dim, float(gate_lb), _p(a_log, _f32p), _p(dt_bias, _f32p), _p(gl, _f32p), _p(gg, _f32p))
        L.or_kda_recur_step(heads, dim, _p(s, _f32p), _p(qt, _f32p), _p(kt, _f32p), _p(vt, _f32p), _p(gg, _f32p), _p(bt, _f32p),
                            _p(o[t], _f32p))
    return o.reshape(-1), s


def attn_res(prefix, blocks, w, eps):
    prefix, blocks, w = _c(prefix, np.float32), _c(blocks, np.float32), _c(w, np.float32)
    out = np.empty_like(prefix)
    lib().or_attn_res(prefix.size, float(eps), _p(prefix, _f32p), _p(blocks, _f32p), blocks.shape[0], _p(w, _f32p), _p(out, _f32p))
    return out


class MoeK3:
    """K3 latent MoE layer (model.rs:2150-2380), one token at a time.

    experts: list of (w1, w2, w3), each = (packed, scales) uint8 arrays over the latent width;
    shared: (gate [si, d], up [si, d], down [d, si]) f32 arrays or None.
    """

    def __init__(self, gate_w, gate_b, routed_down, routed_norm, routed_up, experts, shared, top_k, rms_eps=1e-6):
        self.gate_w, self.gate_b = _c(gate_w, np.float32), _c(gate_b, np.float32)
        self.routed_down, self.routed_norm, self.routed_up = (_c(routed_down, np.float32), _c(routed_norm, np.float32),
                                                            _c(routed_up, np.float32))
        self.n_experts, self.d = self.gate_w.shape
        self.rh = self.routed_down.shape[0]
        self.top_k, self.rms_eps = top_k, float(rms_eps)
        self.shared = None if shared is None else tuple(_c(a, np.float32) for a in shared)
        self._keep = []
        n = self.n_experts
        self._pp = (_u8p * (3 * n))()
        self._sp = (_u8p * (3 * n))()
        for e, tri in enumerate(experts):
            for j, (p, s) in enumerate(tri):
                p, s = _c(p, np.uint8), _c(s, np.uint8)
                self._keep += [p, s]
                self._pp[3 * e + j] = _p(p, _u8p)
                self._sp[3 * e + j] = _p(s, _u8p)
        self.inter = experts[0][0][0].shape[0]

    def forward(self, x, use_q8=True):
        x = _c(x, np.float32)
        d = _MoeK3Desc()
        d.d, d.rh, d.inter, d.n_experts, d.top_k = self.d, self.rh, self.inter, self.n_experts, self.top_k
        d.rms_eps, d.use_q8 = self.rms_eps, int(use_q8)
        d.gate_w, d.gate_b = _p(self.gate_w, _f32p), _p(self.gate_b, _f32p)
        d.routed_down, d.routed_norm, d.routed_up = (_p(self.routed_down, _f32p), _p(self.routed_norm, _f32p),
                                                     _p(self.routed_up, _f32p))
        if self.shared is not None:
            d.shared_inter = self.shared[0].shape[0]
            d.shared_gate, d.shared_up, d.shared_down = (_p(a, _f32p) for a in self.shared)
        d.packed = C.cast(self._pp, C.POINTER(_u8p))
        d.scales = C.cast(self._sp, C.POINTER(_u8p))
        out = np.empty(self.d, np.float32)
        ids = np.empty(self.top_k, np.int32)
        w = np.empty(self.top_k, np.float32)
        lib().or_moe_k3_forward(C.byref(d), _p(x, _f32p), _p(out, _f32p), _p(ids, _i32p), _p(w, _f32p))
        return out, ids, w


# ---------------------------------------------------------------- MLA
class MlaCache:
    """q8_0 MLA cache in the reference's per-head layout (model.rs:765-781)."""

    def __init__(self, nh, nope, rope, vd, cap):
        self.nh, self.nope, self.rope, self.vd, self.cap = nh, nope, rope, vd, cap
        self.n = 0
        self._h = lib().or_mla_new(nh, nope, rope, vd, cap)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().or_mla_free(self._h)
            self._h = None

    def push(self, k_row, v_row):
        k_row, v_row = _c(k_row, np.float32), _c(v_row, np.float32)
        assert self.n < self.cap
        lib().or_mla_push(self._h, _p(k_row, _f32p), _p(v_row, _f32p))
        self.n += 1

    def to_f32(self):
        k = np.empty((self.n, self.nh, self.nope + self.rope), np.float32)
        v = np.empty((self.n, self.nh, self.vd), np.float32)
        lib().or_mla_to_f32(self._h, _p(k, _f32p), _p(v, _f32p))
        return k, v

    def attn_mqa(self, q, pos, scale):
        q = _c(q, np.float32)
        out = np.empty((self.nh, self.vd), np.float32)
        lib().or_mla_attn_flash_q8_mqa(self._h, _p(q, _f32p), pos, float(scale), _p(out, _f32p))
        return out

    def attn_head(self, qh, h, pos, scale):
        qh = _c(qh, np.float32)
        out = np.empty(self.vd, np.float32)
        lib().or_mla_attn_flash_q8(self._h, _p(qh, _f32p), h, pos, float(scale), _p(out, _f32p))
        return out

    def attn_ref_head(self, qh, h, pos, scale):
        qh = _c(qh, np.float32)
        out = np.zeros(self.vd, np.float32)
        lib().or_mla_attn_ref_q8(self._h, _p(qh, _f32p), h, pos, float(scale), _p(out, _f32p))
        return out


def mla_attn_ref_f32(k, v, qh, h, pos, scale):
    k, v, qh = _c(k, np.float32), _c(v, np.float32), _c(qh, np.float32)
    _, nh, hd = k.shape
    vd = v.shape[2]
    out = np.empty(vd, np.float32)
    lib().or_mla_attn_ref_f32(_p(k, _f32p), _p(v, _f32p), nh, hd, vd, _p(qh, _f32p), h, pos, float(scale), _p(out, _f32p))
    return out


def mla_attn_flash_f32(k, v, qh, h, pos, scale):
    k, v, qh = _c(k, np.float32), _c(v, np.float32), _c(qh, np.float32)
    _, nh, hd = k.shape
    vd = v.shape[2]
    out = np.empty(vd, np.float32)
    lib().or_mla_attn_flash_f32(_p(k, _f32p), _p(v, _f32p), nh, hd, vd, _p(qh, _f32p), h, pos, float(scale), _p(out, _f32p))
    return out


class MlaAbsCache:
    """q8_0 cache of one shared latent row per position (absorbed form)."""

    def __init__(self, lat, vd, cap):
        self.lat, self.vd, self.cap, self.n = lat, vd, cap, 0
        self._h = lib().or_mla_abs_new(lat, vd, cap)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().or_mla_abs_free(self._h)
            self._h = None

    def push(self, row):
        row = _c(row, np.float32)
        assert self.n < self.cap
        lib().or_mla_abs_push(self._h, _p(row, _f32p))
        self.n += 1

    def push_many(self, rows):
        for r in _c(rows, np.float32):
            self.push(r)

    def attn(self, q, pos, scale):
        q = _c(q, np.float32)
        nh = q.shape[0]
        out = np.empty((nh, self.vd), np.float32)
        lib().or_mla_abs_attn(self._h, _p(q, _f32p), nh, pos, float(scale), _p(out, _f32p))
        return out

    def attn_f64(self, q, pos, scale):
        q = _c(q, np.float32)
        nh = q.shape[0]
        out = np.empty((nh, self.vd), np.float64)
        lib().or_mla_abs_attn_f64(self._h, _p(q, _f32p), nh, pos, float(scale), _p(out, _f64p))
        return out


def f32_to_f16_bits(a):
    a = _c(a, np.float32).ravel()
    return np.array([lib().or_f32_to_f16(float(v)) for v in a], np.uint16)
