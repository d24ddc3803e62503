"""Host-side mirror of the engine's operator interface for the quantized decode
path, on top of the C ABI.  Names and argument meaning follow the Rust
functions they stand in for:

    matvec_packed(packed, scales, rows, cols, x)        src/mxfp4.rs:458
    Q8Head.from_f32(w, rows, cols) / .matvec(x)         src/model.rs:274, 290
    quantize_q8(x)                                      src/q8.rs:40

Like the engine's operators, size mismatches raise (the Rust code asserts).
numpy arrays go through the host-pointer entry points (copies inside the
call); torch CUDA tensors go through the `_dev` entry points on torch's
current stream.
"""
import ctypes as C

import numpy as np

from . import lib as _l


def _np_ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def _is_torch_cuda(x):
    return type(x).__module__.startswith("torch") and getattr(x, "is_cuda", False)


class Context:
    """One GPU binding (mk_init). Thread-compatible, not re-entrant."""

    _default = None

    def __init__(self, device=0):
        L = _l.load()
        h = C.c_void_p()
        _l.check(L.mk_init(int(device), C.byref(h)))
        self._h = h
        self.device = int(device)
        self._L = L

    @classmethod
    def default(cls):
        if cls._default is None:
            cls._default = cls(0)
        return cls._default

    def close(self):
        if getattr(self, "_h", None):
            self._L.mk_shutdown(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def use_torch_stream(self):
        """Run subsequent calls on torch's current CUDA stream of this device."""
        import torch
        s = torch.cuda.current_stream(self.device).cuda_stream
        _l.check(self._L.mk_set_stream(self._h, C.c_void_p(s)))
        self._stream = s

    def _follow_torch(self):
        """Every call that takes torch CUDA tensors runs on torch's current stream, so that it is ordered
        after the work that produced its inputs and before the work that reads its outputs."""
        import torch
        if torch.cuda.current_stream(self.device).cuda_stream != getattr(self, "_stream", None):
            self.use_torch_stream()

    def sync(self):
        _l.check(self._L.mk_sync(self._h))

    @property
    def launches(self):
        return int(self._L.mk_launch_count(self._h))

    def device_info(self):
        sm, ma, mi, mem = C.c_int32(), C.c_int32(), C.c_int32(), C.c_uint64()
        _l.check(self._L.mk_device_info(self._h, C.byref(sm), C.byref(ma), C.byref(mi), C.byref(mem)))
        return {"sm_count": sm.value, "cc": (ma.value, mi.value), "mem_bytes": mem.value}

    def set_option(self, name, value):
        _l.check(self._L.mk_set_option(self._h, name.encode(), int(value)))

    def prof_enable(self, on=True):
        _l.check(self._L.mk_prof_enable(self._h, int(bool(on))))

    def prof_read(self, category):
        """(launches, total device ms) of one kernel category since prof_enable(True)."""
        n, ms = C.c_int64(), C.c_double()
        _l.check(self._L.mk_prof_read(self._h, _l.PROF_CATEGORIES[category], C.byref(n), C.byref(ms)))
        return n.value, ms.value

    def status_word(self):
        v = C.c_int32()
        _l.check(self._L.mk_status_word(self._h, C.byref(v)))
        return v.value


def _act_mode(act, strict):
    m = {"q8": _l.MK_ACT_Q8, "q8x2": _l.MK_ACT_Q8X2}[act]
    return m | (_l.MK_ACT_STRICT if strict else 0)


class _Weight:
    def __init__(self, ctx, handle, rows, cols):
        self.ctx, self._h, self.rows, self.cols = ctx, handle, int(rows), int(cols)

    def free(self):
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._L.mk_weight_free(self.ctx._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    @property
    def device_bytes(self):
        return int(self.ctx._L.mk_weight_bytes(self._h))

    def _run(self, fn_host, fn_dev, x, act, strict, extra=()):
        import_torch = _is_torch_cuda(x)
        mode = _act_mode(act, strict)
        if import_torch:
            import torch
            self.ctx._follow_torch()
            assert x.dtype == torch.float32 and x.is_contiguous()
            batch = 1 if x.dim() == 1 else x.shape[0]
            assert x.shape[-1] == self.cols, "x length must equal cols"
            y = torch.empty((batch, self.rows), dtype=torch.float32, device=x.device)
            return batch, y, fn_dev, (C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), batch, mode)
        x = np.ascontiguousarray(x, dtype=np.float32)
        batch = 1 if x.ndim == 1 else x.shape[0]
        assert x.shape[-1] == self.cols, "x length must equal cols"
        y = np.empty((batch, self.rows), np.float32)
        return batch, y, fn_host, (_np_ptr(x), _np_ptr(y), batch, mode)


class MxFp4Weight(_Weight):
    """An MXFP4 matrix resident on the GPU: packed u8 [rows, cols/2] + ue8m0 scales
    u8 [rows, cols/32] (BinFile::mxfp4_parts, src/weights.rs:619-626)."""

    def __init__(self, packed, scales, rows, cols, ctx=None):
        ctx = ctx or Context.default()
        h = C.c_void_p()
        if _is_torch_cuda(packed):
            ctx._follow_torch()
            assert packed.numel() == rows * cols // 2 and scales.numel() == rows * cols // 32
            _l.check(ctx._L.mk_weight_mxfp4(ctx._h, C.c_void_p(packed.data_ptr()), C.c_void_p(scales.data_ptr()),
                                            rows, cols, 1, C.byref(h)))
        else:
            packed = np.ascontiguousarray(packed, dtype=np.uint8)
            scales = np.ascontiguousarray(scales, dtype=np.uint8)
            assert packed.size == rows * cols // 2, "packed must hold rows*cols/2 bytes"
            assert scales.size == rows * cols // 32, "scales must hold rows*cols/32 bytes"
            _l.check(ctx._L.mk_weight_mxfp4(ctx._h, _np_ptr(packed), _np_ptr(scales), rows, cols, 0, C.byref(h)))
        super().__init__(ctx, h, rows, cols)

    def matvec(self, x, act="q8", strict=False):
        """y = W x (mxfp4::matvec_packed). x: [cols] or [batch, cols]."""
        L = self.ctx._L
        batch, y, fn, args = self._run(L.mk_matvec_mxfp4, L.mk_matvec_mxfp4_dev, x, act, strict)
        _l.check(fn(self.ctx._h, self._h, *args))
        return y[0] if (x.ndim if hasattr(x, "ndim") else x.dim()) == 1 else y

    def matvec_noalloc(self, x, act="q8", strict=False):
        """matvec for callers that must not allocate device memory while running (their
        memory is fully budgeted, or a cudaMalloc stall is not acceptable): the activation
        scratch is a fixed array inside the library.  x: torch CUDA tensor [batch, cols]
        (or [cols]) with batch <= 8 and cols <= 16384; larger shapes raise.  Calls share
        that array, so keep them on one stream."""
        import torch
        assert _is_torch_cuda(x) and x.dtype == torch.float32 and x.is_contiguous()
        self.ctx._follow_torch()
        batch = 1 if x.dim() == 1 else x.shape[0]
        assert x.shape[-1] == self.cols, "x length must equal cols"
        y = torch.empty((batch, self.rows), dtype=torch.float32, device=x.device)
        _l.check(self.ctx._L.mk_matvec_mxfp4_noalloc_dev(self.ctx._h, self._h, C.c_void_p(x.data_ptr()),
                                                         C.c_void_p(y.data_ptr()), batch, _act_mode(act, strict)))
        return y[0] if x.dim() == 1 else y

    def dequant(self):
        """mxfp4::dequant on the GPU -> f32 [rows, cols] (numpy)."""
        out = np.empty((self.rows, self.cols), np.float32)
        _l.check(self.ctx._L.mk_dequant_mxfp4(self.ctx._h, self._h, _np_ptr(out)))
        return out

    def export(self):
        p = np.empty((self.rows, self.cols // 2), np.uint8)
        s = np.empty((self.rows, self.cols // 32), np.uint8)
        _l.check(self.ctx._L.mk_weight_export(self.ctx._h, self._h, _np_ptr(p), _np_ptr(s)))
        return p, s


class F32Weight(_Weight):
    """A dense f32 matrix [rows, cols] resident on the GPU (the operand of the engine's
    matvec, src/model.rs:199)."""

    def __init__(self, w, rows, cols, ctx=None):
        ctx = ctx or Context.default()
        h = C.c_void_p()
        if _is_torch_cuda(w):
            import torch
            ctx._follow_torch()
            assert w.dtype == torch.float32 and w.is_contiguous() and w.numel() == rows * cols
            _l.check(ctx._L.mk_weight_f32(ctx._h, C.c_void_p(w.data_ptr()), rows, cols, 1, C.byref(h)))
        else:
            w = np.ascontiguousarray(w, dtype=np.float32)
            assert w.size == rows * cols, "w must hold rows*cols floats"
            _l.check(ctx._L.mk_weight_f32(ctx._h, _np_ptr(w), rows, cols, 0, C.byref(h)))
        super().__init__(ctx, h, rows, cols)

    def matvec(self, x):
        """out[r] = dot(w[r], x) with the engine's dot() order (model::matvec). x: [cols] or [batch, cols]."""
        L = self.ctx._L
        batch, y, fn, args = self._run(L.mk_matvec_f32, L.mk_matvec_f32_dev, x, "q8", False)
        _l.check(fn(self.ctx._h, self._h, *args[:3]))
        return y[0] if (x.ndim if hasattr(x, "ndim") else x.dim()) == 1 else y


class Vq1Weight(_Weight):
    """A VQ1 matrix resident on the GPU: codebook f32 [256, 16] + index bytes u8 [rows, cols/16]
    (src/quant.rs:313-346)."""

    def __init__(self, codebook, indices, rows, cols, ctx=None):
        ctx = ctx or Context.default()
        cb = np.ascontiguousarray(codebook, dtype=np.float32)
        idx = np.ascontiguousarray(indices, dtype=np.uint8)
        assert cb.size == 256 * 16 and idx.size == rows * cols // 16
        h = C.c_void_p()
        _l.check(ctx._L.mk_weight_vq1(ctx._h, _np_ptr(cb), _np_ptr(idx), rows, cols, 0, C.byref(h)))
        super().__init__(ctx, h, rows, cols)

    def matvec(self, x):
        """quant::matvec_vq: out[r] = sum_c W[r, c] x[c], bit-identical to the engine. x: [cols] or [batch, cols]."""
        L = self.ctx._L
        batch, y, fn, args = self._run(L.mk_matvec_vq1, L.mk_matvec_vq1_dev, x, "q8", False)
        _l.check(fn(self.ctx._h, self._h, *args[:3]))
        return y[0] if (x.ndim if hasattr(x, "ndim") else x.dim()) == 1 else y


def dequant_fp8(w, scales, rows, cols, ctx=None):
    """dequant::dequant_fp8 (src/dequant.rs:27-41) on the GPU: numpy u8 in, f32 [rows, cols] out."""
    ctx = ctx or Context.default()
    w = np.ascontiguousarray(w, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    assert w.size == rows * cols and scales.size == -(-rows // 128) * -(-cols // 128)
    out = np.empty((rows, cols), np.float32)
    _l.check(ctx._L.mk_dequant_fp8(ctx._h, _np_ptr(w), _np_ptr(scales), rows, cols, _np_ptr(out)))
    return out


def dequant_any(dtype, blob, rows, cols, ctx=None):
    """mxfp4::dequant_any (src/mxfp4.rs:228-240) on the GPU: `blob` is the raw bytes of an "mxfp4" (packed || scales) or
    "mxfp4sq" (packed || scales || smax) tensor of a model file -> f32 [rows, cols]."""
    ctx = ctx or Context.default()
    code = {"mxfp4": 1, "mxfp4sq": 4}[dtype] if isinstance(dtype, str) else int(dtype)
    b = np.ascontiguousarray(blob, dtype=np.uint8).ravel()
    need = rows * cols // 2 + rows * cols // 32 + (4 if code == 4 else 0)
    assert b.size == need, "blob has the wrong size for this dtype and shape"
    out = np.empty((rows, cols), np.float32)
    _l.check(ctx._L.mk_dequant_mxfp4_blob(ctx._h, code, _np_ptr(b), rows, cols, _np_ptr(out)))
    return out


def matvec(w, rows, cols, x, ctx=None):
    """Drop-in for model::matvec / metal::gpu_matvec with borrowed host slices."""
    h = F32Weight(w, rows, cols, ctx)
    try:
        return h.matvec(x)
    finally:
        h.free()


def rmsnorm(x, w, eps, ctx=None):
    """rmsnorm (src/model.rs:599-605) on torch CUDA rows x [n, len] (or [len]) with weights w [len]."""
    import torch
    ctx = ctx or Context.default()
    assert _is_torch_cuda(x) and _is_torch_cuda(w) and x.dtype == torch.float32 and w.dtype == torch.float32
    assert x.is_contiguous() and w.is_contiguous() and x.shape[-1] == w.numel()
    ctx._follow_torch()
    n = 1 if x.dim() == 1 else x.shape[0]
    out = torch.empty_like(x)
    _l.check(ctx._L.mk_rmsnorm_dev(ctx._h, C.c_void_p(x.data_ptr()), C.c_void_p(w.data_ptr()), n, x.shape[-1], float(eps),
                                   C.c_void_p(out.data_ptr())))
    return out


def attn_res(prefix, blocks, w, eps, ctx=None):
    """attn_res (src/model.rs:625-669) on torch CUDA rows: prefix [d], blocks [b, d] (b may be 0), w [d] -> [d]."""
    import torch
    ctx = ctx or Context.default()
    assert all(_is_torch_cuda(t) and t.dtype == torch.float32 and t.is_contiguous() for t in (prefix, blocks, w))
    ctx._follow_torch()
    d = prefix.numel()
    b = blocks.shape[0] if blocks.numel() else 0
    assert w.numel() == d and (b == 0 or blocks.shape[1] == d)
    out = torch.empty_like(prefix)
    _l.check(ctx._L.mk_attn_res_dev(ctx._h, C.c_void_p(prefix.data_ptr()), C.c_void_p(blocks.data_ptr()) if b else None, d, b,
                                    C.c_void_p(w.data_ptr()), d, float(eps), C.c_void_p(out.data_ptr())))
    return out


class KdaLayer:
    """The device-resident state of one KDA layer (KdaCache, src/model.rs) and the decode step between the
    projections and o_proj (kda_forward, src/model.rs:1203-1228).  Parameter arrays are host float32."""

    def __init__(self, heads, dim, q_conv, k_conv, v_conv, a_log, dt_bias, o_norm, kconv=4, gate_lb=-5.0, rms_eps=1e-6, ctx=None):
        self.ctx = ctx or Context.default()
        self.heads, self.dim, self.kconv = int(heads), int(dim), int(kconv)
        keep = [np.ascontiguousarray(a, dtype=np.float32) for a in (q_conv, k_conv, v_conv, a_log, dt_bias, o_norm)]
        proj = self.heads * self.dim
        assert all(a.size == proj * self.kconv for a in keep[:3]) and keep[3].size == self.dim
        assert keep[4].size == proj and keep[5].size == self.dim
        d = _l.KdaDesc()
        d.heads, d.dim, d.kconv, d.gate_lb, d.rms_eps = self.heads, self.dim, self.kconv, float(gate_lb), float(rms_eps)
        d.q_conv, d.k_conv, d.v_conv, d.a_log, d.dt_bias, d.o_norm = (a.ctypes.data for a in keep)
        h = C.c_void_p()
        _l.check(self.ctx._L.mk_kda_create(self.ctx._h, C.byref(d), C.byref(h)))
        self._h = h

    def step(self, q_raw, k_raw, v_raw, g_low, beta_raw, g2):
        """torch CUDA float32 vectors (q, k, v, g_low, g2 [heads * dim]; beta_raw [heads]) -> o [heads * dim]."""
        import torch
        ins = (q_raw, k_raw, v_raw, g_low, beta_raw, g2)
        assert all(_is_torch_cuda(t) and t.dtype == torch.float32 and t.is_contiguous() for t in ins)
        self.ctx._follow_torch()
        proj = self.heads * self.dim
        assert all(t.numel() == proj for t in (q_raw, k_raw, v_raw, g_low, g2)) and beta_raw.numel() == self.heads
        o = torch.empty(proj, dtype=torch.float32, device=q_raw.device)
        _l.check(self.ctx._L.mk_kda_step_dev(self.ctx._h, self._h, *(C.c_void_p(t.data_ptr()) for t in ins), C.c_void_p(o.data_ptr())))
        return o

    def steps(self, rows, g_low, ld_x, offsets):
        """Several consecutive positions in one launch (mk_kda_steps_dev).  rows: torch CUDA float32 [n, ld_x], every row holding
        q, k, v, g2 [heads * dim each] and beta [heads] at `offsets` = (q, k, v, g2, beta); g_low: [n, heads * dim] -> o [n, heads * dim]."""
        import torch
        assert _is_torch_cuda(rows) and rows.is_contiguous() and _is_torch_cuda(g_low) and g_low.is_contiguous()
        self.ctx._follow_torch()
        n, proj = rows.shape[0], self.heads * self.dim
        o = torch.empty((n, proj), dtype=torch.float32, device=rows.device)
        base = rows.data_ptr()
        oq, ok, ov, og2, ob = (C.c_void_p(base + 4 * int(x)) for x in offsets)
        _l.check(self.ctx._L.mk_kda_steps_dev(self.ctx._h, self._h, n, oq, ok, ov, C.c_void_p(g_low.data_ptr()), ob, og2,
                                              C.c_void_p(o.data_ptr()), int(ld_x), proj, proj))
        return o

    def reset(self):
        _l.check(self.ctx._L.mk_kda_reset(self.ctx._h, self._h))

    def export_state(self):
        """(S [heads, dim, dim], conv [3, kconv - 1, heads * dim]) as host arrays."""
        s = np.empty((self.heads, self.dim, self.dim), np.float32)
        conv = np.empty((3, max(self.kconv - 1, 0), self.heads * self.dim), np.float32)
        _l.check(self.ctx._L.mk_kda_export(self.ctx._h, self._h, _np_ptr(s), C.c_void_p(conv.ctypes.data)))
        return s, conv

    def import_state(self, s, conv):
        s = np.ascontiguousarray(s, dtype=np.float32)
        conv = np.ascontiguousarray(conv, dtype=np.float32)
        assert s.size == self.heads * self.dim * self.dim and conv.size == 3 * (self.kconv - 1) * self.heads * self.dim
        _l.check(self.ctx._L.mk_kda_import(self.ctx._h, self._h, _np_ptr(s), C.c_void_p(conv.ctypes.data)))

    def free(self):
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._L.mk_kda_free(self.ctx._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def matvec_packed(packed, scales, rows, cols, x, act="q8", strict=False, ctx=None):
    """Drop-in for mxfp4::matvec_packed / metal::gpu_matvec_fp4 with borrowed host
    slices: registers the matrix, multiplies, frees.  Callers that reuse a matrix
    keep an MxFp4Weight instead (the engine's device weight cache)."""
    w = MxFp4Weight(packed, scales, rows, cols, ctx)
    try:
        return w.matvec(x, act=act, strict=strict)
    finally:
        w.free()


class Q8Head(_Weight):
    """Row-wise q8_0 matrix (model::Q8Head, src/model.rs:261-348)."""

    def __init__(self, ctx, handle, rows, cols, scale_type):
        super().__init__(ctx, handle, rows, cols)
        self.scale_type = scale_type

    @classmethod
    def from_f32(cls, w, rows, cols, scale="f32", ctx=None):
        """Q8Head::from_f32: quantizes on the GPU (bit-identical for f32 scales)."""
        ctx = ctx or Context.default()
        st = {"f32": _l.MK_SCALE_F32, "f16": _l.MK_SCALE_F16}[scale]
        h = C.c_void_p()
        if _is_torch_cuda(w):
            ctx._follow_torch()
            assert w.numel() == rows * cols and w.is_contiguous()
            _l.check(ctx._L.mk_weight_q8_from_f32(ctx._h, C.c_void_p(w.data_ptr()), rows, cols, st, 1, C.byref(h)))
        else:
            w = np.ascontiguousarray(w, dtype=np.float32)
            assert w.size == rows * cols
            _l.check(ctx._L.mk_weight_q8_from_f32(ctx._h, _np_ptr(w), rows, cols, st, 0, C.byref(h)))
        return cls(ctx, h, rows, cols, st)

    @classmethod
    def from_q8(cls, q, scales, rows, cols, ctx=None):
        ctx = ctx or Context.default()
        q = np.ascontiguousarray(q, dtype=np.int8)
        st = _l.MK_SCALE_F16 if scales.dtype in (np.float16, np.uint16) else _l.MK_SCALE_F32
        scales = np.ascontiguousarray(scales)
        assert q.size == rows * cols and scales.size == rows * cols // 32
        h = C.c_void_p()
        _l.check(ctx._L.mk_weight_q8(ctx._h, _np_ptr(q), _np_ptr(scales), rows, cols, st, 0, C.byref(h)))
        return cls(ctx, h, rows, cols, st)

    def matvec(self, x, act="q8", strict=False, want_argmax=False, out=None, argmax_out=None):
        """Q8Head::matvec: logits [rows] (or [batch, rows]); optionally the greedy pick.  Host arrays only: `out`
        (float32 [batch, rows]) and `argmax_out` (int32 [batch]) are caller-owned result buffers, as the engine's
        `out: &mut [f32]` is; views of pinned memory spare the staging copy of a pageable destination."""
        L = self.ctx._L
        batch, y, fn, args = self._run(L.mk_matvec_q8, L.mk_matvec_q8_dev, x, act, strict)
        if out is not None:
            assert not _is_torch_cuda(x) and out.dtype == np.float32 and out.flags.c_contiguous and out.size == batch * self.rows
            y = out.reshape(batch, self.rows)
            args = (args[0], _np_ptr(y)) + tuple(args[2:])
        am = None
        if want_argmax:
            if _is_torch_cuda(x):
                import torch
                self.ctx._follow_torch()
                am = torch.empty(batch, dtype=torch.int32, device=x.device)
                amp = C.c_void_p(am.data_ptr())
            else:
                am = np.empty(batch, np.int32) if argmax_out is None else argmax_out
                assert am.dtype == np.int32 and am.size == batch
                amp = _np_ptr(am)
        else:
            amp = C.c_void_p(0)
        _l.check(fn(self.ctx._h, self._h, *args, amp))
        one = (x.ndim if hasattr(x, "ndim") else x.dim()) == 1
        y = y[0] if one else y
        return (y, am) if want_argmax else y

    def export(self):
        q = np.empty((self.rows, self.cols), np.int8)
        s = np.empty((self.rows, self.cols // 32), np.float16 if self.scale_type == _l.MK_SCALE_F16 else np.float32)
        _l.check(self.ctx._L.mk_weight_export(self.ctx._h, self._h, _np_ptr(q), _np_ptr(s)))
        return q, s


class MoeLayer:
    """One MoE layer resident on the GPU.

    Default: the noaux_tc router of moe_forward (src/model.rs:2153-2173) feeding MXFP4
    experts with the SwiGLU-clamp body of ds_moe (src/deepseek.rs:1038-1108), plus one
    unweighted MXFP4 shared expert.
    router="sqrt_softplus": DeepSeek's gate_forward (src/deepseek.rs:16-58) with route_scale.
    activation="situ": the K3 body (src/model.rs:2202-2380) - SiTU, routing weight applied
    to the expert outputs; with routed_down / routed_up (F32Weight) and routed_norm the
    experts work on the latent h = routed_down x and the layer returns
    routed_up rmsnorm(y); shared_f32 = (gate, down, up) F32Weights is the f32 shared expert.

    experts: list over expert ids of (w1, w2, w3) MxFp4Weight triples, or None for an
    expert that lives on another GPU (expert parallel); shared: one triple or None.
    `dx` is the layer's input/output width, `d` the width the experts work on.
    """

    def __init__(self, gate_w, gate_b, experts, shared, top_k, swiglu_limit=10.0, ctx=None, router="sigmoid",
                 route_scale=1.0, activation="swiglu_clamp", routed_down=None, routed_up=None, routed_norm=None,
                 rms_eps=1e-6, shared_f32=None, strict=False, act="q8"):
        ctx = ctx or Context.default()
        self.ctx = ctx
        self.n_experts = len(experts)
        self.resident = [t is not None for t in experts]     # routed experts held by this GPU (expert parallelism: a subset)
        self.top_k = int(top_k)
        first = next(t for t in list(experts) + [shared] if t is not None)
        self.inter, self.d = first[0].rows, first[0].cols
        self.dx = routed_down.cols if routed_down is not None else self.d
        self.has_shared = shared is not None
        self._keep = (experts, shared, routed_down, routed_up, shared_f32)
        tbl = (C.c_void_p * (3 * self.n_experts))()
        for e, tri in enumerate(experts):
            for j in range(3):
                tbl[3 * e + j] = tri[j]._h if tri is not None else None
        desc = _l.MoeDesc()
        desc.n_experts, desc.top_k, desc.d, desc.inter = self.n_experts, self.top_k, self.dx, self.inter
        desc.swiglu_limit = float(swiglu_limit)
        desc.activation = {"swiglu_clamp": _l.MK_MOE_SWIGLU_CLAMP, "situ": _l.MK_MOE_SITU}[activation]
        desc.router = {"sigmoid": _l.MK_ROUTER_SIGMOID, "sqrt_softplus": _l.MK_ROUTER_SQRT_SOFTPLUS}[router]
        desc.route_scale, desc.rms_eps = float(route_scale), float(rms_eps)
        # act="fp4x6": calls of >= 4 rows run the experts on the block-scaled tcgen05 path (six E2M1 limbs per activation; widths must be multiples of 256)
        desc.act_mode = _l.MK_ACT_FP4X6 if act == "fp4x6" else (_l.MK_ACT_Q8 | (_l.MK_ACT_STRICT if strict else 0))
        if routed_down is not None:
            rn = np.ascontiguousarray(routed_norm, dtype=np.float32)
            assert rn.size == self.d, "routed_norm must hold one weight per latent column"
            desc.latent = self.d
            desc.routed_down, desc.routed_up, desc.routed_norm = routed_down._h, routed_up._h, _np_ptr(rn)
        for j in range(3):
            desc.shared_f32[j] = shared_f32[j]._h if shared_f32 is not None else None
        self._gate_w = gate_w
        if gate_w is not None:
            gw = np.ascontiguousarray(gate_w, dtype=np.float32)
            assert gw.shape == (self.n_experts, self.dx)
            gb = np.ascontiguousarray(gate_b if gate_b is not None else np.zeros(self.n_experts), dtype=np.float32)
            desc.gate_w, desc.gate_b = _np_ptr(gw), _np_ptr(gb)
        desc.experts = C.cast(tbl, C.POINTER(C.c_void_p))
        for j in range(3):
            desc.shared[j] = shared[j]._h if shared is not None else None
        h = C.c_void_p()
        _l.check(ctx._L.mk_moe_create(ctx._h, C.byref(desc), C.byref(h)))
        self._h = h

    def free(self):
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._L.mk_moe_free(self.ctx._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def route(self, x, want_logits=False):
        """Router only: (ids [n, top_k] int32, weights [n, top_k] f32[, logits [n, E]])."""
        if _is_torch_cuda(x):
            import torch
            self.ctx._follow_torch()
            xs = x.reshape(-1, self.dx)
            n = xs.shape[0]
            ids = torch.empty((n, self.top_k), dtype=torch.int32, device=x.device)
            w = torch.empty((n, self.top_k), dtype=torch.float32, device=x.device)
            lg = torch.empty((n, self.n_experts), dtype=torch.float32, device=x.device) if want_logits else None
            _l.check(self.ctx._L.mk_moe_route_dev(self.ctx._h, self._h, C.c_void_p(xs.data_ptr()), n, C.c_void_p(ids.data_ptr()),
                                                  C.c_void_p(w.data_ptr()), C.c_void_p(lg.data_ptr()) if want_logits else None))
            return (ids, w, lg) if want_logits else (ids, w)
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.dx)
        n = x.shape[0]
        ids = np.empty((n, self.top_k), np.int32)
        w = np.empty((n, self.top_k), np.float32)
        lg = np.empty((n, self.n_experts), np.float32) if want_logits else None
        _l.check(self.ctx._L.mk_moe_route(self.ctx._h, self._h, _np_ptr(x), n, _np_ptr(ids), _np_ptr(w),
                                          _np_ptr(lg) if want_logits else None))
        return (ids, w, lg) if want_logits else (ids, w)

    def moe_forward(self, x, want_routing=False):
        """moe_forward / ds_moe for n token rows: x [n, d] (or [d]) -> out of the same shape."""
        L = self.ctx._L
        if _is_torch_cuda(x):
            import torch
            self.ctx._follow_torch()
            xs = x.reshape(-1, self.dx)
            assert xs.dtype == torch.float32 and xs.is_contiguous()
            n = xs.shape[0]
            out = torch.empty_like(xs)
            ids = torch.empty((n, self.top_k), dtype=torch.int32, device=x.device) if want_routing else None
            w = torch.empty((n, self.top_k), dtype=torch.float32, device=x.device) if want_routing else None
            _l.check(L.mk_moe_forward_dev(self.ctx._h, self._h, C.c_void_p(xs.data_ptr()), n, C.c_void_p(out.data_ptr()),
                                          C.c_void_p(ids.data_ptr()) if want_routing else None,
                                          C.c_void_p(w.data_ptr()) if want_routing else None))
            out = out.reshape(x.shape)
        else:
            xa = np.ascontiguousarray(x, dtype=np.float32)
            xs = xa.reshape(-1, self.dx)
            n = xs.shape[0]
            out = np.empty_like(xs)
            ids = np.empty((n, self.top_k), np.int32) if want_routing else None
            w = np.empty((n, self.top_k), np.float32) if want_routing else None
            _l.check(L.mk_moe_forward(self.ctx._h, self._h, _np_ptr(xs), n, _np_ptr(out),
                                      _np_ptr(ids) if want_routing else None, _np_ptr(w) if want_routing else None))
            out = out.reshape(xa.shape)
        return (out, ids, w) if want_routing else out

    def experts_dev(self, x, pair_row, pair_expert, pair_weight):
        """Grouped experts on explicit pairs (torch CUDA tensors): outs [n_pairs, d]."""
        import torch
        self.ctx._follow_torch()
        n_pairs = pair_row.numel()
        outs = torch.empty((n_pairs, self.d), dtype=torch.float32, device=x.device)
        _l.check(self.ctx._L.mk_moe_experts_dev(self.ctx._h, self._h, C.c_void_p(x.data_ptr()), x.shape[0],
                                                C.c_void_p(pair_row.data_ptr()), C.c_void_p(pair_expert.data_ptr()),
                                                C.c_void_p(pair_weight.data_ptr()), n_pairs, C.c_void_p(outs.data_ptr())))
        return outs

    def combine_dev(self, outs, n_tokens, slots):
        import torch
        self.ctx._follow_torch()
        out = torch.empty((n_tokens, self.d), dtype=torch.float32, device=outs.device)
        _l.check(self.ctx._L.mk_moe_combine_dev(self.ctx._h, C.c_void_p(outs.data_ptr()), n_tokens, slots, self.d,
                                                C.c_void_p(out.data_ptr())))
        return out


class MlaCache:
    """q8_0 MLA KV cache on the GPU (model::MlaCache, src/model.rs:765-781) with the
    all-heads decode attention (mla_attn_flash_q8_mqa, src/model.rs:1804-1908).

    layout "per_head": the engine's layout (nope K and V q8_0 per head, rope f32 once).
    layout "absorbed": one shared q8_0 latent row of width `nope` per position
    (rope = 0), V = its first vd columns.  n_seqs independent sequences.
    """

    def __init__(self, n_heads, nope, rope, vd, max_positions, n_seqs=1, layout="per_head", ctx=None):
        ctx = ctx or Context.default()
        self.ctx = ctx
        self.H, self.nope, self.rope, self.vd = n_heads, nope, rope, vd
        self.cap, self.n_seqs, self.layout = max_positions, n_seqs, layout
        d = _l.MlaDesc(0 if layout == "per_head" else 1, n_heads, nope, rope, vd, max_positions, n_seqs)
        h = C.c_void_p()
        _l.check(ctx._L.mk_mla_create(ctx._h, C.byref(d), C.byref(h)))
        self._h = h

    def free(self):
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._L.mk_mla_free(self.ctx._h, self._h)
        self._h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def positions(self, seq=0):
        n = self.ctx._L.mk_mla_positions(self.ctx._h, self._h, seq)
        if n < 0:
            _l.check(n)
        return n

    def reset(self, seq=-1):
        _l.check(self.ctx._L.mk_mla_reset(self.ctx._h, self._h, seq))

    def push(self, k_row, v_row=None, seq=0):
        """MlaCache::push for one or more consecutive positions.
        per_head: k_row [n, H, nope+rope], v_row [n, H, vd]; absorbed: k_row [n, nope]."""
        L = self.ctx._L
        kdim = self.nope if self.layout == "absorbed" else self.H * (self.nope + self.rope)
        if _is_torch_cuda(k_row):
            self.ctx._follow_torch()
            n = k_row.numel() // kdim
            vp = C.c_void_p(v_row.data_ptr()) if v_row is not None else None
            _l.check(L.mk_mla_append_dev(self.ctx._h, self._h, seq, C.c_void_p(k_row.data_ptr()), vp, n))
            return
        k = np.ascontiguousarray(k_row, dtype=np.float32)
        assert k.size % kdim == 0, "k_row has the wrong size"
        n = k.size // kdim
        v = None
        if self.layout != "absorbed":
            v = np.ascontiguousarray(v_row, dtype=np.float32)
            assert v.size == n * self.H * self.vd, "v_row has the wrong size"
        _l.check(L.mk_mla_append(self.ctx._h, self._h, seq, _np_ptr(k), _np_ptr(v) if v is not None else None, n))

    def mla_attn_flash_q8_mqa(self, q, pos, scale, seq=0):
        """Attention of q [H, nope+rope] over positions 0..=pos -> [H, vd]."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        assert q.size == self.H * (self.nope + self.rope), "q has the wrong size"
        out = np.empty((self.H, self.vd), np.float32)
        _l.check(self.ctx._L.mk_mla_attend(self.ctx._h, self._h, seq, _np_ptr(q), int(pos), float(scale), _np_ptr(out)))
        return out

    def attend_batch(self, q, scale):
        """All sequences at once (torch CUDA q [n_seqs, H, qdim]) over all positions each holds."""
        import torch
        self.ctx._follow_torch()
        assert q.is_contiguous() and q.dtype == torch.float32 and q.numel() == self.n_seqs * self.H * (self.nope + self.rope)
        out = torch.empty((self.n_seqs, self.H, self.vd), dtype=torch.float32, device=q.device)
        _l.check(self.ctx._L.mk_mla_attend_batch_dev(self.ctx._h, self._h, C.c_void_p(q.data_ptr()), float(scale),
                                                     C.c_void_p(out.data_ptr())))
        return out

    def decode_step(self, k_row, v_row, q, scale, seq=0):
        """One position appended at the device-side count, then attention over everything held (torch CUDA tensors;
        per_head: k_row [H, nope+rope], v_row [H, vd], q [H, nope+rope]) -> [H, vd]."""
        import torch
        self.ctx._follow_torch()
        out = torch.empty((self.H, self.vd), dtype=torch.float32, device=q.device)
        vp = C.c_void_p(v_row.data_ptr()) if v_row is not None else None
        _l.check(self.ctx._L.mk_mla_decode_step_dev(self.ctx._h, self._h, seq, C.c_void_p(k_row.data_ptr()), vp, C.c_void_p(q.data_ptr()),
                                                    float(scale), C.c_void_p(out.data_ptr())))
        return out

    def prefill(self, k_rows, v_rows, q_rows, scale, seq=0):
        """n consecutive positions in one go: rows appended together, row b attends up to its own position (torch CUDA
        tensors; per_head: k_rows [n, H, nope+rope], v_rows [n, H, vd], q_rows [n, H, nope+rope]) -> [n, H, vd]."""
        import torch
        self.ctx._follow_torch()
        n = q_rows.shape[0]
        out = torch.empty((n, self.H, self.vd), dtype=torch.float32, device=q_rows.device)
        vp = C.c_void_p(v_rows.data_ptr()) if v_rows is not None else None
        _l.check(self.ctx._L.mk_mla_prefill_dev(self.ctx._h, self._h, seq, C.c_void_p(k_rows.data_ptr()), vp, C.c_void_p(q_rows.data_ptr()),
                                                int(n), float(scale), C.c_void_p(out.data_ptr())))
        return out

    def export(self, seq=0):
        """Cache contents in the engine's layout: dict of kq, ks (, kr, vq, vs)."""
        n = self.positions(seq)
        kvh = 1 if self.layout == "absorbed" else self.H
        out = {"kq": np.empty((n, kvh, self.nope), np.int8), "ks": np.empty((n, kvh, self.nope // 32), np.float32)}
        ptr = lambda k: _np_ptr(out[k]) if k in out and out[k].size else None
        if self.layout != "absorbed":
            out["kr"] = np.empty((n, self.rope), np.float32)
            out["vq"] = np.empty((n, kvh, self.vd), np.int8)
            out["vs"] = np.empty((n, kvh, self.vd // 32), np.float32)
        _l.check(self.ctx._L.mk_mla_export(self.ctx._h, self._h, seq, ptr("kq"), ptr("ks"), ptr("kr"), ptr("vq"), ptr("vs")))
        return out


def _mla_to_f32(self, seq=0):
    """MlaCache::to_f32: (k [n, H, nope + rope], v [n, H, vd]) float32 (absorbed: (k [n, nope], None))."""
    n = self.positions(seq)
    if self.layout == "absorbed":
        k, v = np.empty((n, self.nope), np.float32), None
    else:
        k, v = np.empty((n, self.H, self.nope + self.rope), np.float32), np.empty((n, self.H, self.vd), np.float32)
    _l.check(self.ctx._L.mk_mla_export_f32(self.ctx._h, self._h, seq, _np_ptr(k), _np_ptr(v) if v is not None else None))
    return k, v


def _mla_assign_f32(self, k, v=None, seq=0):
    """MlaCache::assign_f32: replaces the sequence's contents by f32 rows (requantized on the way in)."""
    k = np.ascontiguousarray(k, dtype=np.float32)
    kdim = self.nope if self.layout == "absorbed" else self.H * (self.nope + self.rope)
    n = k.size // kdim
    vv = None if self.layout == "absorbed" else np.ascontiguousarray(v, dtype=np.float32)
    _l.check(self.ctx._L.mk_mla_import_f32(self.ctx._h, self._h, seq, _np_ptr(k), _np_ptr(vv) if vv is not None else None, n))


MlaCache.to_f32 = _mla_to_f32
MlaCache.assign_f32 = _mla_assign_f32


def quantize_q8(x, ctx=None):
    """q8::quantize_q8 on the GPU: (q int8 [n], scales f32 [n/32])."""
    ctx = ctx or Context.default()
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    assert x.size % 32 == 0, "q8 blocks are 32 wide"
    q = np.empty(x.size, np.int8)
    s = np.empty(x.size // 32, np.float32)
    _l.check(ctx._L.mk_quantize_q8(ctx._h, _np_ptr(x), x.size, _np_ptr(q), _np_ptr(s)))
    return q, s
