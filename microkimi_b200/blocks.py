"""The two attention blocks of a decode layer over the device calls of this package.

`KdaBlock.forward` stands in for kda_forward (src/model.rs:1179-1232) and `MlaBlock.forward`
for mla_forward (src/model.rs:1939-2022): one token, x and the result are torch CUDA float32
vectors [d], weights and caches stay on the GPU.  The projections that read the same input
are stacked into one matrix at load, so a block is a handful of launches: every row of a
stacked matvec is the same dot() the engine computes for that row, the stacking changes no
bit.  Only views and copies happen in torch; all arithmetic runs in the library's kernels.
"""
import ctypes as C

import numpy as np

from . import lib as _l
from .ops import Context, F32Weight, KdaLayer, MlaCache, rmsnorm


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class KdaBlock:
    """kda_forward.  Weights (host float32, the engine's shapes): q_proj, k_proj, v_proj, g_proj
    [heads*dim, d]; f_a [fa, d]; f_b [heads*dim, fa]; b_proj [heads, d]; o_proj [d, heads*dim];
    q_conv, k_conv, v_conv [heads*dim, kconv]; a_log [dim]; dt_bias [heads*dim]; o_norm [dim]."""

    def __init__(self, heads, dim, w, gate_lb=-5.0, rms_eps=1e-6, ctx=None):
        self.ctx = ctx or Context.default()
        self.heads, self.dim, self.proj = int(heads), int(dim), int(heads) * int(dim)
        d = _f32(w["q_proj"]).shape[1]
        self.d, self.fa = d, _f32(w["f_a"]).shape[0]
        assert self.proj % 4 == 0 and self.fa % 4 == 0, "slices of the stacked result must stay 16-byte aligned"
        # rows in this order: q, k, v, g2 (heads*dim each), f_a (fa), beta (heads)
        stacked = np.concatenate([_f32(w[k]).reshape(-1, d) for k in ("q_proj", "k_proj", "v_proj", "g_proj", "f_a", "b_proj")])
        self.w_x = F32Weight(stacked, stacked.shape[0], d, ctx=self.ctx)
        self.f_b = F32Weight(_f32(w["f_b"]), self.proj, self.fa, ctx=self.ctx)
        self.o_proj = F32Weight(_f32(w["o_proj"]), d, self.proj, ctx=self.ctx)
        kconv = _f32(w["q_conv"]).size // self.proj
        self.state = KdaLayer(heads, dim, w["q_conv"], w["k_conv"], w["v_conv"], w["a_log"], w["dt_bias"], w["o_norm"],
                              kconv=kconv, gate_lb=gate_lb, rms_eps=rms_eps, ctx=self.ctx)

    def forward(self, x):
        p = self.proj
        y = self.w_x.matvec(x)                                   # src/model.rs:1191-1207, one launch
        q, k, v, g2 = y[0:p], y[p:2 * p], y[2 * p:3 * p], y[3 * p:4 * p]
        fa, beta = y[4 * p:4 * p + self.fa], y[4 * p + self.fa:]
        g_low = self.f_b.matvec(fa)                              # :1197-1199
        o = self.state.step(q, k, v, g_low, beta, g2)            # :1211-1228
        return self.o_proj.matvec(o)                             # :1229-1230

    def free(self):
        for h in (self.w_x, self.f_b, self.o_proj, self.state):
            h.free()


class MlaBlock:
    """mla_forward with the q8_0 cache (no positional encoding: the rope slice is the shared part of K).
    Weights (host float32): q_a [qa, d], q_a_ln [qa], q_b [heads*(nope+rope), qa], kv_a [kva+rope, d],
    kv_a_ln [kva], kv_b [heads*(nope+v), kva], g_proj [heads*v, d], o_proj [d, heads*v]."""

    def __init__(self, heads, nope, rope, vd, w, max_positions, rms_eps=1e-6, ctx=None):
        import torch
        self.ctx = ctx or Context.default()
        self.H, self.nope, self.rope, self.vd, self.eps = int(heads), int(nope), int(rope), int(vd), float(rms_eps)
        d = _f32(w["q_a"]).shape[1]
        self.d, self.qa, self.kva = d, _f32(w["q_a"]).shape[0], _f32(w["kv_a_ln"]).size
        assert self.qa % 4 == 0 and (self.kva + self.rope) % 4 == 0 and self.kva % 4 == 0
        stacked = np.concatenate([_f32(w[k]).reshape(-1, d) for k in ("q_a", "kv_a", "g_proj")])
        self.w_x = F32Weight(stacked, stacked.shape[0], d, ctx=self.ctx)
        self.q_b = F32Weight(_f32(w["q_b"]), self.H * (nope + rope), self.qa, ctx=self.ctx)
        self.kv_b = F32Weight(_f32(w["kv_b"]), self.H * (nope + vd), self.kva, ctx=self.ctx)
        self.o_proj = F32Weight(_f32(w["o_proj"]), d, self.H * vd, ctx=self.ctx)
        dev = torch.device("cuda", self.ctx.device)
        self.q_a_ln = torch.from_numpy(_f32(w["q_a_ln"])).to(dev)
        self.kv_a_ln = torch.from_numpy(_f32(w["kv_a_ln"])).to(dev)
        self.cache = MlaCache(heads, nope, rope, vd, max_positions, ctx=self.ctx)
        self.scale = float(np.float32(nope + rope) ** np.float32(-0.5))   # (mla_qh as f32).powf(-0.5), :1977

    def forward(self, x):
        import torch
        H, nope, rope, vd = self.H, self.nope, self.rope, self.vd
        y = self.w_x.matvec(x)                                              # q_a, kv_a, g_proj of x: :1949, :1957, :2016
        qa, c, g = y[:self.qa], y[self.qa:self.qa + self.kva + rope], y[self.qa + self.kva + rope:]
        q = self.q_b.matvec(rmsnorm(qa, self.q_a_ln, self.eps, ctx=self.ctx))             # :1950-1954
        kb = self.kv_b.matvec(rmsnorm(c[:self.kva], self.kv_a_ln, self.eps, ctx=self.ctx))  # :1959-1962
        kb = kb.view(H, nope + vd)
        k_new = torch.cat([kb[:, :nope], c[self.kva:].unsqueeze(0).expand(H, rope)], dim=1).contiguous()  # :1964-1973
        v_new = kb[:, nope:].contiguous()
        self.cache.push(k_new, v_new)                                       # :1974
        attn = self.cache.attend_batch(q.view(1, H, nope + rope), self.scale).view(-1)   # :1982-1988
        _l.check(self.ctx._L.mk_sigmoid_gate_dev(self.ctx._h, C.c_void_p(attn.data_ptr()), C.c_void_p(g.data_ptr()), attn.numel()))
        return self.o_proj.matvec(attn)                                     # :2020-2021

    def free(self):
        for h in (self.w_x, self.q_b, self.kv_b, self.o_proj, self.cache):
            h.free()
