"""GPU parity tests for the f32 pieces of the decode path (model::matvec, rmsnorm),
through the C ABI, against the CPU oracle on the same seeded inputs.

The kernels keep the engine's dot() order (src/model.rs:63-82: 8 accumulators, separate
multiply and add, fixed reduction, sequential tail), so every comparison here is
bit-exact.
"""
import os

import numpy as np
import pytest

from conftest import GOLDEN, bits
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mk():
    import microkimi_b200 as m
    m.Context.default()
    return m


def oracle_matvec(w, x):
    return np.stack([O.matvec_f32(w, x[b]) for b in range(x.shape[0])])


# shapes: the tiled path (cols % 4 == 0) with and without a tail of cols % 8, one row tile that
# is not full, and the generic path (cols % 4 != 0)
@pytest.mark.parametrize("rows,cols", [(128, 512), (512, 128), (37, 200), (64, 36), (5, 8), (33, 1028), (19, 101), (7, 3)])
@pytest.mark.parametrize("batch", [1, 2, 3, 5, 9, 17, 50, 64])     # from 48 rows on: the register-tiled 16 x 16 product
def test_f32_matvec_bit_exact(mk, rows, cols, batch):
    rng = np.random.default_rng(rows * 1000 + cols + batch)
    w = (rng.standard_normal((rows, cols)) * 0.05).astype(np.float32)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    h = mk.F32Weight(w, rows, cols)
    y = h.matvec(x)
    ref = oracle_matvec(w, x)
    assert np.array_equal(bits(y), bits(ref))
    y1 = h.matvec(x[0])
    assert np.array_equal(bits(y1), bits(ref[0]))
    h.free()


def test_f32_matvec_device_pointers_and_large(mk):
    import torch
    rows, cols, batch = 2048, 7168, 4
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    w = torch.randn((rows, cols), device="cuda", generator=gen) * 0.02
    x = torch.randn((batch, cols), device="cuda", generator=gen)
    h = mk.F32Weight(w, rows, cols)
    y = h.matvec(x).cpu().numpy()
    ref = oracle_matvec(w.cpu().numpy(), x.cpu().numpy())
    assert np.array_equal(bits(y), bits(ref))
    h.free()


def test_f32_matvec_golden_ds_expert(mk):
    """The DeepSeek expert of ref/ds_golden2.json (src/selftest.rs:314-323) through three GPU
    matvecs and the host-side SwiGLU-clamp: same tolerance as the reference's check (1e-4)."""
    g = np.load(os.path.join(GOLDEN, "ds_gate_expert.npz"))
    w1, w2, w3, x, want = g["ex_w1"], g["ex_w2"], g["ex_w3"], g["ex_x"], g["ex_out"]
    limit = 10.0
    inter, d = w1.shape
    gate = mk.matvec(w1, inter, d, x)
    up = mk.matvec(w3, inter, d, x)
    gl, ul = np.minimum(gate, limit), np.clip(up, -limit, limit)
    act = ((gl / (1.0 + np.exp(-gl))) * ul).astype(np.float32)
    y = mk.matvec(w2, d, inter, act)
    assert np.abs(y - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    assert np.array_equal(bits(gate), bits(O.matvec_f32(w1, x)))


@pytest.mark.parametrize("n,length", [(1, 128), (3, 512), (5, 100), (2, 7)])
def test_rmsnorm_bit_exact(mk, n, length):
    import torch
    rng = np.random.default_rng(n * 100 + length)
    x = rng.standard_normal((n, length)).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(length)).astype(np.float32)
    out = mk.rmsnorm(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), 1e-6).cpu().numpy()
    ref = np.stack([O.rmsnorm(x[i], w, 1e-6) for i in range(n)])
    assert np.array_equal(bits(out), bits(ref))


def test_f32_matvec_argument_errors(mk):
    from microkimi_b200 import lib as L
    w = np.zeros((4, 8), np.float32)
    h = mk.F32Weight(w, 4, 8)
    with pytest.raises(AssertionError):
        h.matvec(np.zeros(7, np.float32))
    fp4 = mk.MxFp4Weight(np.zeros((16, 16), np.uint8), np.zeros((16, 1), np.uint8), 16, 32)
    with pytest.raises(L.MkError):
        # an MXFP4 handle passed to the f32 entry point is refused, not reinterpreted
        L.check(h.ctx._L.mk_matvec_f32(h.ctx._h, fp4._h, None, None, 1))
    h.free()
    fp4.free()


# ------------------------------------------------------------------ VQ1 codebook matvec by lookup table
@pytest.mark.parametrize("rows,cols", [(7, 16), (130, 272), (7168, 2048), (300, 7168)])
@pytest.mark.parametrize("batch", [1, 3, 9])
def test_vq1_matvec_bit_exact(mk, rows, cols, batch):
    """quant::matvec_vq (src/quant.rs:340-346; lutgemv.rs:208-238): bit-identical to the CPU, as the
    reference's own LUT kernel is to its gather kernel."""
    rng = np.random.default_rng(rows + cols + batch)
    cb = (rng.standard_normal((256, 16)) * 0.05).astype(np.float32)
    idx = rng.integers(0, 256, (rows, cols // 16), dtype=np.uint8)
    x = rng.standard_normal((batch, cols)).astype(np.float32)
    w = mk.Vq1Weight(cb, idx, rows, cols)
    y = w.matvec(x)
    ref = np.stack([O.matvec_vq(cb, idx, x[b]) for b in range(batch)])
    assert np.array_equal(bits(y), bits(ref))
    assert np.array_equal(bits(w.matvec(x[0])), bits(ref[0]))
    w.free()


# ------------------------------------------------------------------ KDA decode step, AttnRes
def _kda_params(rng, heads, dim, kconv):
    proj = heads * dim
    cw = [(rng.standard_normal((proj, kconv)) * 0.5).astype(np.float32) for _ in range(3)]
    a_log = np.log(rng.uniform(1.0, 16.0, dim)).astype(np.float32)      # the builder's A_log = ln(U(1, 16))
    dt_bias = (rng.standard_normal(proj) * 0.3).astype(np.float32)
    o_norm = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    return cw, a_log, dt_bias, o_norm


# (4, 128): the engine's heads and kda_dim; (2, 64): the other register-resident size; (3, 40): the generic kernel
# with a partly filled last warp; kconv 2: a one-row window
@pytest.mark.parametrize("heads,dim,kconv", [(4, 128, 4), (2, 64, 4), (3, 40, 4), (2, 128, 2), (1, 8, 3)])
def test_kda_step_against_oracle(mk, heads, dim, kconv):
    """kda_forward between its projections and o_proj (src/model.rs:1203-1228), 8 tokens in a row.  Every sum keeps
    the engine's order, exp comes from double precision rounded once: tolerance 1e-6 relative to the largest value
    (a differing last bit of one exp), and the run normally is bit-identical, which the test reports."""
    import torch
    rng = np.random.default_rng(heads * 1000 + dim + kconv)
    cw, a_log, dt_bias, o_norm = _kda_params(rng, heads, dim, kconv)
    proj = heads * dim
    ref = O.KdaLayer(heads, dim, *cw, a_log, dt_bias, o_norm, kconv=kconv, gate_lb=-5.0, rms_eps=1e-6)
    dev = mk.KdaLayer(heads, dim, *cw, a_log, dt_bias, o_norm, kconv=kconv, gate_lb=-5.0, rms_eps=1e-6)
    exact = True
    for t in range(8):
        ins = [rng.standard_normal(proj).astype(np.float32) for _ in range(3)]
        ins += [rng.standard_normal(proj).astype(np.float32), rng.standard_normal(heads).astype(np.float32),
                rng.standard_normal(proj).astype(np.float32)]
        want = ref.step(*ins)
        got = dev.step(*[torch.from_numpy(a).cuda() for a in ins]).cpu().numpy()
        assert np.abs(got - want).max() <= 1e-6 * max(1.0, np.abs(want).max())
        exact &= np.array_equal(bits(got), bits(want))
    s, conv = dev.export_state()
    assert np.abs(s - ref.s).max() <= 1e-6 * max(1.0, np.abs(ref.s).max())
    for i in range(3):
        assert np.array_equal(bits(conv[i]), bits(ref.conv[i]))       # raw inputs, moved only
    print(f"kda {heads}x{dim}: bit-identical over 8 tokens: {exact}")
    dev.free()


@pytest.mark.parametrize("heads,dim,kconv", [(4, 128, 4), (2, 64, 4), (3, 40, 4), (2, 128, 2)])
def test_kda_several_positions_in_one_launch_equal_single_steps(mk, heads, dim, kconv):
    """The engine's kda_prefill loop (src/model.rs:1281-1300) as one launch: outputs and final state equal n single-step
    launches bit for bit, from strided rows as the stacked projections leave them."""
    import torch
    rng = np.random.default_rng(7 * heads + dim + kconv)
    cw, a_log, dt_bias, o_norm = _kda_params(rng, heads, dim, kconv)
    proj, n = heads * dim, 9
    ld = 4 * proj + heads + 5                       # q, k, v, g2, beta and a few unrelated columns
    rows = torch.from_numpy(rng.standard_normal((n, ld)).astype(np.float32)).cuda()
    g_low = torch.from_numpy(rng.standard_normal((n, proj)).astype(np.float32)).cuda()
    off = (0, proj, 2 * proj, 3 * proj, 4 * proj)
    one = mk.KdaLayer(heads, dim, *cw, a_log, dt_bias, o_norm, kconv=kconv, gate_lb=-5.0, rms_eps=1e-6)
    many = mk.KdaLayer(heads, dim, *cw, a_log, dt_bias, o_norm, kconv=kconv, gate_lb=-5.0, rms_eps=1e-6)
    want = []
    for t in range(n):
        r = rows[t]
        want.append(one.step(r[0:proj].contiguous(), r[proj:2 * proj].contiguous(), r[2 * proj:3 * proj].contiguous(), g_low[t].contiguous(),
                             r[4 * proj:4 * proj + heads].contiguous(), r[3 * proj:4 * proj].contiguous()).cpu().numpy())
    got = many.steps(rows, g_low, ld, off).cpu().numpy()
    assert np.array_equal(bits(got), bits(np.stack(want)))
    (s1, c1), (s2, c2) = one.export_state(), many.export_state()
    assert np.array_equal(bits(s1), bits(s2)) and np.array_equal(bits(c1), bits(c2))
    one.free()
    many.free()


def test_kda_state_snapshot_restore_and_reset(mk):
    """Cache snapshot / restore (the engine clones the layer caches before a draft batch and restores them on a
    partial accept, src/spec.rs:214, 294-299): a restored state replays the same bits; reset = a new sequence."""
    import torch
    rng = np.random.default_rng(3)
    heads, dim = 4, 128
    cw, a_log, dt_bias, o_norm = _kda_params(rng, heads, dim, 4)
    dev = mk.KdaLayer(heads, dim, *cw, a_log, dt_bias, o_norm)
    proj = heads * dim
    toks = [[torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda() for n in (proj, proj, proj, proj, heads, proj)]
            for _ in range(5)]
    first = [dev.step(*toks[t]).clone() for t in range(2)]
    snap = dev.export_state()
    tail = [dev.step(*toks[t]).clone() for t in range(2, 5)]
    dev.import_state(*snap)
    again = [dev.step(*toks[t]) for t in range(2, 5)]
    assert all(torch.equal(a, b) for a, b in zip(tail, again))
    dev.reset()
    fresh = [dev.step(*toks[t]) for t in range(2)]
    assert all(torch.equal(a, b) for a, b in zip(first, fresh))
    dev.free()


@pytest.mark.parametrize("d,b", [(512, 3), (7168, 8), (100, 1), (64, 0)])
def test_attn_res_against_oracle(mk, d, b):
    """attn_res (src/model.rs:625-669): same tolerance rule as the KDA step (one exp per row)."""
    import torch
    rng = np.random.default_rng(d + b)
    prefix = rng.standard_normal(d).astype(np.float32)
    blocks = rng.standard_normal((b, d)).astype(np.float32)
    w = (rng.standard_normal(d) * 0.1).astype(np.float32)
    want = O.attn_res(prefix, blocks, w, 1e-5)
    got = mk.attn_res(torch.from_numpy(prefix).cuda(), torch.from_numpy(blocks).cuda(), torch.from_numpy(w).cuda(), 1e-5).cpu().numpy()
    assert np.abs(got - want).max() <= 1e-6 * max(1.0, np.abs(want).max())


def test_attn_res_golden(mk):
    """The AttnRes vector of the reference's selftest (src/selftest.rs:165-180), its tolerance (1e-4 relative + 1e-6)."""
    import torch
    g = np.load(os.path.join(GOLDEN, "situ_attn_res.npz"))
    w = g["norm_w"] * g["proj_w"]
    got = mk.attn_res(torch.from_numpy(g["prefix"]).cuda(), torch.from_numpy(g["blocks"]).cuda(), torch.from_numpy(w).cuda(), 1e-5)
    assert (np.abs(got.cpu().numpy() - g["out"]) <= 1e-6 + 1e-4 * np.abs(g["out"])).all()


def test_kda_step_shared_memory_form_equals_register_form(mk):
    """kda_dim 64 / 128 run with each column of S in registers by default; the option "kda_smem" stages S in shared
    memory instead (the form every other width divisible by 4 takes).  Same operations in the same order: same bits."""
    import torch
    rng = np.random.default_rng(77)
    ctx = mk.Context.default()
    for heads, dim in ((4, 128), (2, 64)):
        cw, a_log, dt_bias, o_norm = _kda_params(rng, heads, dim, 4)
        a, b = (mk.KdaLayer(heads, dim, *cw, a_log, dt_bias, o_norm) for _ in range(2))
        proj = heads * dim
        for t in range(4):
            ins = [torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda() for n in (proj, proj, proj, proj, heads, proj)]
            ya = a.step(*ins)
            ctx.set_option("kda_smem", 1)
            try:
                yb = b.step(*ins)
            finally:
                ctx.set_option("kda_smem", 0)
            assert torch.equal(ya, yb)
        sa, ca = a.export_state()
        sb, cb = b.export_state()
        assert np.array_equal(bits(sa), bits(sb)) and np.array_equal(bits(ca), bits(cb))
        a.free(), b.free()


def test_kda_and_attn_res_argument_errors(mk):
    """Bad descriptors and pointers are refused with a status, nothing is launched."""
    import ctypes as C
    import torch
    from microkimi_b200 import lib as L
    rng = np.random.default_rng(5)
    cw, a_log, dt_bias, o_norm = _kda_params(rng, 2, 64, 4)
    big = _kda_params(rng, 1, 2048, 4)
    with pytest.raises(L.MkError):
        mk.KdaLayer(1, 2048, *big[0], *big[1:])                         # kda_dim above 1024
    one = [c[:, :1].copy() for c in cw]
    with pytest.raises(L.MkError):
        mk.KdaLayer(2, 64, *one, a_log, dt_bias, o_norm, kconv=1)       # a conv of width 1 has no window
    layer = mk.KdaLayer(2, 64, *cw, a_log, dt_bias, o_norm)
    ctx = layer.ctx
    v = torch.zeros(128, device="cuda")
    with pytest.raises(L.MkError):
        L.check(ctx._L.mk_kda_step_dev(ctx._h, layer._h, C.c_void_p(v.data_ptr()), None, None, None, None, None, C.c_void_p(v.data_ptr())))
    with pytest.raises(L.MkError):
        L.check(ctx._L.mk_attn_res_dev(ctx._h, C.c_void_p(v.data_ptr()), None, 128, 3, C.c_void_p(v.data_ptr()), 128, 1e-5,
                                       C.c_void_p(v.data_ptr())))      # 3 blocks announced, no block rows given
    assert ctx.status_word() == 0
    layer.free()
