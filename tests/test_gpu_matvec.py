"""GPU parity tests for the dequant-fused matvecs, through the C ABI, against the
CPU oracle on the same seeded inputs.

Tolerances (the reference's vocabulary, src/parity.rs:12-14, selftest.rs:601-646):
  dequantized values, quantized bytes, scales ........ bit-exact
  MK_ACT_STRICT outputs vs the CPU q8 path ........... bit-exact
  default outputs vs the CPU q8 path ................. 1e-5 * max|ref| (f32 summation order only)
  default outputs vs the CPU exact-f32 path .......... 1e-3 * max|ref| on the reference's own test
                                                       pattern (selftest.rs:601-646).  On N(0,1) activations
                                                       the reference's q8 path itself sits ~6e-3 from its
                                                       f32 path (measured below on the CPU oracle), so there
                                                       the 1e-3 bound is held by MK_ACT_Q8X2 instead.
  MK_ACT_Q8X2 outputs vs the CPU exact-f32 path ...... 1e-4 * max|ref| (asserted; the spec asks 1e-3)
"""
import os

import numpy as np
import pytest

from conftest import GOLDEN, bits, pattern, pattern_matrix
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mk():
    import microkimi_b200 as m
    m.Context.default()
    return m


def rel(a, ref):
    return np.abs(a.astype(np.float64) - ref.astype(np.float64)).max() / max(np.abs(ref).max(), 1e-12)


# ------------------------------------------------------------------ dequant / registration
def test_dequant_golden_fp4_block(mk):
    g = np.load(os.path.join(GOLDEN, "ds_fp4.npz"))
    rows, cols = int(g["rows"]), int(g["cols"])
    w = mk.MxFp4Weight(g["packed"], g["scales"], rows, cols)
    assert np.array_equal(bits(w.dequant()), bits(g["dequant"].reshape(rows, cols)))


def test_dequant_reference_numpy_fixture(mk):
    g = np.load(os.path.join(GOLDEN, "mxfp4_numpy_dequant.npz"))
    rows, cols = g["packed"].shape[0], g["packed"].shape[1] * 2
    w = mk.MxFp4Weight(g["packed"], g["scales"], rows, cols)
    assert np.array_equal(bits(w.dequant()), bits(g["dequant"]))


@pytest.mark.parametrize("rows,cols", [(1, 32), (3, 64), (17, 96), (64, 128), (333, 1024), (2048, 512)])
def test_dequant_and_export_random_blobs_bit_exact(mk, rows, cols):
    rng = np.random.default_rng(rows * 131 + cols)
    packed = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(0, 255, (rows, cols // 32), dtype=np.uint8)
    scales.flat[0] = 0
    scales.flat[-1] = 254
    w = mk.MxFp4Weight(packed, scales, rows, cols)
    assert np.array_equal(bits(w.dequant()), bits(O.mxfp4_dequant(packed, scales, rows, cols)))
    p2, s2 = w.export()
    assert np.array_equal(p2, packed) and np.array_equal(s2, scales)


def test_quantize_q8_bit_exact(mk):
    rng = np.random.default_rng(11)
    x = rng.standard_normal(7168).astype(np.float32)
    x[32:64] = 0.0
    x[100] = 1e-30
    x[64:96] *= 1e-20
    q, s = mk.quantize_q8(x)
    q0, s0 = O.q8_quantize(x)
    assert np.array_equal(q, q0) and np.array_equal(bits(s), bits(s0))
    x = np.zeros(64, np.float32)
    x[3], x[40] = 12.7, -3.3                     # src/q8.rs:320-334
    q, s = mk.quantize_q8(x)
    assert s[0] == np.float32(12.7) / np.float32(127.0) and q[3] == 127 and q.min() >= -127


# ------------------------------------------------------------------ MXFP4 matvec
SHAPES = [(128, 512), (512, 128), (64, 128), (3, 64), (1, 32), (256, 1024), (2048, 4096), (4096, 2048), (333, 1024),
          (40, 96)]


def _case(rows, cols, zero_rows=None):
    w = pattern_matrix(rows, cols)
    if zero_rows:
        w[zero_rows[0]:zero_rows[1]] = 0.0
    p, s = O.mxfp4_quantize(w)
    x = pattern(np.arange(cols, dtype=np.uint64) + np.uint64(4242))
    return p, s, x


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_mxfp4_matvec_against_oracle(mk, rows, cols):
    """The shapes of selftest.rs:534-646 (PACKED-EMUL / Q8-EMUL) plus ragged ones."""
    p, s, x = _case(rows, cols)
    w = mk.MxFp4Weight(p, s, rows, cols)
    ref_q8 = O.mxfp4_matvec(p, s, x, use_q8=True)
    ref_f32 = O.mxfp4_matvec(p, s, x, use_q8=False)
    y_strict = w.matvec(x, strict=True)
    assert np.array_equal(bits(y_strict), bits(ref_q8))
    y = w.matvec(x)
    assert rel(y, ref_q8) <= 1e-5
    assert rel(y, ref_f32) <= 1e-3
    y2 = w.matvec(x, act="q8x2")
    assert rel(y2, ref_f32) <= 1e-4


def test_mxfp4_matvec_zero_block_and_subnormal_scale(mk):
    p, s, x = _case(64, 128, zero_rows=(2, 4))
    assert (s[2:4] == 0).all()
    w = mk.MxFp4Weight(p, s, 64, 128)
    ref = O.mxfp4_matvec(p, s, x, use_q8=True)
    assert np.array_equal(bits(w.matvec(x, strict=True)), bits(ref))
    assert (w.matvec(x)[2:4] == 0).all()
    # scale bytes 1 and 2 (2^-127 is subnormal once halved) with non-zero codes
    s[5, :] = 1
    s[6, :] = 2
    w = mk.MxFp4Weight(p, s, 64, 128)
    xb = (x * np.float32(1e30)).astype(np.float32)
    ref = O.mxfp4_matvec(p, s, xb, use_q8=True)
    assert np.array_equal(bits(w.matvec(xb, strict=True)), bits(ref))


@pytest.mark.parametrize("batch", [2, 3, 8, 9, 17])
def test_mxfp4_matvec_batched_equals_single_token(mk, batch):
    """model.rs:2398-2411: a batch is bit-identical, per position, to single-token calls."""
    rng = np.random.default_rng(batch)
    rows, cols = 272, 512
    wf = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    p, s = O.mxfp4_quantize(wf)
    xs = rng.standard_normal((batch, cols)).astype(np.float32)
    w = mk.MxFp4Weight(p, s, rows, cols)
    ys = w.matvec(xs, strict=True)
    yd = w.matvec(xs)
    for t in range(batch):
        ref = O.mxfp4_matvec(p, s, xs[t], use_q8=True)
        assert np.array_equal(bits(ys[t]), bits(ref))
        assert rel(yd[t], ref) <= 1e-5
        assert np.array_equal(bits(yd[t]), bits(w.matvec(xs[t]))), "a batch must equal single-token calls bit for bit"
    y2 = w.matvec(xs, act="q8x2")
    for t in range(batch):
        assert rel(y2[t], O.mxfp4_matvec(p, s, xs[t], use_q8=False)) <= 1e-4
        assert np.array_equal(bits(y2[t]), bits(w.matvec(xs[t], act="q8x2")))


def test_mxfp4_expert_down_projection_full_size(mk):
    """One MoE expert down-projection: W 7168x2048 from N(0, 0.02) through the
    reference quantizer, x ~ N(0, 1), batch 1, one fixed seed."""
    rng = np.random.default_rng(20250101)
    rows, cols = 7168, 2048
    wf = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    p, s = O.mxfp4_quantize(wf)
    x = rng.standard_normal(cols).astype(np.float32)
    w = mk.MxFp4Weight(p, s, rows, cols)
    assert np.array_equal(bits(w.dequant()), bits(O.mxfp4_dequant(p, s, rows, cols)))
    ref_q8 = O.mxfp4_matvec(p, s, x, use_q8=True, n_threads=8)
    ref_f32 = O.mxfp4_matvec(p, s, x, use_q8=False, n_threads=8)
    assert np.array_equal(bits(w.matvec(x, strict=True)), bits(ref_q8))
    y = w.matvec(x)
    assert rel(y, ref_q8) <= 1e-5
    # Gaussian activations: the reference's own q8 path is a few 1e-3 away from its f32 path
    assert 1e-3 < rel(ref_q8, ref_f32) < 2e-2 and rel(y, ref_f32) < 2e-2
    assert rel(w.matvec(x, act="q8x2"), ref_f32) <= 1e-4
    assert int(np.argmax(w.matvec(x, act="q8x2"))) == int(np.argmax(ref_f32))
    # the drop-in call with borrowed slices gives the same bits
    assert np.array_equal(bits(mk.matvec_packed(p, s, rows, cols, x)), bits(y))


def test_mxfp4_matvec_linearity_property(mk):
    """Size-independent property: integer activations with block maximum 127 survive
    q8_0 exactly (dx = 1), so the result must equal the dense f64 product."""
    rng = np.random.default_rng(5)
    rows, cols = 1024, 2048
    p = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
    s = rng.integers(118, 124, (rows, cols // 32), dtype=np.uint8)
    a = rng.integers(-31, 32, cols).astype(np.float32)
    b = rng.integers(-31, 32, cols).astype(np.float32)
    a[::32], b[::32] = 127, -127   # block max 127 -> dx = 1 exactly, integers survive q8
    w = mk.MxFp4Weight(p, s, rows, cols)
    ya, yb = w.matvec(a), w.matvec(b)
    dense = O.mxfp4_dequant(p, s, rows, cols).astype(np.float64)
    assert rel(ya, (dense @ a).astype(np.float32)) <= 1e-5
    assert rel(yb, (dense @ b).astype(np.float32)) <= 1e-5


# ------------------------------------------------------------------ q8_0 lm_head
@pytest.mark.parametrize("rows,cols,scale", [(512, 256, "f32"), (333, 96, "f32"), (16, 32, "f32"), (4096, 7168, "f32"),
                                             (512, 256, "f16"), (333, 96, "f16")])
def test_q8_head_from_f32_and_matvec(mk, rows, cols, scale):
    """model.rs:3866-3881 plus bit-level checks of the stored bytes."""
    rng = np.random.default_rng(rows + cols)
    wf = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    wf[1, :32] = 0.0
    x = rng.standard_normal(cols).astype(np.float32)
    head = mk.Q8Head.from_f32(wf, rows, cols, scale=scale)
    q, s = head.export()
    if scale == "f32":
        q0, s0 = O.q8head_from_f32(wf)
        assert np.array_equal(q, q0) and np.array_equal(bits(s), bits(s0))
        ref = O.q8head_matvec(q0, s0, x, n_threads=8)
    else:
        q0, s0 = O.q8head_from_f32_f16s(wf)
        assert np.array_equal(q, q0) and np.array_equal(s.view(np.uint16), s0)
        ref = O.q8head_matvec_f16s(q0, s0, x, n_threads=8)
    y_strict, am = head.matvec(x, strict=True, want_argmax=True)
    assert np.array_equal(bits(y_strict), bits(ref))
    assert int(am[0]) == O.argmax(ref)
    y, am = head.matvec(x, want_argmax=True)
    assert rel(y, ref) <= 1e-5
    f32 = O.matvec_f32(wf, x, n_threads=8)
    assert np.abs(y - f32).max() / (f32.max() - f32.min()) < 1e-2     # model.rs:3878
    assert int(am[0]) == int(np.argmax(y))
    if rows >= 512:
        assert int(am[0]) == O.argmax(f32)
    y2 = head.matvec(x, act="q8x2")
    wdq = q0.astype(np.float64).reshape(rows, -1, 32) * (s0.view(np.float16) if scale == "f16" else s0).astype(np.float64)[:, :, None]
    assert rel(y2, (wdq.reshape(rows, cols) @ x.astype(np.float64)).astype(np.float32)) <= 1e-4


@pytest.mark.parametrize("batch", [2, 8, 11])
def test_q8_head_batched(mk, batch):
    rng = np.random.default_rng(77 + batch)
    rows, cols = 1000, 512
    wf = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    xs = rng.standard_normal((batch, cols)).astype(np.float32)
    head = mk.Q8Head.from_f32(wf, rows, cols)
    q0, s0 = O.q8head_from_f32(wf)
    ys, am = head.matvec(xs, strict=True, want_argmax=True)
    yd = head.matvec(xs)
    for t in range(batch):
        ref = O.q8head_matvec(q0, s0, xs[t])
        assert np.array_equal(bits(ys[t]), bits(ref))
        assert int(am[t]) == O.argmax(ref)
        assert rel(yd[t], ref) <= 1e-5
    # caller-owned result buffers (the engine's `out: &mut [f32]`), here views of pinned memory
    import torch
    yp, ap = torch.empty((batch, rows), dtype=torch.float32).pin_memory(), torch.empty(batch, dtype=torch.int32).pin_memory()
    y2, am2 = head.matvec(xs, strict=True, want_argmax=True, out=yp.numpy(), argmax_out=ap.numpy())
    assert np.array_equal(bits(yp.numpy()), bits(ys)) and np.array_equal(ap.numpy(), am)
    assert np.shares_memory(y2, yp.numpy())


def test_q8_head_prequantized_rows_and_argmax_ties(mk):
    rng = np.random.default_rng(3)
    rows, cols = 64, 64
    q = rng.integers(-127, 128, (rows, cols)).astype(np.int8)
    s = np.full((rows, 2), 0.01, np.float32)
    q[40] = q[7]                      # identical rows -> identical logits: the lower index wins
    q[7] = q[40] = 127
    head = mk.Q8Head.from_q8(q, s, rows, cols)
    x = np.ones(cols, np.float32)
    y, am = head.matvec(x, strict=True, want_argmax=True)
    assert y[7] == y[40] == y.max() and int(am[0]) == 7
    q2, s2 = head.export()
    assert np.array_equal(q2, q) and np.array_equal(s2, s)


def test_device_pointer_entry_points(mk):
    import torch
    rng = np.random.default_rng(9)
    rows, cols = 512, 1024
    wf = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    p, s = O.mxfp4_quantize(wf)
    x = rng.standard_normal((3, cols)).astype(np.float32)
    ctx = mk.Context.default()
    ctx.use_torch_stream()
    w = mk.MxFp4Weight(p, s, rows, cols)
    xd = torch.from_numpy(x).cuda()
    yd = w.matvec(xd)
    torch.cuda.synchronize()
    assert np.array_equal(bits(yd.cpu().numpy()), bits(w.matvec(x)))
    head = mk.Q8Head.from_f32(torch.from_numpy(wf).cuda(), rows, cols)
    y, am = head.matvec(xd, want_argmax=True)
    torch.cuda.synchronize()
    y_host, am_host = mk.Q8Head.from_f32(wf, rows, cols).matvec(x, want_argmax=True)
    assert np.array_equal(bits(y.cpu().numpy()), bits(y_host)) and np.array_equal(am.cpu().numpy(), am_host)


def test_argument_errors_are_statuses_not_crashes(mk):
    with pytest.raises(AssertionError):
        mk.MxFp4Weight(np.zeros(10, np.uint8), np.zeros(1, np.uint8), 4, 32)
    import ctypes as C
    L, ctx = mk.lib.load(), mk.Context.default()
    h = C.c_void_p()
    rc = L.mk_weight_mxfp4(ctx._h, None, None, 4, 32, 0, C.byref(h))
    assert rc == -1 and b"NULL" in L.mk_last_error()
    z = np.zeros(64, np.uint8)
    rc = L.mk_weight_mxfp4(ctx._h, z.ctypes.data_as(C.c_void_p), z.ctypes.data_as(C.c_void_p), 4, 33, 0, C.byref(h))
    assert rc == -1
    w = mk.MxFp4Weight(np.zeros((4, 16), np.uint8), np.zeros((4, 1), np.uint8), 4, 32)
    x = np.zeros(32, np.float32)
    rc = L.mk_matvec_q8(ctx._h, w._h, x.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p), 1, 0, None)
    assert rc == -1 and b"format" in L.mk_last_error()
    assert ctx.status_word() == 0


def test_fp8_dequant_bit_exact(mk):
    """dequant::dequant_fp8 against the torch-generated block of ref/ds_golden.json and, for every byte
    value and extreme scale bytes, against the oracle (NaN encodings, -0.0, subnormal scales)."""
    g = np.load(os.path.join(GOLDEN, "ds_fp8.npz"))
    rows, cols = int(g["rows"]), int(g["cols"])
    out = mk.dequant_fp8(g["w_packed"], g["scales"], rows, cols)
    assert np.array_equal(bits(out), bits(g["dequant"].reshape(rows, cols)))
    rng = np.random.default_rng(8)
    w = rng.integers(0, 256, (200, 300), dtype=np.uint8)
    w[0, :256] = np.arange(256)
    s = rng.integers(0, 255, (2, 3), dtype=np.uint8)
    s[0, 0], s[1, 2] = 0, 254
    got, ref = mk.dequant_fp8(w, s, 200, 300), O.dequant_fp8(w, s, 200, 300)
    nan = np.isnan(ref)
    assert np.array_equal(nan, np.isnan(got))
    assert np.array_equal(bits(got)[~nan], bits(ref)[~nan])


def test_device_calls_replay_from_a_cuda_graph(mk):
    """Device-pointer calls launch on the caller's stream and neither allocate nor synchronize once warm, so a
    decode loop can capture them in a CUDA graph: the replay on new inputs gives the bits of the direct call."""
    import torch
    rng = np.random.default_rng(31)
    rows, cols = 768, 1024
    wf = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    p, s = O.mxfp4_quantize(wf)
    ctx = mk.Context.default()
    w = mk.MxFp4Weight(p, s, rows, cols)
    head = mk.Q8Head.from_f32(wf, rows, cols)
    f32w = mk.F32Weight(wf, rows, cols)
    x = torch.from_numpy(rng.standard_normal((1, cols)).astype(np.float32)).cuda()
    for _ in range(2):                      # warm: workspaces grow here, not under capture
        w.matvec(x), head.matvec(x, want_argmax=True), f32w.matvec(x)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y1 = w.matvec(x)
        y2, am = head.matvec(x, want_argmax=True)
        y3 = f32w.matvec(x)
    x2 = torch.from_numpy(rng.standard_normal((1, cols)).astype(np.float32)).cuda()
    x.copy_(x2)
    g.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in (y1, y2, am, y3)]
    want = [w.matvec(x2), *head.matvec(x2, want_argmax=True), f32w.matvec(x2)]
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    assert ctx.status_word() == 0


def test_dequant_any_both_mxfp4_flavours(mk):
    """mxfp4::dequant_any (src/mxfp4.rs:228-240): raw blobs as a model file holds them, bit-exact on the GPU."""
    rng = np.random.default_rng(31)
    rows, cols = 40, 256
    w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
    w[2, 32:64] = 0.0
    p, s = O.mxfp4_quantize(w)
    blob = np.concatenate([p.ravel(), s.ravel()])
    assert np.array_equal(bits(mk.dequant_any("mxfp4", blob, rows, cols)), bits(O.mxfp4_dequant(p, s, rows, cols)))
    p2, s2, smax = O.mxfp4sq_quantize(w)
    blob2 = np.concatenate([p2.ravel(), s2.ravel(), np.array([smax], np.float32).view(np.uint8)])
    assert np.array_equal(bits(mk.dequant_any("mxfp4sq", blob2, rows, cols)), bits(O.mxfp4sq_dequant(p2, s2, smax, rows, cols)))
    with pytest.raises(AssertionError):
        mk.dequant_any("mxfp4sq", blob, rows, cols)          # the trailing smax is missing
