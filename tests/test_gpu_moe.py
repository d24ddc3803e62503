"""GPU parity tests of the MoE layer (router, top-k, grouped MXFP4 experts, combine)
through the C ABI against the CPU oracle.

  router logits ................ bit-exact (same dot() order as src/model.rs:63-82)
  selected expert ids .......... identical, in slot order (src/parity.rs:215-241 asks for exact ids)
  routing weights .............. 1e-6 relative (one exp() per score; last-ulp freedom)
  layer output ................. 1e-3 * max|ref| against the CPU q8 path (the spec's bound).  The gap is
                                 not smooth: gate/up sums differ from the CPU in the last bit (f32
                                 summation order), which now and then flips the q8 rounding of one
                                 activation element by one step; one flip moves the w2 output by
                                 ~5e-4 of its maximum at d=7168, inter=2048 (measured), 0 otherwise.
"""
import numpy as np
import pytest

from conftest import bits
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mk():
    import microkimi_b200 as m
    m.Context.default()
    return m


def make_layer(mk, n_experts, top_k, d, inter, seed, bias_scale=0.0):
    rng = np.random.default_rng(seed)
    gate_w = (rng.standard_normal((n_experts, d)) * 0.02).astype(np.float32)
    gate_b = (rng.standard_normal(n_experts) * bias_scale).astype(np.float32)
    host, dev = [], []
    for e in range(n_experts + 1):
        tri_h, tri_d = [], []
        for rows, cols in ((inter, d), (d, inter), (inter, d)):
            p, s = O.mxfp4_quantize((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
            tri_h.append((p, s))
            tri_d.append(mk.MxFp4Weight(p, s, rows, cols))
        host.append(tri_h)
        dev.append(tuple(tri_d))
    ref = O.MoeDs(gate_w, gate_b, host[:-1], host[-1], top_k)
    layer = mk.MoeLayer(gate_w, gate_b, dev[:-1], dev[-1], top_k)
    return layer, ref, rng


def rel(a, ref):
    return np.abs(a.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-12)


@pytest.mark.parametrize("n_experts,top_k,d,inter,batches", [
    (16, 4, 256, 128, (1, 2, 3, 16, 40)),
    (40, 8, 512, 64, (1, 7)),
    (8, 2, 7168, 2048, (1, 5)),
])
def test_moe_forward_against_oracle(mk, n_experts, top_k, d, inter, batches):
    layer, ref, rng = make_layer(mk, n_experts, top_k, d, inter, seed=n_experts * 7 + d)
    for b in batches:
        x = rng.standard_normal((b, d)).astype(np.float32)
        out, ids, w = layer.moe_forward(x, want_routing=True)
        ids_r, w_r, lg = layer.route(x, want_logits=True)
        assert np.array_equal(ids, ids_r) and np.array_equal(bits(w), bits(w_r))
        for t in range(b):
            o_ref, ids_ref, w_ref = ref.forward(x[t], use_q8=True, n_threads=8)
            _, _, lg_ref = O.router_k3(ref.gate_w, ref.gate_b, x[t], top_k)
            assert np.array_equal(bits(lg[t]), bits(lg_ref)), "router logits must be bit-exact"
            assert np.array_equal(ids[t], ids_ref), "expert ids must match in slot order"
            assert np.abs(w[t] - w_ref).max() <= 1e-6 * np.abs(w_ref).max()
            assert rel(out[t], o_ref) <= 1e-3
        # a batch is, per token, what single-token calls give (src/model.rs:2449-2456)
        single = np.stack([layer.moe_forward(x[t]) for t in range(b)])
        assert np.array_equal(bits(single), bits(out))


def test_router_bias_and_ties(mk):
    """Bias enters the selection only; equal keys resolve to the lower expert id."""
    layer, ref, rng = make_layer(mk, 12, 3, 64, 32, seed=5, bias_scale=0.2)
    x = rng.standard_normal((6, 64)).astype(np.float32)
    ids, w = layer.route(x)
    for t in range(6):
        ids_ref, w_ref, _ = O.router_k3(ref.gate_w, ref.gate_b, x[t], 3)
        assert np.array_equal(ids[t], ids_ref)
        assert abs(float(w[t].sum()) - 1.0) < 1e-5
    gw = np.zeros((12, 64), np.float32)      # all logits 0 -> all keys equal -> ids 0, 1, 2
    tie = mk.MoeLayer(gw, None, layer._keep[0], layer._keep[1], 3)
    ids, w = tie.route(x[:1])
    assert ids[0].tolist() == [0, 1, 2]


def test_explicit_pairs_and_missing_experts(mk):
    """The expert-parallel primitive: explicit (row, expert, weight) pairs; pairs that name an
    expert that is not resident are reported through the status word, not computed."""
    import torch
    layer, ref, rng = make_layer(mk, 6, 2, 128, 64, seed=11)
    ctx = mk.Context.default()
    x = rng.standard_normal((3, 128)).astype(np.float32)
    pr = np.array([0, 0, 1, 2, 2, 2, 1], np.int32)
    pe = np.array([3, 6, 0, 3, 5, 6, 2], np.int32)       # 6 = the shared expert
    pw = np.array([0.25, 1.0, 0.5, 0.75, 0.1, 1.0, 0.3], np.float32)
    ctx.use_torch_stream()
    outs = layer.experts_dev(torch.from_numpy(x).cuda(), torch.from_numpy(pr).cuda(), torch.from_numpy(pe).cuda(),
                             torch.from_numpy(pw).cuda())
    torch.cuda.synchronize()
    outs = outs.cpu().numpy()
    lib = O.lib()
    for p in range(len(pr)):
        # one expert through the oracle: a 1-expert layer with the weight forced via top_k = 1 is awkward,
        # so restate the three matvecs (src/deepseek.rs:1078-1090) with the oracle's pieces
        tri = ref._sh if pe[p] == 6 else None
        if tri is None:
            e = int(pe[p])
            tri = [(ref._keep[6 * e + 2 * j], ref._keep[6 * e + 2 * j + 1]) for j in range(3)]
        g = O.mxfp4_matvec(tri[0][0], tri[0][1], x[pr[p]], use_q8=True)
        u = O.mxfp4_matvec(tri[2][0], tri[2][1], x[pr[p]], use_q8=True)
        gl, ul = np.minimum(g, np.float32(10.0)), np.clip(u, -10.0, 10.0).astype(np.float32)
        silu = (gl / (np.float32(1.0) + np.exp(-gl).astype(np.float32))).astype(np.float32)
        act = ((pw[p] * silu).astype(np.float32) * ul).astype(np.float32)
        o = O.mxfp4_matvec(tri[1][0], tri[1][1], act, use_q8=True)
        assert rel(outs[p], o) <= 1e-3
    assert ctx.status_word() == 0
    # an expert that is not resident
    experts = list(layer._keep[0])
    experts[4] = None
    part = mk.MoeLayer(ref.gate_w, ref.gate_b, experts, layer._keep[1], 2)
    pe2 = np.array([4, 1], np.int32)
    part.experts_dev(torch.from_numpy(x).cuda(), torch.tensor([0, 1], dtype=torch.int32).cuda(),
                     torch.from_numpy(pe2).cuda(), torch.tensor([1.0, 1.0]).cuda())
    torch.cuda.synchronize()
    assert ctx.status_word() == -1


# ------------------------------------------------------------------ DeepSeek router (sqrt-softplus)
def _dummy_experts(mk, n_experts, d, inter):
    z = lambda r, c: mk.MxFp4Weight(np.zeros((r, c // 2), np.uint8), np.zeros((r, c // 32), np.uint8), r, c)
    return [(z(inter, d), z(d, inter), z(inter, d)) for _ in range(n_experts)]


def test_ds_router_matches_golden_gate(mk):
    """gate_forward (src/deepseek.rs:16-58) on the reference's own vector: the 'gate' section of
    ref/ds_golden2.json (3 tokens x 32 experts, top-6, route_scale 1.5), which the reference checks
    in src/selftest.rs:259-311 with sorted ids and a 1e-3 weight tolerance."""
    import os
    from conftest import GOLDEN
    g = np.load(os.path.join(GOLDEN, "ds_gate_expert.npz"))
    gw, gb, x = g["gate_w"], g["gate_bias"], g["gate_x"]
    d = gw.shape[1]
    # the router works on rows of any multiple of 32; the golden d is 16, so pad rows with zeros
    # (zero columns add exact zeros to every accumulator: same logits)
    dp = 32
    gwp = np.zeros((32, dp), np.float32); gwp[:, :d] = gw
    xp = np.zeros((3, dp), np.float32); xp[:, :d] = x
    layer = mk.MoeLayer(gwp, gb, _dummy_experts(mk, 32, dp, 32), None, 6, router="sqrt_softplus", route_scale=1.5)
    ids, w = layer.route(xp)
    scale = np.abs(g["gate_weights"]).max()
    for t in range(3):
        assert sorted(ids[t].tolist()) == sorted(g["gate_indices"][t].tolist())
        want = dict(zip(g["gate_indices"][t].tolist(), g["gate_weights"][t].tolist()))
        for i, wi in zip(ids[t].tolist(), w[t].tolist()):
            assert abs(wi - want[i]) <= 1e-5 + 1e-3 * scale
        ids_o, w_o = O.gate_ds(gw, gb, x[t], 6, 1.5)
        assert np.array_equal(ids[t], ids_o), "slot order must match the CPU's"
        assert np.abs(w[t] - w_o).max() <= 1e-6 * np.abs(w_o).max()


@pytest.mark.parametrize("n_experts,top_k,d,batch", [(64, 6, 256, 5), (896, 16, 512, 19)])
def test_ds_router_against_oracle(mk, n_experts, top_k, d, batch):
    rng = np.random.default_rng(n_experts + d)
    gw = (rng.standard_normal((n_experts, d)) * 0.3).astype(np.float32)   # logits on both sides of the softplus knee
    gb = (rng.standard_normal(n_experts) * 0.1).astype(np.float32)
    x = rng.standard_normal((batch, d)).astype(np.float32)
    x[0] *= 8.0                                                             # some logits above the threshold of 20
    layer = mk.MoeLayer(gw, gb, _dummy_experts(mk, n_experts, d, 32), None, top_k, router="sqrt_softplus", route_scale=2.5)
    ids, w = layer.route(x)
    for t in range(batch):
        ids_o, w_o = O.gate_ds(gw, gb, x[t], top_k, 2.5)
        assert np.array_equal(ids[t], ids_o)
        assert np.abs(w[t] - w_o).max() <= 2e-6 * np.abs(w_o).max()


# ------------------------------------------------------------------ K3 latent MoE (SiTU)
def make_k3_layer(mk, n_experts, top_k, d, rh, inter, si, seed):
    rng = np.random.default_rng(seed)
    g = lambda *shape, s=0.02: (rng.standard_normal(shape) * s).astype(np.float32)
    gate_w, gate_b = g(n_experts, d), g(n_experts, s=0.05)
    routed_down, routed_up = g(rh, d, s=0.05), g(d, rh, s=0.05)
    routed_norm = (1.0 + 0.1 * rng.standard_normal(rh)).astype(np.float32)
    shared = (g(si, d, s=0.05), g(si, d, s=0.05), g(d, si, s=0.05))     # gate, up, down
    host, dev = [], []
    for e in range(n_experts):
        tri_h, tri_d = [], []
        for rows, cols in ((inter, rh), (rh, inter), (inter, rh)):
            p, s = O.mxfp4_quantize(g(rows, cols, s=0.2))
            tri_h.append((p, s))
            tri_d.append(mk.MxFp4Weight(p, s, rows, cols))
        host.append(tri_h)
        dev.append(tuple(tri_d))
    ref = O.MoeK3(gate_w, gate_b, routed_down, routed_norm, routed_up, host, shared, top_k, rms_eps=1e-6)
    layer = mk.MoeLayer(gate_w, gate_b, dev, None, top_k, activation="situ",
                        routed_down=mk.F32Weight(routed_down, rh, d), routed_up=mk.F32Weight(routed_up, d, rh),
                        routed_norm=routed_norm, rms_eps=1e-6,
                        shared_f32=(mk.F32Weight(shared[0], si, d), mk.F32Weight(shared[2], d, si), mk.F32Weight(shared[1], si, d)))
    return layer, ref, rng


@pytest.mark.parametrize("n_experts,top_k,d,rh,inter,si,batches", [
    (896, 16, 512, 128, 64, 128, (1, 2, 5, 20)),     # the engine's micro configuration (src/config.rs:47-79)
    (24, 4, 256, 64, 32, 96, (1, 3)),
])
def test_k3_latent_moe_against_oracle(mk, n_experts, top_k, d, rh, inter, si, batches):
    """moe_forward of the K3 engine (src/model.rs:2150-2380): ids exact, output within 1e-3 * max
    of the CPU q8 path (the f32 projections are bit-exact; the MXFP4 expert sums differ from the
    CPU in summation order only, and SiTU's tanh/exp are correctly rounded here)."""
    layer, ref, rng = make_k3_layer(mk, n_experts, top_k, d, rh, inter, si, seed=n_experts + d)
    for b in batches:
        x = rng.standard_normal((b, d)).astype(np.float32)
        out, ids, w = layer.moe_forward(x, want_routing=True)
        for t in range(b):
            o_ref, ids_ref, w_ref = ref.forward(x[t], use_q8=True)
            assert np.array_equal(ids[t], ids_ref)
            assert np.abs(w[t] - w_ref).max() <= 1e-6 * np.abs(w_ref).max()
            assert rel(out[t], o_ref) <= 1e-3
        single = np.stack([layer.moe_forward(x[t]) for t in range(b)])
        assert np.array_equal(bits(single), bits(out))


def test_situ_without_latent_and_bad_descriptors(mk):
    """MK_MOE_SITU on the model width (no latent projections): weights multiply the expert outputs."""
    from microkimi_b200 import lib as L
    rng = np.random.default_rng(3)
    E, k, d, inter = 8, 2, 128, 64
    gate_w = (rng.standard_normal((E, d)) * 0.02).astype(np.float32)
    host, dev = [], []
    for e in range(E):
        tri_h, tri_d = [], []
        for rows, cols in ((inter, d), (d, inter), (inter, d)):
            p, s = O.mxfp4_quantize((rng.standard_normal((rows, cols)) * 0.2).astype(np.float32))
            tri_h.append((p, s)); tri_d.append(mk.MxFp4Weight(p, s, rows, cols))
        host.append(tri_h); dev.append(tuple(tri_d))
    layer = mk.MoeLayer(gate_w, None, dev, None, k, activation="situ")
    x = rng.standard_normal((3, d)).astype(np.float32)
    out, ids, w = layer.moe_forward(x, want_routing=True)
    for t in range(3):
        y = np.zeros(d, np.float32)
        for slot in range(k):
            tri = host[ids[t, slot]]
            a = O.mxfp4_matvec(tri[0][0], tri[0][1], x[t], use_q8=True)
            u = O.mxfp4_matvec(tri[2][0], tri[2][1], x[t], use_q8=True)
            act = np.array([O.lib().or_situ(float(a[j]), float(u[j])) for j in range(inter)], np.float32)
            o = O.mxfp4_matvec(tri[1][0], tri[1][1], act, use_q8=True)
            y = (y + (w[t, slot] * o).astype(np.float32)).astype(np.float32)
        assert rel(out[t], y) <= 1e-3
    # the K3 body takes its shared expert as f32 matrices: an MXFP4 shared triple is refused
    with pytest.raises(L.MkError):
        mk.MoeLayer(gate_w, None, dev, dev[0], k, activation="situ")


def test_expert_parallel_entry_point_with_one_rank(mk):
    """mk_moe_forward_ep_dev with world = 1: the same grouping rule, exchange kernel (no peer to push to,
    its own flag to wait for) and table combine as on several GPUs; results equal mk_moe_forward_dev bit for bit."""
    import ctypes as C
    import torch
    from microkimi_b200 import lib as L
    layer, ref, rng = make_layer(mk, 16, 4, 256, 128, seed=123)
    ctx = mk.Context.default()
    ctx.use_torch_stream()
    ep, handle = C.c_void_p(), (C.c_uint8 * 64)()
    L.check(ctx._L.mk_moe_ep_create(ctx._h, layer._h, 0, 1, 16, C.byref(ep), handle))
    try:
        for n in (1, 2, 7, 16, 3):
            x = torch.from_numpy(rng.standard_normal((n, 256)).astype(np.float32)).cuda()
            want = layer.moe_forward(x)
            got = torch.empty_like(x)
            L.check(ctx._L.mk_moe_forward_ep_dev(ctx._h, layer._h, ep, C.c_void_p(x.data_ptr()), n, C.c_void_p(got.data_ptr()), None, None))
            torch.cuda.synchronize()
            assert torch.equal(got, want)
        with pytest.raises(L.MkError):   # more rows than the exchange table holds
            x = torch.zeros((17, 256), device="cuda")
            L.check(ctx._L.mk_moe_forward_ep_dev(ctx._h, layer._h, ep, C.c_void_p(x.data_ptr()), 17, C.c_void_p(x.data_ptr()), None, None))
        assert ctx.status_word() == 0
    finally:
        L.check(ctx._L.mk_moe_ep_free(ctx._h, ep))


# ------------------------------------------------------------------ block-scaled tensor-core path (act="fp4x6")
@pytest.mark.parametrize("n_experts,top_k,d,inter,batch", [(16, 4, 256, 256, 40), (12, 3, 512, 768, 97), (6, 2, 1024, 256, 33), (8, 2, 512, 256, 7)])
def test_block_scaled_tensor_core_experts_track_the_exact_f32_path(mk, n_experts, top_k, d, inter, batch):
    """Calls of >= 4 rows with act="fp4x6" run the experts as tcgen05 block-scaled products: E2M1 weights and their ue8m0
    scales as registered, activations as six E2M1 limbs.  Held to the engine's exact-f32 path (MICROKIMI_NO_Q8,
    src/mxfp4.rs:488-539) at 1e-3 of max |ref| (the bound of src/parity.rs:12-14); measured ~1e-5.  Ids are the router's,
    unchanged; a row's result does not depend on the rows it shares a tile with."""
    layer, ref, rng = make_layer(mk, n_experts, top_k, d, inter, seed=3 * n_experts + d)
    tc = mk.MoeLayer(ref.gate_w, ref.gate_b, layer._keep[0], layer._keep[1], top_k, act="fp4x6")
    x = rng.standard_normal((batch, d)).astype(np.float32)
    x[3] *= 50.0                       # a row with a large dynamic range
    x[5, ::2] = 0.0
    out, ids, w = tc.moe_forward(x, want_routing=True)
    ids_q, _ = layer.route(x)
    assert np.array_equal(ids, ids_q)
    worst = 0.0
    for t in range(batch):
        o_ref, ids_ref, _ = ref.forward(x[t], use_q8=False, n_threads=8)
        assert np.array_equal(ids[t], ids_ref)
        worst = max(worst, rel(out[t], o_ref))
    assert worst <= 1e-3, worst
    # the same rows in another order and another batch: bit-identical per row
    perm = rng.permutation(batch)
    out2 = tc.moe_forward(np.ascontiguousarray(x[perm][:batch - 1]))
    assert np.array_equal(bits(out2), bits(out[perm][:batch - 1]))
    assert mk.Context.default().status_word() == 0
