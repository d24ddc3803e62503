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
