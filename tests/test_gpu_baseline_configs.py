"""GPU parity tests at the FULL sizes of the benchmark configurations, through the C ABI, against the
CPU oracle.  The toy-size files next to this one cover the edge cases; this one makes every launch
shape of the real workloads (item splits of the expert kernels, KV splits and the merge of the
attention kernels, the full vocabulary) meet the oracle.

  q8_0 lm_head 163840 x 7168 ...... quantized bytes / scales of a row sample bit-exact, strict-mode
                                    logits of the sample bit-exact, default mode 1e-5, greedy pick
                                    equal to the oracle's over ALL rows                (batch 1, 8)
  MoE layer 384 + 1 experts ....... ids exact in slot order, weights 1e-6, outputs <= 1e-3 max|ref|
                                    (src/parity.rs:12-14), batch rows == single-token bits
                                                                                      (batch 1, 16, 256)
  MLA absorbed, 64 heads .......... <= 1e-3 max|ref| for the tcgen05 and mma.sync kernels, 2e-4 for
                                    the exact-integer kernel, ctx 4096 / 16384 / 65536 (batch 1, 8)
  MLA per-head layout, 64 heads ... 2e-4 at the same contexts (a head sample on the CPU side)

Inputs are seeded synthetic tensors with the stated shapes and distributions.  Weights that would
take minutes to quantize on the CPU at full size are assembled from a pool (see each test).
"""
import numpy as np
import pytest

from conftest import bits
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mk():
    import microkimi_b200 as m
    ctx = m.Context.default()
    ctx.use_torch_stream()
    return m


def rel(a, ref):
    return np.abs(a.astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-12)


# ------------------------------------------------------------------ q8_0 lm_head, 163840 x 7168
def test_lm_head_full_vocabulary(mk):
    """Q8Head::from_f32 + ::matvec (src/model.rs:274-335) on the whole 163840 x 7168 matrix.  The f32
    matrix is drawn on the GPU (N(0, 0.02)); a seeded sample of 4096 rows comes back to the host and
    goes through the oracle's own quantizer and matvec; the greedy pick is compared over all rows by
    running the oracle's matvec on the exported q8_0 matrix (whose bytes the sample pins)."""
    import torch
    V, D = 163840, 7168
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(20)
    wf = torch.empty((V, D), dtype=torch.float32, device=dev)
    wf.normal_(0.0, 0.02, generator=gen)
    head = mk.Q8Head.from_f32(wf, V, D)
    rng = np.random.default_rng(21)
    sample = np.sort(rng.choice(V, 4096, replace=False))
    sample[:3] = (0, 1, 15)
    sample[-2:] = (V - 2, V - 1)
    sample = np.unique(sample)
    w_s = wf[torch.from_numpy(sample).to(dev)].cpu().numpy()
    del wf
    torch.cuda.empty_cache()
    q_all, s_all = head.export()
    q_ref, s_ref = O.q8head_from_f32(w_s)
    assert np.array_equal(q_all[sample], q_ref), "quantized bytes of the sampled rows"
    assert np.array_equal(bits(s_all[sample]), bits(s_ref)), "block scales of the sampled rows"
    for batch in (1, 8):
        x = rng.standard_normal((batch, D)).astype(np.float32)
        xd = torch.from_numpy(x).to(dev)
        y, am = head.matvec(xd, want_argmax=True)
        ys = head.matvec(xd, strict=True)
        torch.cuda.synchronize()
        y, am, ys = y.cpu().numpy(), am.cpu().numpy(), ys.cpu().numpy()
        for b in range(batch):
            full = O.q8head_matvec(q_all, s_all, x[b], n_threads=O.num_threads())
            want = O.q8head_matvec(q_ref, s_ref, x[b])
            assert np.array_equal(bits(full[sample]), bits(want))            # the oracle is row-wise
            assert np.array_equal(bits(ys[b, sample]), bits(want)), "strict mode reproduces the CPU bits"
            assert np.array_equal(bits(ys[b]), bits(full))
            assert np.abs(y[b] - full).max() <= 1e-5 * np.abs(full).max()
            assert int(am[b]) == O.argmax(full), "greedy pick over the whole vocabulary"
    # the host-pointer entry point on the same matrix
    yh, amh = head.matvec(x[0], want_argmax=True)
    assert np.array_equal(bits(yh), bits(y[0])) and int(amh[0]) == int(am[0])
    assert mk.Context.default().status_word() == 0
    head.free()


# ------------------------------------------------------------------ MoE layer, 384 + 1 experts, top-8
POOL = 6          # distinct quantized matrices per kind (w1, w2, w3); experts are row rotations of them


def _pool_layer(mk):
    """384 routed + 1 shared experts of 2048 x 7168 / 7168 x 2048 MXFP4.  Quantizing 1155 matrices of 14.7 M
    weights with the searched quantizer takes minutes on the host, so POOL matrices per kind are drawn
    from N(0, 0.02) and quantized (mxfp4::quantize, src/mxfp4.rs:38-138), and expert e takes pool matrix
    e % POOL rotated by 16 * (e // POOL + 1) rows: every expert is a distinct, correctly quantized matrix."""
    import torch
    E, k, d, inter = 384, 8, 7168, 2048
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(33)
    shapes = ((inter, d), (d, inter), (inter, d))
    pool_h = [[O.mxfp4_quantize((rng.standard_normal(s) * 0.02).astype(np.float32)) for _ in range(POOL)] for s in shapes]
    pool_d = [[(torch.from_numpy(p).to(dev), torch.from_numpy(s).to(dev)) for (p, s) in kind] for kind in pool_h]

    def shift(e):
        return 16 * (e // POOL + 1)

    def host_expert(e):
        return [(np.roll(pool_h[j][e % POOL][0], shift(e), axis=0), np.roll(pool_h[j][e % POOL][1], shift(e), axis=0))
                for j in range(3)]

    experts = []
    for e in range(E + 1):
        tri = []
        for j, (r, c) in enumerate(shapes):
            p, s = pool_d[j][e % POOL]
            tri.append(mk.MxFp4Weight(torch.roll(p, shift(e), 0).contiguous(), torch.roll(s, shift(e), 0).contiguous(), r, c))
        experts.append(tuple(tri))
    torch.cuda.synchronize()
    gate_w = (rng.standard_normal((E, d)) * 0.02).astype(np.float32)
    layer = mk.MoeLayer(gate_w, None, experts[:-1], experts[-1], k)
    return layer, gate_w, host_expert, pool_h, (E, k, d, inter)


@pytest.fixture(scope="module")
def big_moe(mk):
    out = _pool_layer(mk)
    yield out
    out[0].free()
    for tri in out[0]._keep[0] + [out[0]._keep[1]]:
        for w in tri:
            w.free()


def _oracle_for(gate_w, host_expert, pool_h, dims, tokens):
    """An oracle layer whose table holds the real matrices of every expert the oracle's own router
    selects for `tokens` (plus the shared expert); entries nobody selects point at a pool matrix."""
    E, k, d, inter = dims
    need = set()
    for x in tokens:
        ids, _, _ = O.router_k3(gate_w, np.zeros(E, np.float32), x, k)
        need.update(int(i) for i in ids)
    filler = [pool_h[j][0] for j in range(3)]
    table = [host_expert(e) if e in need else filler for e in range(E)]
    return O.MoeDs(gate_w, np.zeros(E, np.float32), table, host_expert(E), k), need


@pytest.mark.parametrize("batch,checked", [(1, 1), (16, 16), (256, 8)])
def test_moe_layer_384_experts(mk, big_moe, batch, checked):
    """moe_forward's router (src/model.rs:2153-2173) feeding ds_moe's expert body (src/deepseek.rs:1038-1108)
    at 384 + 1 experts, top-8, hidden 7168, intermediate 2048; tokens N(0, 1)."""
    layer, gate_w, host_expert, pool_h, dims = big_moe
    E, k, d, inter = dims
    rng = np.random.default_rng(100 + batch)
    x = rng.standard_normal((batch, d)).astype(np.float32)
    out, ids, w = layer.moe_forward(x, want_routing=True)
    ids_r, w_r, lg = layer.route(x, want_logits=True)
    assert np.array_equal(ids, ids_r) and np.array_equal(bits(w), bits(w_r))
    # routing of EVERY token against the oracle's router (cheap), outputs of a token sample
    zero_b = np.zeros(E, np.float32)
    for t in range(batch):
        ids_ref, w_ref, lg_ref = O.router_k3(gate_w, zero_b, x[t], k)
        assert np.array_equal(bits(lg[t]), bits(lg_ref)), "router logits must be bit-exact"
        assert np.array_equal(ids[t], ids_ref), "expert ids must match in slot order"
        assert np.abs(w[t] - w_ref).max() <= 1e-6 * np.abs(w_ref).max()
    pick = list(range(batch)) if checked == batch else sorted(rng.choice(batch, checked, replace=False).tolist())
    ref, need = _oracle_for(gate_w, host_expert, pool_h, dims, [x[t] for t in pick])
    worst = 0.0
    for t in pick:
        o_ref, ids_ref, _ = ref.forward(x[t], use_q8=True, n_threads=O.num_threads())
        assert set(int(i) for i in ids_ref) <= need
        worst = max(worst, rel(out[t], o_ref))
    assert worst <= 1e-3, worst
    # a token's result does not depend on the batch it travels in (src/model.rs:2398-2411)
    for t in pick[:4]:
        assert np.array_equal(bits(layer.moe_forward(x[t])), bits(out[t]))
    if batch >= 4:
        # the block-scaled tensor-core path on the same weights: held to the engine's exact-f32 path (src/mxfp4.rs:488-539)
        tc = mk.MoeLayer(gate_w, None, layer._keep[0], layer._keep[1], k, act="fp4x6")
        out_tc, ids_tc, _ = tc.moe_forward(x, want_routing=True)
        assert np.array_equal(ids_tc, ids)
        worst_tc = max(rel(out_tc[t], ref.forward(x[t], use_q8=False, n_threads=O.num_threads())[0]) for t in pick)
        assert worst_tc <= 1e-3, worst_tc
        assert rel(out_tc, out) <= 3e-2          # and near the q8 path, whose own distance to the f32 path is ~6e-3
        tc.free()
    assert mk.Context.default().status_word() == 0


# ------------------------------------------------------------------ MLA decode attention, 64 heads
def _lens(ctx_len, batch):
    return [ctx_len - 37 * s for s in range(batch)]      # ragged: the sequences of a batch end in different tiles


@pytest.mark.parametrize("ctx_len", [4096, 16384, 65536])
@pytest.mark.parametrize("batch", [1, 8])
def test_mla_absorbed_full_context(mk, ctx_len, batch):
    """One shared q8_0 latent row (512 + 64) per position, 64 heads, softmax scale 1/sqrt(192), rows and
    queries N(0, 1): the per-position recipe of mla_attn_flash_q8_mqa (src/model.rs:1833-1890)."""
    import torch
    H, lat, vd = 64, 576, 512
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(ctx_len + batch)
    lens = _lens(ctx_len, batch)
    cache = mk.MlaCache(H, lat, 0, vd, ctx_len, n_seqs=batch, layout="absorbed")
    check = sorted({0, batch - 1, batch // 2})
    refs = {}
    for s, n in enumerate(lens):
        rows = torch.randn((n, lat), dtype=torch.float32, device=dev, generator=gen)
        for lo in range(0, n, 8192):
            cache.push(rows[lo:lo + 8192].contiguous(), seq=s)
        if s in check:
            r = O.MlaAbsCache(lat, vd, n)
            r.push_many(rows.cpu().numpy())
            refs[s] = r
    q = torch.randn((batch, H, lat), dtype=torch.float32, device=dev, generator=gen)
    qh = q.cpu().numpy()
    scale = np.float32(1.0 / np.sqrt(192.0))
    want = {s: refs[s].attn(qh[s], lens[s] - 1, scale) for s in check}
    ctx = mk.Context.default()
    for opt, tol in ((None, 1e-3), ("mla_no_t5", 1e-3), ("mla_no_tc", 2e-4)):
        if opt:
            ctx.set_option(opt, 1)
        try:
            out = cache.attend_batch(q, scale)
            torch.cuda.synchronize()
        finally:
            if opt:
                ctx.set_option(opt, 0)
        out = out.cpu().numpy()
        assert np.isfinite(out).all()
        for s in check:
            assert rel(out[s], want[s]) <= tol, (opt, s, rel(out[s], want[s]))
    assert ctx.status_word() == 0
    cache.free()


@pytest.mark.parametrize("ctx_len,batch", [(4096, 1), (4096, 8), (16384, 1), (16384, 8), (65536, 1)])
def test_mla_per_head_full_context(mk, ctx_len, batch):
    """The engine's cache layout (src/model.rs:765-781) at 64 heads, nope 128 / rope 64 / v 128.  Heads are
    independent in mla_attn_flash_q8_mqa, so the CPU side builds its cache from a sample of heads (head 0,
    which supplies the shared rope part, is always in it) and compares those heads."""
    import torch
    H, nope, rope, vd = 64, 128, 64, 128
    hd = nope + rope
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7 * ctx_len + batch)
    lens = _lens(ctx_len, batch)
    cache = mk.MlaCache(H, nope, rope, vd, ctx_len, n_seqs=batch)
    heads = [0, 21, 42, 63]
    hsel = torch.tensor(heads, device=dev)
    check = sorted({0, batch - 1})
    refs = {}
    for s, n in enumerate(lens):
        ks = {h: [] for h in range(2)}
        for lo in range(0, n, 4096):
            m = min(4096, n - lo)
            kk = torch.randn((m, H, hd), dtype=torch.float32, device=dev, generator=gen)
            kk[:, 1:, nope:] = kk[:, :1, nope:]                  # the rope part is shared by the heads
            vv = torch.randn((m, H, vd), dtype=torch.float32, device=dev, generator=gen)
            cache.push(kk, vv, seq=s)
            if s in check:
                ks[0].append(kk[:, hsel].cpu().numpy())
                ks[1].append(vv[:, hsel].cpu().numpy())
        if s in check:
            K, V = np.concatenate(ks[0]), np.concatenate(ks[1])
            r = O.MlaCache(len(heads), nope, rope, vd, n)
            for j in range(n):
                r.push(K[j], V[j])
            refs[s] = r
    q = torch.randn((batch, H, hd), dtype=torch.float32, device=dev, generator=gen)
    qh = q.cpu().numpy()
    scale = np.float32(1.0 / np.sqrt(192.0))
    ctx = mk.Context.default()
    for opt in (None, "mla_no_tc"):
        if opt:
            ctx.set_option(opt, 1)
        try:
            out = cache.attend_batch(q, scale)
            torch.cuda.synchronize()
        finally:
            if opt:
                ctx.set_option(opt, 0)
        out = out.cpu().numpy()
        for s in check:
            want = refs[s].attn_mqa(qh[s][heads], lens[s] - 1, scale).reshape(len(heads), vd)
            assert rel(out[s][heads], want) <= 2e-4, (opt, s)
    assert ctx.status_word() == 0
    cache.free()
