"""GPU parity tests for the two attention blocks of a decode layer (kda_forward, src/model.rs:1179-1232;
mla_forward, src/model.rs:1939-2022) at the micro configuration's widths (src/config.rs:47-75), against the
same blocks composed from the CPU oracle's pieces, over several consecutive tokens of one sequence."""
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mk():
    import microkimi_b200 as m
    m.Context.default()
    return m


def gauss(rng, *shape, s=0.02):
    return (rng.standard_normal(shape) * s).astype(np.float32)


def test_kda_block_against_oracle(mk):
    import torch
    from microkimi_b200.blocks import KdaBlock
    rng = np.random.default_rng(21)
    d, H, D, fa = 512, 4, 128, 128
    p = H * D
    # projections gauss 0.02 as the model builder's fallback branch draws them, scaled up so that the gates move
    w = {"q_proj": gauss(rng, p, d, s=0.1), "k_proj": gauss(rng, p, d, s=0.1), "v_proj": gauss(rng, p, d, s=0.1),
         "g_proj": gauss(rng, p, d, s=0.1), "f_a": gauss(rng, fa, d, s=0.1), "f_b": gauss(rng, p, fa, s=0.1),
         "b_proj": gauss(rng, H, d, s=0.1), "o_proj": gauss(rng, d, p), "q_conv": gauss(rng, p, 4, s=0.5),
         "k_conv": gauss(rng, p, 4, s=0.5), "v_conv": gauss(rng, p, 4, s=0.5),
         "a_log": np.log(rng.uniform(1, 16, D)).astype(np.float32), "dt_bias": gauss(rng, p, s=0.3), "o_norm": np.ones(D, np.float32)}
    blk = KdaBlock(H, D, w, gate_lb=-5.0, rms_eps=1e-5)
    ref = O.KdaLayer(H, D, w["q_conv"], w["k_conv"], w["v_conv"], w["a_log"], w["dt_bias"], w["o_norm"], gate_lb=-5.0, rms_eps=1e-5)
    mv = O.matvec_f32
    for t in range(6):
        x = rng.standard_normal(d).astype(np.float32)
        g_low = mv(w["f_b"], mv(w["f_a"], x))
        o = ref.step(mv(w["q_proj"], x), mv(w["k_proj"], x), mv(w["v_proj"], x), g_low, mv(w["b_proj"], x), mv(w["g_proj"], x))
        want = mv(w["o_proj"], o)
        got = blk.forward(torch.from_numpy(x).cuda()).cpu().numpy()
        # the matvecs are bit-exact; the step holds 1e-6 relative (one exp may round differently)
        assert np.abs(got - want).max() <= 2e-6 * max(1.0, np.abs(want).max())
    blk.free()


def test_mla_block_against_oracle(mk):
    import torch
    from microkimi_b200.blocks import MlaBlock
    rng = np.random.default_rng(22)
    d, H, qa, kva, nope, rope, vd = 512, 4, 128, 64, 128, 64, 128
    w = {"q_a": gauss(rng, qa, d, s=0.05), "q_a_ln": (1 + 0.1 * rng.standard_normal(qa)).astype(np.float32),
         "q_b": gauss(rng, H * (nope + rope), qa, s=0.1), "kv_a": gauss(rng, kva + rope, d, s=0.05),
         "kv_a_ln": (1 + 0.1 * rng.standard_normal(kva)).astype(np.float32), "kv_b": gauss(rng, H * (nope + vd), kva, s=0.1),
         "g_proj": gauss(rng, H * vd, d, s=0.05), "o_proj": gauss(rng, d, H * vd)}
    n_tok = 40
    blk = MlaBlock(H, nope, rope, vd, w, max_positions=64, rms_eps=1e-5)
    cache = O.MlaCache(H, nope, rope, vd, 64)
    mv = O.matvec_f32
    scale = np.float32(nope + rope) ** np.float32(-0.5)
    for t in range(n_tok):
        x = rng.standard_normal(d).astype(np.float32)
        q = mv(w["q_b"], O.rmsnorm(mv(w["q_a"], x), w["q_a_ln"], 1e-5))                       # :1948-1954
        c = mv(w["kv_a"], x)                                                                   # :1956-1957
        kb = mv(w["kv_b"], O.rmsnorm(c[:kva], w["kv_a_ln"], 1e-5)).reshape(H, nope + vd)       # :1959-1962
        k_new = np.concatenate([kb[:, :nope], np.broadcast_to(c[kva:], (H, rope))], axis=1)    # :1964-1973
        cache.push(k_new, kb[:, nope:])
        attn = cache.attn_mqa(q, t, scale).reshape(-1)                                         # :1982-1988
        g = mv(w["g_proj"], x)
        attn = np.array([a * O.lib().or_sigmoid(float(b)) for a, b in zip(attn, g)], np.float32)   # :2015-2019
        want = mv(w["o_proj"], attn)
        got = blk.forward(torch.from_numpy(x).cuda()).cpu().numpy()
        # the q8 attention kernel's tolerance (different but fixed summation order over positions)
        assert np.abs(got - want).max() <= 2e-4 * max(np.abs(want).max(), 1e-3), t
    assert blk.cache.positions() == n_tok
    blk.free()
