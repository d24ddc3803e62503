"""Generates the committed golden fixtures from the reference checkout.

Run once where the reference project's checkout is at hand:

    python tests/golden/make_golden.py /path/to/reference

It (1) extracts the vectors the reference's own `selftest` consumes for this
path from ref/ds_golden.json (fp4 block and fp8 block, src/selftest.rs:205-234) and
ref/ds_golden2.json (gate + expert, src/selftest.rs:259-323), and (2) imports
the two reference Python helpers that touch this path - ref/mxfp4_numpy.py
(dequant) and nano/export.py::quantize_mxfp4 (naive-scale quantizer) - and
records their outputs on seeded random inputs.  The fixtures are small .npz
files next to this script; tests never read the reference checkout.
"""
import importlib.util
import json
import os
import sys

import numpy as np

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
REF = sys.argv[1]
OUT = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    # 1. torch-generated fp4 block the reference selftest checks dequant against
    g = json.load(open(os.path.join(REF, "ref/ds_golden.json")))["fp4"]
    np.savez(os.path.join(OUT, "ds_fp4.npz"),
             rows=np.int64(g["rows"]), cols=np.int64(g["cols"]),
             packed=np.array(g["packed"], np.uint8), scales=np.array(g["scales"], np.uint8),
             dequant=np.array(g["dequant"], np.float32))

    # 1b. torch-generated fp8 e4m3 + ue8m0 (128 x 128 blocks) matrix of the same file (src/selftest.rs:205-224)
    g8 = json.load(open(os.path.join(REF, "ref/ds_golden.json")))["fp8"]
    np.savez_compressed(os.path.join(OUT, "ds_fp8.npz"),
                        rows=np.int64(g8["rows"]), cols=np.int64(g8["cols"]),
                        w_packed=np.array(g8["w_packed"], np.uint8), scales=np.array(g8["scales"], np.uint8),
                        dequant=np.array(g8["dequant"], np.float32))

    # 2. DeepSeek gate (3 tokens x 32 experts, top-6, route_scale 1.5) and SwiGLU-clamp expert
    g2 = json.load(open(os.path.join(REF, "ref/ds_golden2.json")))
    gate, ex = g2["gate"], g2["expert"]
    np.savez(os.path.join(OUT, "ds_gate_expert.npz"),
             gate_x=np.array(gate["x"], np.float32).reshape(3, 16),
             gate_w=np.array(gate["gate_w"], np.float32).reshape(32, 16),
             gate_bias=np.array(gate["bias"], np.float32),
             gate_indices=np.array(gate["indices"], np.int32).reshape(3, 6),
             gate_weights=np.array(gate["weights"], np.float32).reshape(3, 6),
             ex_x=np.array(ex["x"], np.float32),
             ex_w1=np.array(ex["w1"], np.float32).reshape(16, 8),
             ex_w2=np.array(ex["w2"], np.float32).reshape(8, 16),
             ex_w3=np.array(ex["w3"], np.float32).reshape(16, 8),
             ex_out=np.array(ex["out"], np.float32))

    # 3. reference numpy dequant on random blobs (all 16 codes, scale bytes 90..139 plus 0 and 1)
    mx = _load(os.path.join(REF, "ref/mxfp4_numpy.py"), "ref_mxfp4_numpy")
    rng = np.random.default_rng(20240601)
    rows, cols = 24, 256
    packed = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
    scales = rng.integers(90, 140, (rows, cols // 32), dtype=np.uint8)
    # bytes 0 and 1 exercise the subnormal scales.  Bytes near 254 are left out:
    # numpy's float32 exp2 is off by an ulp there, while the engine's exp2_i
    # (src/mxfp4.rs:10-16) builds the power of two from its bit pattern.
    scales[0, 0], scales[1, 1] = 0, 1
    with np.errstate(all="ignore"):
        deq = mx.dequant_mxfp4(packed, scales).astype(np.float32)
    np.savez(os.path.join(OUT, "mxfp4_numpy_dequant.npz"), packed=packed, scales=scales, dequant=deq)

    # 4. reference naive-rule quantizer (nano/export.py) on seeded gaussian + edge rows
    ex_mod = _load(os.path.join(REF, "nano/export.py"), "ref_nano_export")
    w = (rng.standard_normal((16, 128)) * 0.02).astype(np.float32)
    w[3, :32] = 0.0                      # all-zero block -> scale byte 0
    w[4, 32:64] = np.float32(6.0 * 0.25) * np.sign(rng.standard_normal(32)).astype(np.float32)
    w[5, 0] = -0.0
    p, s = ex_mod.quantize_mxfp4(w)
    np.savez(os.path.join(OUT, "export_quantize_naive.npz"), w=w, packed=p.astype(np.uint8), scales=s.astype(np.uint8))
    # 5. the KDA recurrence and AttnRes vectors of the reference's `selftest` (src/selftest.rs:131-180): the
    #    inputs and calls of ref/make_golden.py (seed 42, chunk_kda of the vendored fla shim, the AttnRes formula)
    import torch
    sys.path.insert(0, os.path.join(REF, "nano", "vendor"))
    from fla.ops.kda import chunk_kda
    tg = torch.Generator().manual_seed(42)
    T, H, K, V = 3, 4, 128, 128
    q = torch.randn(1, T, H, K, generator=tg)
    k = torch.randn(1, T, H, K, generator=tg)
    v = torch.randn(1, T, H, V, generator=tg)
    graw = torch.randn(1, T, H, K, generator=tg)
    beta = torch.randn(1, T, H, generator=tg)
    a_log = torch.randn(K, generator=tg)
    dt_bias = torch.randn(H * K, generator=tg)
    o, S = chunk_kda(q, k, v, graw, beta, A_log=a_log, dt_bias=dt_bias, scale=None, initial_state=None,
                     output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True,
                     use_beta_sigmoid_in_kernel=True, safe_gate=True, lower_bound=-5.0)
    f = lambda t: t.flatten().numpy().astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "kda_recurrence.npz"), T=np.int64(T), H=np.int64(H), K=np.int64(K),
                        q=f(q), k=f(k), v=f(v), g=f(graw), beta=f(beta), A_log=f(a_log), dt_bias=f(dt_bias), o=f(o), S=f(S))
    # the same generator goes on: 2 x 16 SiTU inputs, then the AttnRes inputs (D = 512, 3 blocks + prefix, eps 1e-5)
    gs = torch.randn(16, generator=tg) * 6.0
    us = torch.randn(16, generator=tg) * 30.0
    situ = 4.0 * torch.tanh(gs / 4.0) * torch.sigmoid(gs) * (25.0 * torch.tanh(us / 25.0))
    D, B = 512, 3
    blocks = torch.randn(B, D, generator=tg)
    prefix = torch.randn(D, generator=tg)
    norm_w = torch.randn(D, generator=tg)
    proj_w = torch.randn(D, generator=tg)
    vv = torch.cat([blocks, prefix.unsqueeze(0)], dim=0)
    kk = vv * torch.rsqrt(vv.pow(2).mean(-1, keepdim=True) + 1e-5)
    probs = (kk * (norm_w * proj_w)).sum(-1).softmax(-1)
    out = (probs.unsqueeze(-1) * vv).sum(0)
    np.savez_compressed(os.path.join(OUT, "situ_attn_res.npz"), situ_g=f(gs), situ_u=f(us), situ_out=f(situ),
                        blocks=blocks.numpy().astype(np.float32), prefix=f(prefix), norm_w=f(norm_w), proj_w=f(proj_w), out=f(out))
    print("wrote fixtures to", OUT)


if __name__ == "__main__":
    main()
