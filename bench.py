#!/usr/bin/env python
"""Benchmark of the quantized decode hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (this library)
    python bench.py --impl reference --gpus N --steps K ...  (CPU restatement of the reference path)

Headline workload: the q8_0 lm_head GEMV - W is vocab 163840 x hidden 7168 drawn from
N(0, 0.02) and quantized row-wise to q8_0 (32-wide blocks, int8 values + one f32
scale per block, the engine's layout); x is f32[7168] from N(0, 1); batch 1.  A
step is one logits projection (activation quantization + GEMV + greedy argmax).
With N > 1 GPUs the vocabulary is sharded V/N rows per rank and the complete f32 logits and the greedy
token reach every rank (peer-memory exchange kernel, or the NCCL all-gather with --collective nccl);
--token-only times the greedy step that exchanges only the ranks' (maximum, index) pairs instead (both
peer forms are timed, the other one as an extra key); total work is fixed, so scaling is "strong".

metric = quantized GB/s: algorithmic bytes of one step (int8 values + block
scales + x + logits) divided by the step time, summed over all ranks.
Prints ONE JSON line on rank 0.  After the headline measurement the same line carries, under
"extra", bounded runs of the other workloads of the path (single-expert MXFP4 GEMV, the MoE
layer, absorbed MLA decode attention, the lm_head at batch 8; expert-parallel MoE at N > 1);
--no-extra skips them.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

VOCAB, HIDDEN = 163840, 7168
SIGMA_W = 0.02
L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the lm_head kernel on one GPU holding the whole
# matrix, from an ncu capture of this command (1.321224 GB read + 4.7 MB written); a constant, not re-measured per run
NCU_TRAFFIC_PER_LAUNCH_N1 = 1.3259e9
CPU_SAMPLE_ROWS = 32768  # bounded sample of the workload for the CPU legs (235 MB of int8, > any LLC)
METRIC = "quantized GB/s, q8_0 lm_head GEMV"
ACT_MODE = "q8 (the engine's default integer path: q8_0 activation, exact int32 block dots, f32 rescale)"


def algorithmic_bytes(rows, cols, batch, scale_bytes=4):
    """int8 values + block scales + x (f32) + logits (f32), per step."""
    return rows * cols + rows * (cols // 32) * scale_bytes + batch * cols * 4 + batch * rows * 4


def workload_config(world, batch, gather_logits=False):
    """The `config` object of the JSON line; both arms print the same one."""
    return {"workload": f"q8_0 lm_head GEMV {VOCAB}x{HIDDEN} (f32 block scales), batch {batch}, vocab-sharded {world} way(s)"
                        + ("" if world == 1 else (", complete f32 logits on every rank" if gather_logits else
                                                  ", greedy token on every rank, f32 logits sharded (token-only exchange)")),
            "batch": batch, "rows_per_gpu": VOCAB // world, "act_mode": ACT_MODE,
            "l2": "inputs larger than L2: every timed pass streams a weight shard that is not resident "
                  "(shards below 4 x L2 rotate over copies until they exceed it)",
            "algorithmic_bytes_per_step": algorithmic_bytes(VOCAB // world, HIDDEN, batch) * world}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.time()] + [c.strip() for c in line.split(",")])

    def stop(self, window=None):
        """Median SM clock and the throttle reasons seen; `window` = (t0, t1) wall-clock seconds keeps only the
        samples taken while the load ran (all samples if none fell inside)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = self.rows
        inside = [r for r in rows if window and window[0] <= r[0] <= window[1]]
        where = "timed regions + about 1 s of the same steps" if inside else "whole run"
        for r in (inside or rows):
            r = r[1:]
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for n, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except (ValueError, IndexError):
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": where}


# ---------------------------------------------------------------- CPU legs (the oracle is the thing timed here)
def cpu_leg(steps, warmup, rows=CPU_SAMPLE_ROWS):
    """Times the CPU restatement of Q8Head::matvec on a bounded sample of the workload: the first `rows`
    vocabulary rows.  All host cores this process may use, counted from its affinity mask - not from
    OMP_NUM_THREADS, which torchrun sets to 1 for its children."""
    from oracle import oracle as O
    threads = O.host_threads()
    O.set_num_threads(threads)
    rng = np.random.default_rng(1234)
    w = rng.standard_normal((rows, HIDDEN), dtype=np.float32) * np.float32(SIGMA_W)
    q, s = O.q8head_from_f32(w)
    del w
    x = rng.standard_normal(HIDDEN).astype(np.float32)
    for _ in range(max(1, warmup)):
        O.q8head_matvec(q, s, x, n_threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.q8head_matvec(q, s, x, n_threads=threads)
    dt = (time.perf_counter() - t0) / steps
    gbs = algorithmic_bytes(rows, HIDDEN, 1) / dt / 1e9
    return {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"first {rows} of {VOCAB} vocabulary rows x {HIDDEN}, batch 1, {steps} steps after {max(1, warmup)} "
                      f"warm-up, C restatement of Q8Head::matvec (src/model.rs:290-335) with {threads} OpenMP threads"}, dt


def run_reference(args):
    """The reference arm: the engine's own CPU implementation of the path.  The engine is Rust and no Rust
    toolchain exists on this machine, so the arm times the line-by-line C restatement of Q8Head::matvec
    (the oracle) with all host threads.  Under torchrun rank 0 alone runs; the others leave at once."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    cb, dt = cpu_leg(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": workload_config(world, args.batch, not args.token_only),
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- helpers shared by the workloads
def _timed(torch, fn, steps, warmup):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _graph_time(torch, ctx, body, calls, reps):
    """`body()` enqueues `calls` library calls; they are captured as ONE CUDA graph and replayed: what a decode
    loop that replays its token pays per call, without the host's launch cost.  Returns ms per call."""
    body()                                   # first-use set-up (workspace growth, attributes) stays outside the capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    ctx.use_torch_stream()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(reps):
        g.replay()
    g1.record()
    torch.cuda.synchronize()
    return g0.elapsed_time(g1) / (reps * calls)


def _rand_mxfp4(torch, mk, ctx, gen, dev, rows, cols):
    """Synthetic MXFP4 matrix: uniform codes, scale bytes 118..123 (the kernels' speed does not depend on values)."""
    p = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device=dev, generator=gen)
    s = torch.randint(118, 124, (rows, cols // 32), dtype=torch.uint8, device=dev, generator=gen)
    return mk.MxFp4Weight(p, s, rows, cols, ctx=ctx)


def _roof(alg_bytes, ms, note=None):
    peak, kind = measured_peaks()
    ach = alg_bytes / (ms * 1e-3) / 1e9
    r = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_kind": kind}
    if note:
        r["note"] = note
    return r


# ---------------------------------------------------------------- workloads beside the headline
def measure_mxfp4_gemv(torch, mk, ctx, dev, rows=7168, cols=2048, batch=1, copies=128, steps=256, warmup=20, act="q8",
                       graph=True):
    """One MXFP4 matvec (the down-projection of one expert, 7168 x 2048 by default) over `copies` rotating matrices,
    so that every call reads a matrix that is not in L2."""
    gen = torch.Generator(device=dev)
    gen.manual_seed(11)
    ws = [_rand_mxfp4(torch, mk, ctx, gen, dev, rows, cols) for _ in range(copies)]
    x = torch.randn((batch, cols), dtype=torch.float32, device=dev, generator=gen)
    ms_call = _timed(torch, lambda i: ws[i % copies].matvec(x, act=act), steps, warmup)
    ctx.prof_enable(True)
    _timed(torch, lambda i: ws[i % copies].matvec(x, act=act), steps, 0)
    n, kms = ctx.prof_read("matvec_mxfp4")
    ctx.prof_enable(False)
    graph_us = None
    if graph:
        def body():
            for w in ws:
                w.matvec(x, act=act)
        graph_us = _graph_time(torch, ctx, body, copies, max(3, steps // copies)) * 1e3
    alg = rows * cols // 2 + rows * cols // 32 + batch * (cols + rows) * 4
    out = {"workload": f"MXFP4 GEMV {rows}x{cols}, batch {batch}, ring of {copies} cold matrices", "act": act,
           "us_per_call_host_loop": ms_call * 1e3, "kernel_us": kms / max(n, 1) * 1e3, "graph_us_per_call": graph_us,
           "algorithmic_bytes": alg, "status_word": ctx.status_word(),
           "roofline": _roof(alg, (graph_us * 1e-3) if graph_us else ms_call,
                             "whole call (activation quantization + GEMV) " + ("inside a CUDA graph" if graph_us else "from a host loop"))}
    for w in ws:
        w.free()
    return out


def build_moe_layers(torch, mk, ctx, dev, experts, copies, seed=3, act="q8"):
    E, k, d, inter = experts, 8, 7168, 2048
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    layers = []
    for _ in range(copies):
        ex = [tuple(_rand_mxfp4(torch, mk, ctx, gen, dev, r, c) for r, c in ((inter, d), (d, inter), (inter, d)))
              for _ in range(E + 1)]
        gw = (torch.randn((E, d), generator=gen, device=dev) * 0.02).cpu().numpy()
        layers.append(mk.MoeLayer(gw, None, ex[:-1], ex[-1], k, ctx=ctx, act=act))
    return layers, gen


def tc_twins(mk, ctx, layers):
    """The same layers (same registered weights) with the experts of large calls on the block-scaled tcgen05 path."""
    return [mk.MoeLayer(l._gate_w, None, l._keep[0], l._keep[1], l.top_k, ctx=ctx, act="fp4x6") for l in layers]


def free_moe_layers(layers):
    for l in layers:
        ex, sh = l._keep[0], l._keep[1]
        l.free()
        for tri in list(ex) + [sh]:
            if tri is not None:
                for w in tri:
                    w.free()


def measure_moe(torch, mk, ctx, dev, layers, gen, batch, steps, warmup, graph=False):
    """One MoE FFN layer: 384 routed MXFP4 experts + 1 shared, top-8, hidden 7168, intermediate 2048, sigmoid router;
    tokens N(0,1).  `layers` rotate so that the timed passes stay cold in L2."""
    E, k, d, inter, copies = layers[0].n_experts, 8, 7168, 2048, len(layers)
    x = torch.randn((batch, d), dtype=torch.float32, device=dev, generator=gen)
    _, ids, _ = layers[0].moe_forward(x, want_routing=True)
    distinct = int(torch.unique(ids).numel())
    per_expert = 3 * (inter * d // 2 + inter * d // 32)
    alg = E * d * 4 + (distinct + 1) * per_expert + 2 * batch * d * 4
    ms = _timed(torch, lambda i: layers[i % copies].moe_forward(x), steps, warmup)
    l0 = ctx.launches
    layers[0].moe_forward(x)
    launches = ctx.launches - l0
    ctx.prof_enable(True)
    _timed(torch, lambda i: layers[i % copies].moe_forward(x), steps, 0)
    n_e, ms_e = ctx.prof_read("experts")
    n_r, ms_r = ctx.prof_read("router")
    ctx.prof_enable(False)
    graph_ms = None
    if graph:
        def body():
            for l in layers:
                l.moe_forward(x)
        graph_ms = _graph_time(torch, ctx, body, copies, max(3, steps // copies))
    return {"workload": f"MoE layer {E}+1 MXFP4 experts, top-{k}, {d}x{inter}, batch {batch}, {copies} rotating layers",
            "batch": batch, "distinct_experts_routed": distinct, "ms_per_layer": ms, "graph_ms_per_layer": graph_ms,
            "tokens_per_s": batch / (ms * 1e-3), "experts_ms": ms_e / steps if n_e else None,
            "router_ms": ms_r / steps if n_r else None, "launches_per_call": launches, "algorithmic_bytes": alg,
            "status_word": ctx.status_word(), "roofline": _roof(alg, ms, "whole layer call, not one kernel")}


def measure_mla(torch, mk, ctx, dev, layout, ctx_len, batch, steps, warmup):
    """q8_0 MLA decode attention, 64 heads.  absorbed: one shared 512+64 latent row per position (648 B with f32
    scales); per_head: the engine's layout at nope 128 / rope 64 / v 128 (18,688 B per position).  Cache rows N(0,1),
    `batch` independent sequences of `ctx_len` positions, softmax scale 1/sqrt(192)."""
    H, B, n = 64, batch, ctx_len
    gen = torch.Generator(device=dev)
    gen.manual_seed(4)
    if layout == "absorbed":
        cache = mk.MlaCache(H, 576, 0, 512, n, n_seqs=B, layout="absorbed", ctx=ctx)
        qdim, per_pos = 576, 576 + 18 * 4
        for s_ in range(B):
            for lo in range(0, n, 8192):
                m = min(8192, n - lo)
                cache.push(torch.randn((m, 576), dtype=torch.float32, device=dev, generator=gen), seq=s_)
    else:
        cache = mk.MlaCache(H, 128, 64, 128, n, n_seqs=B, ctx=ctx)
        qdim, per_pos = 192, H * 128 + H * 4 * 4 + 64 * 4 + H * 128 + H * 4 * 4
        for s_ in range(B):
            for lo in range(0, n, 1024):
                m = min(1024, n - lo)
                kk = torch.randn((m, H, 192), dtype=torch.float32, device=dev, generator=gen)
                vv = torch.randn((m, H, 128), dtype=torch.float32, device=dev, generator=gen)
                cache.push(kk, vv, seq=s_)
    q = torch.randn((B, H, qdim), dtype=torch.float32, device=dev, generator=gen)
    scale = 1.0 / np.sqrt(192.0)
    ms = _timed(torch, lambda i: cache.attend_batch(q, scale), steps, warmup)
    alg = B * n * per_pos + B * H * (qdim + cache.vd) * 4
    flops = B * n * 2 * H * (qdim + cache.vd) if layout == "absorbed" else B * n * 2 * H * (192 + 128)
    tf = flops / (ms * 1e-3) / 1e12
    tpeak, tkind = measured_tflops()
    out = {"workload": f"q8_0 MLA decode attention, {layout} layout, 64 heads, ctx {n}, batch {B}", "ms_per_call": ms,
           "algorithmic_bytes": alg, "tflops": tf, "frac_of_bf16_peak": tf / tpeak, "bf16_peak": tpeak, "bf16_peak_kind": tkind,
           "status_word": ctx.status_word(),
           "roofline": _roof(alg, ms, "cache smaller than L2 stays resident between calls" if alg < L2_BYTES else None)}
    cache.free()
    return out


def measure_decode(torch, mk, dev, local, world=1, rank=0, dist=None, n_prompt=64, n_new=256, cpu_tokens=0, path=None, profile_prefill=False):
    """Whole-token decode of the 93-layer micro skeleton (the engine's historical configuration: 69 KDA + 24 MLA layers,
    896 MXFP4 experts top-16 per MoE layer, q8_0 lm_head over 163840 rows, q8_0 MLA caches): a synthetic model file with the
    builder's shapes and distributions, a seeded 64-token prompt prefilled layer by layer (one GPU), then 256 greedy steps whose token ids
    never leave the GPU.  One CUDA graph replay per token; at N > 1 the experts are block-partitioned over the ranks and the
    lm_head rows sharded, exchanged by peer-memory stores (the token is recorded once per buffer parity of the exchanges)."""
    import tempfile

    from microkimi_b200 import model as M
    own = mk.Context(local)                       # a context of its own: its stream is a real stream, so the token can be recorded
    stream = torch.cuda.Stream(device=dev)
    out = {"workload": f"decode of the 93-layer micro skeleton, {n_prompt}-token prompt + {n_new} greedy steps, "
                       f"expert-parallel x{world}" if world > 1 else
                       f"decode of the 93-layer micro skeleton, {n_prompt}-token prompt + {n_new} greedy steps, one GPU"}
    path = path or os.path.join(tempfile.gettempdir(), "mk_bench_microkimi.bin")
    t0 = time.time()
    if rank == 0:
        with torch.cuda.stream(stream):
            own.use_torch_stream()
            M.build_synthetic_bin(path, None, seed=20240, ctx=own)
            torch.cuda.synchronize()
    if dist is not None and world > 1:
        dist.barrier()
    out["build_s"] = round(time.time() - t0, 2)
    t0 = time.time()
    with torch.cuda.stream(stream):
        own.use_torch_stream()
        model = M.Model(path, n_prompt + n_new + 8, use_graph=True, rank=rank, world=world, ctx=own)
        if world > 1:
            model.connect()
        out["load_s"] = round(time.time() - t0, 2)
        out["weight_mb_per_gpu"] = model.weight_bytes / 1e6
        rng = np.random.default_rng(64)
        prompt = rng.integers(0, 163584, n_prompt).astype(np.int32)
        # warm-up: the whole prompt once (the layers' row buffers grow to the prompt's size here, not inside the timed
        # prefill: ~2000 cudaFree / cudaMalloc calls, which took 0.9 s late in a process that holds thousands of
        # allocations), then eager token, recorded token, replays
        model.generate(prompt, 3)
        model.reset()
        torch.cuda.synchronize()

        def sync_all():
            torch.cuda.synchronize()
            if dist is not None and world > 1:
                dist.barrier()
                torch.cuda.synchronize()
        sync_all()
        # the prompt once token by token (the decode path; kept for comparison) ...
        ptok = torch.from_numpy(prompt).to(dev)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(stream)
        for i in range(n_prompt):
            model.forward_dev(ptok[i:i + 1])
        s1.record(stream)
        sync_all()
        out["prompt_token_by_token_ms_per_token"] = s0.elapsed_time(s1) / n_prompt
        model.reset()
        sync_all()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(stream)
        if profile_prefill:
            torch.cuda.profiler.start()           # for `ncu --profile-from-start off`: the launch list of the warm prefill alone
        first = model.generate(prompt, 1)         # ... and layer by layer (mk_model_generate prefills; returns after its own synchronization)
        if profile_prefill:
            torch.cuda.profiler.stop()
        e1.record(stream)
        for _ in range(n_new):
            model.forward_dev(None)               # the previous pick, on the device
        e2.record(stream)
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1), e1.elapsed_time(e2)], dtype=torch.float64, device=dev)
        if dist is not None and world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        prefill_ms, decode_ms = float(t[0].item()), float(t[1].item())
        out.update({"prompt_ms_per_token": prefill_ms / n_prompt, "prefill_tokens_per_s": n_prompt / (prefill_ms * 1e-3),
                    "decode_ms_per_token": decode_ms / n_new,
                    "decode_tokens_per_s": n_new / (decode_ms * 1e-3), "launches_per_token": model.launches_per_token,
                    "first_token": int(first[0]), "status_word": own.status_word()})
        # end to end: every token id goes back to the host before the next step starts (the engine's loop prints and tests it)
        model.reset()
        model.generate(prompt[:4], 1)
        sync_all()
        tok, n_e2e = 1, min(n_new, 64)
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            _, tok = model.forward(tok, want_logits=False)
        e2e = (time.perf_counter() - t0) / n_e2e
        te = torch.tensor([e2e], dtype=torch.float64, device=dev)
        if dist is not None and world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        out["e2e_tokens_per_s"] = 1.0 / float(te.item())
        out["e2e_note"] = "mk_model_forward per token: token id H2D, the token, picked id D2H, synchronize"
        model.free()
    if cpu_tokens and rank == 0:
        from oracle import oracle as O
        threads = O.host_threads()
        O.set_num_threads(threads)
        ref = O.Model(path, cpu_tokens + 4, n_threads=threads)
        tok = int(prompt[0])
        ref.forward(tok)
        t0 = time.perf_counter()
        for _ in range(cpu_tokens):
            tok = O.argmax(ref.forward(tok))
        dt = (time.perf_counter() - t0) / cpu_tokens
        out["cpu_baseline"] = {"value": 1.0 / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
                               "sample": f"{cpu_tokens} decode steps of the same model file, C restatement of Model::forward "
                                         f"(src/model.rs:2889-3031) with {threads} OpenMP threads"}
    own.close()
    return out


def extras_single_gpu(torch, mk, ctx, dev, heads, x1):
    """Bounded runs of the other workloads of the path for the same JSON line (one GPU)."""
    out = {}

    def guard(name, fn):
        t0 = time.time()
        try:
            out[name] = fn()
        except Exception as exc:                      # a failing side workload must not take the headline with it
            out[name] = {"error": f"{type(exc).__name__}: {exc}"}
        out[name]["wall_s"] = round(time.time() - t0, 2)
        torch.cuda.empty_cache()

    def lm_head_b8():
        x8 = torch.randn((8, HIDDEN), dtype=torch.float32, device=dev)
        ctx.prof_enable(True)
        ms = _timed(torch, lambda i: heads[0].matvec(x8, want_argmax=True), 20, 3)
        n, kms = ctx.prof_read("lm_head")
        ctx.prof_enable(False)
        alg = algorithmic_bytes(VOCAB, HIDDEN, 8)
        return {"workload": f"q8_0 lm_head GEMV {VOCAB}x{HIDDEN}, batch 8 (weights read once)", "ms_per_step": ms,
                "kernel_ms": kms / max(n, 1), "algorithmic_bytes": alg, "status_word": ctx.status_word(),
                "roofline": _roof(alg, kms / max(n, 1), "GEMV kernel alone")}
    guard("lm_head_batch8", lm_head_b8)
    guard("config1_mxfp4_gemv_7168x2048", lambda: measure_mxfp4_gemv(torch, mk, ctx, dev))

    def moe():
        layers, gen = build_moe_layers(torch, mk, ctx, dev, 384, 2)
        try:
            res = {f"batch{b}": measure_moe(torch, mk, ctx, dev, layers, gen, b, st, 3, graph=(b == 1))
                   for b, st in ((1, 40), (16, 20), (256, 6))}
            twins = tc_twins(mk, ctx, layers)
            for b, st in ((16, 20), (256, 6)):
                res[f"batch{b}_tcgen05_block_scaled"] = measure_moe(torch, mk, ctx, dev, twins, gen, b, st, 3)
                res[f"batch{b}_tcgen05_block_scaled"]["act_mode"] = ("fp4x6: E2M1 weights + ue8m0 scales as registered, activations as six "
                                                                    "E2M1 limbs (kind::mxf4)")
            for t in twins:
                t.free()
            return res
        finally:
            free_moe_layers(layers)
    guard("config3_moe_layer", moe)
    guard("config4_mla_absorbed", lambda: {f"ctx{n}_batch{b}": measure_mla(torch, mk, ctx, dev, "absorbed", n, b, 30, 3)
                                           for n, b in ((4096, 1), (16384, 8), (65536, 8))})
    guard("mla_per_head_ctx16384_batch8", lambda: measure_mla(torch, mk, ctx, dev, "per_head", 16384, 8, 20, 3))
    for h in heads:
        h.free()
    torch.cuda.empty_cache()
    guard("config5_decode", lambda: measure_decode(torch, mk, dev, ctx.device, cpu_tokens=8))
    return out


def measure_moe_ep(torch, dist, mk, ctx, dev, world, rank, experts, batches, steps, warmup, collective="peer", copies=2):
    """The MoE layer with its routed experts block-partitioned over the ranks (expert parallelism) and the same token
    rows on every rank (decode).  peer: one call per layer, output rows travel by peer-memory stores; nccl: the
    all-to-all form on the same weights (every rank owns batch / world of the rows).  Time = max over ranks."""
    from microkimi_b200 import dist as mkd
    E, k, d, inter = experts, 8, 7168, 2048
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)  # the same router and token rows on every rank
    gw = (torch.randn((E, d), generator=gen, device=dev) * 0.02).cpu().numpy()
    xs = {b: torch.randn((b, d), dtype=torch.float32, device=dev, generator=gen) for b in batches}
    lo, hi = mkd.local_expert_range(E, world, rank)
    layers = []
    for _ in range(copies):
        mine = [None] * E
        for e in range(lo, hi):
            mine[e] = tuple(_rand_mxfp4(torch, mk, ctx, gen, dev, r, c) for r, c in ((inter, d), (d, inter), (inter, d)))
        shared = tuple(_rand_mxfp4(torch, mk, ctx, gen, dev, r, c) for r, c in ((inter, d), (d, inter), (inter, d)))
        layers.append(mk.MoeLayer(gw, None, mine, shared, k, ctx=ctx))
    eps = [mkd.PeerEpMoeLayer(l, max_tokens=16) for l in layers] if collective == "peer" else [mkd.EpMoeLayer(l) for l in layers]
    res = {}
    for b in batches:
        x = xs[b]
        if collective == "peer":
            fn = lambda i: eps[i % copies].forward(x)
        else:
            per = (b + world - 1) // world
            xl = x[rank * per:(rank + 1) * per].contiguous()
            fn = lambda i: eps[i % copies].forward(xl)
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        st = torch.tensor([ctx.status_word()], dtype=torch.int32, device=dev)
        dist.all_reduce(st, op=dist.ReduceOp.MIN)
        res[f"batch{b}"] = {"ms_per_layer": float(t.item()), "tokens_per_s": b / (float(t.item()) * 1e-3), "status_word": int(st.item())}
    for e in eps:
        if hasattr(e, "free"):
            e.free()
    free_moe_layers(layers)
    return {"workload": f"expert-parallel MoE layer, {E}+1 MXFP4 experts over {world} GPUs ({collective}), top-{k}, {d}x{inter}, "
                        f"{copies} rotating layers, the same rows on every rank", **res}


# ---------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist

    import microkimi_b200 as mk

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ctx = mk.Context(local)
    mk.Context._default = ctx
    ctx.use_torch_stream()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()          # nvidia-smi needs a second to start: begin before the weights are made
    batch = args.batch
    rows = VOCAB // world
    shard_bytes = rows * HIDDEN + rows * (HIDDEN // 32) * 4
    # keep every timed pass cold in L2: rotate over copies when a shard is small
    copies = 1 if shard_bytes >= 4 * L2_BYTES else int(np.ceil(4 * L2_BYTES / shard_bytes))
    heads = []
    gen = torch.Generator(device=dev)
    for c in range(copies):
        gen.manual_seed(1000 + 17 * rank + c)
        wf = torch.empty((rows, HIDDEN), dtype=torch.float32, device=dev)
        wf.normal_(0.0, SIGMA_W, generator=gen)
        heads.append(mk.Q8Head.from_f32(wf, rows, HIDDEN, ctx=ctx))
        del wf
    torch.cuda.empty_cache()
    gen.manual_seed(7)
    x = torch.randn((batch, HIDDEN), dtype=torch.float32, device=dev, generator=gen)
    logits = torch.empty((batch, VOCAB), dtype=torch.float32, device=dev) if world > 1 else None
    # N > 1: after the matvec ONE exchange kernel pushes the shard's logits into every rank's gather buffer (peer-memory
    # stores + flags); --collective nccl runs the library all-gather instead, for comparison
    fused = None
    fused_note = None
    if world > 1 and batch <= 2 and args.collective == "peer":
        from microkimi_b200 import dist as mkd
        ok = torch.ones(1, dtype=torch.int32, device=dev)
        try:
            fused = mkd.FusedVocabHead(heads[0], VOCAB, max_batch=batch)
        except Exception as exc:   # e.g. no peer access between two GPUs of this box
            fused_note = f"peer buffers unavailable ({type(exc).__name__}: {exc}); NCCL all-gather used"
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)   # all ranks take the same path
        if int(ok.item()) == 0:
            fused = None
            fused_note = fused_note or "peer buffers unavailable on another rank; NCCL all-gather used"

    def step(i):
        if world == 1:
            y, _ = heads[i % copies].matvec(x, want_argmax=True)
            return y
        if fused is not None:
            return fused.matvec(x, want_argmax=True, head=heads[i % copies], want_logits=not args.token_only)
        y = heads[i % copies].matvec(x)
        # vocab-sharded logits -> full logits on every rank
        if batch == 1:
            dist.all_gather_into_tensor(logits.view(-1), y.view(-1))
        else:
            parts = [logits[:, r * rows:(r + 1) * rows] for r in range(world)]
            dist.all_gather(parts, y)  # strided destination views
        return logits, logits.argmax(dim=1)   # the step ends with the token id, as on the other paths

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    if fused is not None:
        # self-check of the peer path before it is timed: the complete logits and the token id of one step must equal
        # the library all-gather of the same shard results bit for bit, and no bounded wait may have run out
        ptr, am = fused.matvec(x, want_argmax=True, head=heads[0])
        got = fused.logits_tensor(ptr, batch)
        y = heads[0].matvec(x)
        want = torch.empty((world, batch, rows), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(want.view(-1), y.contiguous().view(-1))
        want = want.permute(1, 0, 2).reshape(batch, VOCAB)
        # and the token-only step: the same token, this rank's rows where the call says they are
        ptr_t, am_t = fused.matvec(x, want_argmax=True, head=heads[0], want_logits=False)
        mine_t = fused.local_rows_tensor(ptr_t, batch)
        bad = torch.tensor([int(ctx.status_word() != 0 or not torch.equal(got, want)
                                or not torch.equal(am.view(-1).long(), want.argmax(dim=1))
                                or not torch.equal(am_t.view(-1).long(), want.argmax(dim=1))
                                or not torch.equal(mine_t, want[:, rank * rows:(rank + 1) * rows]))], dtype=torch.int32, device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            fused = None
            fused_note = "peer-memory gather failed its self-check against the NCCL all-gather; NCCL all-gather used"
            for i in range(args.warmup):
                step(i)
            barrier()
    launches0 = ctx.launches
    step(0)
    launches = (ctx.launches - launches0) * args.steps      # kernels of this library inside one timed region
    # `repeats` timed regions of exactly `steps` steps, each between barriers; the line's value is the median region.
    # One more region of the same steps follows with the per-kernel events on (roofline.kernel_ms, the exchange kernel):
    # those events cost about 10 us per step (measured on 2 GPUs: 118 us per step with them, 105-107 us without), so the
    # regions the value comes from run without them.
    region_ms = []
    t_load0 = time.time()
    for rep in range(args.repeats + 1):
        if rep == args.repeats:
            ctx.prof_enable(True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        if world > 1:
            # the hosts leave the barrier tens of microseconds apart; one more untimed step (its exchange ends on all GPUs
            # together) lines the GPUs up, so that the first event is recorded at the same moment on every rank and the
            # region holds the K steps, not the hosts' skew
            step(args.warmup)
        e0.record()
        for i in range(args.steps):
            step(i)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        region_ms.append(float(t.item()))
    kn, kms = ctx.prof_read("lm_head")
    xn_, xms_ = ctx.prof_read("other")     # N > 1, peer path: the exchange kernel (push, flags, wait, token pick)
    ctx.prof_enable(False)
    ms_step_with_events = region_ms.pop() / args.steps
    st = torch.tensor([ctx.status_word()], dtype=torch.int32, device=dev)   # a bounded device-side wait that ran out sets it
    if world > 1:
        dist.all_reduce(st, op=dist.ReduceOp.MIN)
    status_all = int(st.item())
    per_step = sorted(r / args.steps for r in region_ms)
    ms_step = float(np.median(per_step))
    # the other form of the exchange (complete logits on every rank / token only), one timed region, for the same line
    other_ms = None
    if fused is not None:
        def other_step(i):
            return fused.matvec(x, want_argmax=True, head=heads[i % copies], want_logits=args.token_only)
        for i in range(args.warmup):
            other_step(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        other_step(args.warmup)
        e0.record()
        for i in range(args.steps):
            other_step(i)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        other_ms = float(t.item()) / args.steps
    # the timed regions may be shorter than nvidia-smi's sampling period: the same steps go on, untimed, for about
    # a second, and the clocks reported are the samples taken between the start of the first region and here
    for i in range(int(min(20000, max(1, 1.0 / (ms_step * 1e-3))))):
        step(i)
    barrier()
    t_load1 = time.time()

    # ---- end to end through the host-pointer entry point (pinned host buffers)
    xh = torch.empty((batch, HIDDEN), dtype=torch.float32).pin_memory()
    xh.copy_(x.cpu())
    xn = xh.numpy()
    e2e_steps = max(10, min(args.steps, 100))
    if fused is None:
        # caller-owned pinned result buffers, as the engine passes `out: &mut [f32]`
        yp = torch.empty((batch, rows), dtype=torch.float32).pin_memory()
        ap = torch.empty((batch,), dtype=torch.int32).pin_memory()
        yn, an = yp.numpy(), ap.numpy()
        heads[0].matvec(xn, want_argmax=True, out=yn, argmax_out=an)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            yh, amh = heads[i % copies].matvec(xn, want_argmax=True, out=yn, argmax_out=an)
        torch.cuda.synchronize()
        e2e_dt = (time.perf_counter() - t0) / e2e_steps
    else:
        # every rank: x from pinned host memory, the fused matvec + gather, then this rank's rows of the
        # complete logits and the token id back to pinned host memory (the ranks together return the logits once)
        xd = torch.empty_like(x)
        yh = torch.empty((batch, rows), dtype=torch.float32).pin_memory()
        amh = torch.empty((batch,), dtype=torch.int32).pin_memory()
        lo = rank * rows

        def e2e_step(i):
            xd.copy_(xh, non_blocking=True)
            ptr, am = fused.matvec(xd, want_argmax=True, head=heads[i % copies], want_logits=not args.token_only)
            if not args.token_only:
                full = fused.logits_tensor(ptr, batch)
                yh.copy_(full[:, lo:lo + rows], non_blocking=True)
            else:
                yh.copy_(fused.local_rows_tensor(ptr, batch), non_blocking=True)
            amh.copy_(am, non_blocking=True)
            torch.cuda.synchronize()
        e2e_step(0)
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        e2e_dt = (time.perf_counter() - t0) / e2e_steps
    te = torch.tensor([e2e_dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_dt = float(te.item())
    clocks = sampler.stop((t_load0, t_load1)) if rank == 0 else None

    alg_step = algorithmic_bytes(rows, HIDDEN, batch) * world
    value = alg_step / (ms_step * 1e-3) / 1e9
    peak, peak_kind = measured_peaks()
    kern_ms = kms / max(kn, 1)
    achieved = algorithmic_bytes(rows, HIDDEN, batch) / (kern_ms * 1e-3) / 1e9 if kn else None

    # ---- the other workloads of the path, bounded, for the same line
    extra = None
    used_peer = fused is not None
    if not args.no_extra:
        if fused is not None:
            fused.free()
        if world == 1:
            extra = extras_single_gpu(torch, mk, ctx, dev, heads, x)
        else:
            for h in heads:
                h.free()
            torch.cuda.empty_cache()
            extra = {}
            try:
                extra["moe_expert_parallel_peer"] = measure_moe_ep(torch, dist, mk, ctx, dev, world, rank, 384, (1, 4, 16), 30, 5)
            except Exception as exc:
                extra["moe_expert_parallel_peer"] = {"error": f"{type(exc).__name__}: {exc}"}
            torch.cuda.empty_cache()
            try:
                extra["config5_decode"] = measure_decode(torch, mk, dev, local, world, rank, dist)
            except Exception as exc:
                extra["config5_decode"] = {"error": f"{type(exc).__name__}: {exc}"}

    if rank == 0:
        cb = None
        if world == 1 and not args.no_cpu:
            cb, _ = cpu_leg(8, 2)
        cfg = workload_config(world, batch, (not args.token_only) or not used_peer)
        frac = (achieved / peak) if achieved else None
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": cfg,
            "repeats": {"n": args.repeats, "value_from": f"median of {args.repeats} timed regions of {args.steps} steps",
                        "ms_per_step_each": per_step, "ms_per_step_p10": float(np.percentile(per_step, 10)),
                        "ms_per_step_p90": float(np.percentile(per_step, 90))},
            "run": {"weights_mb_per_gpu": shard_bytes * copies / 1e6, "rotating_copies": copies,
                    **({"region_start": "after the barrier one untimed step lines the GPUs up (its exchange ends on all of them together); "
                                        "the first event follows it on the stream"} if world > 1 else {}),
                    "logits_path": ("one GPU" if world == 1 else
                                    (("one exchange kernel after the matvec pushes the shard's logits into every rank's buffer "
                                      "(peer-memory stores + flags, no collective library call)" if not args.token_only else
                                      "token-only step of greedy decode: one exchange kernel after the matvec sends every rank's (maximum, index) "
                                      "pair to every rank (peer-memory stores + flags, no collective library call); every rank gets the token, "
                                      "the logits stay sharded - all of them computed and stored once, as at N = 1") if used_peer
                                     else "NCCL all-gather of the f32 logits + argmax")),
                    **({"note": fused_note} if fused_note else {})},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": frac,
                         "traffic": (NCU_TRAFFIC_PER_LAUNCH_N1 / world) if batch == 1 else None,
                         "traffic_source": "constant from one ncu capture of this kernel on one GPU holding the whole matrix"
                                           + ("" if world == 1 else f", divided by {world} (traffic is proportional to the rows of a shard); "
                                                                    "not captured at this N"),
                         "peak_kind": peak_kind,
                         "peak_note": "the peak is a copy (read + write); a read-only stream such as this GEMV can run a little "
                                      "above it, so frac may exceed 1 - frac_of_nominal_8000 is the bounded figure",
                         "kernel": "qgemv_spread_kernel<q8_0>",
                         "kernel_ms": kern_ms, "kernel_launches": kn,
                         "kernel_ms_from": "CUDA events around every launch of the kernel in one further region of the same steps "
                                           "(ms_per_step_with_kernel_events); the value's regions run without those events", "frac_of_nominal_8000": (achieved / 8000.0) if achieved else None},
            "cpu_baseline": cb,
            "e2e": {"value": alg_step / e2e_dt / 1e9, "unit": "GB/s", "ms_per_step": e2e_dt * 1e3,
                    "h2d_bytes_per_step": batch * HIDDEN * 4, "d2h_bytes_per_step": batch * rows * 4 + batch * 4,
                    "api": "mk_matvec_q8 (host pointers: pinned x, pinned logits and token id)" if not used_peer else
                           ("pinned x -> mk_matvec_q8_gather_dev -> pinned logits rows + token id, per rank" if not args.token_only else
                            "pinned x -> mk_matvec_q8_gather_token_dev -> pinned logits rows + token id, per rank")},
            "gpu_launches": launches,
            "ms_per_step_with_kernel_events": ms_step_with_events,
            **({"exchange_kernel_ms": xms_ / xn_} if (used_peer and xn_) else {}),
            **({("token_only_ms_per_step" if not args.token_only else "complete_logits_on_every_rank_ms_per_step"): other_ms} if other_ms else {}),
            "status_word": status_all,
            "clocks": clocks,
            "decode_tokens_per_s": ((extra or {}).get("config5_decode") or {}).get("decode_tokens_per_s"),
            "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def _side_ctx():
    import torch

    import microkimi_b200 as mk
    torch.cuda.set_device(0)
    ctx = mk.Context(0)
    mk.Context._default = ctx
    ctx.use_torch_stream()
    return torch, mk, ctx, torch.device("cuda", 0)


def run_case_mxfp4(args):
    torch, mk, ctx, dev = _side_ctx()
    print(json.dumps({"case": "mxfp4_gemv", **measure_mxfp4_gemv(torch, mk, ctx, dev, args.rows, args.cols, args.batch, args.copies,
                                                                 args.steps, args.warmup, args.act, args.graph)}), flush=True)


def run_case_moe(args):
    torch, mk, ctx, dev = _side_ctx()
    layers, gen = build_moe_layers(torch, mk, ctx, dev, args.experts, args.copies, act=args.moe_act)
    print(json.dumps({"case": "moe", "act": args.moe_act, **measure_moe(torch, mk, ctx, dev, layers, gen, args.batch, args.steps, args.warmup, args.graph)}),
          flush=True)


def run_case_moe_ep(args):
    import torch
    import torch.distributed as dist

    import microkimi_b200 as mk
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), rank=rank, world_size=world)
    dev = torch.device("cuda", local)
    ctx = mk.Context(local)
    mk.Context._default = ctx
    ctx.use_torch_stream()
    res = measure_moe_ep(torch, dist, mk, ctx, dev, world, rank, args.experts, (args.batch,), args.steps, args.warmup,
                         args.collective, args.copies)
    if rank == 0:
        print(json.dumps({"case": "moe_ep", "n_gpus": world, **res}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def run_case_kda(args):
    """Side workload: the KDA decode step (conv + SiLU, head norms, gate, recurrence, gated RMS) of `--heads`
    heads of width 128, `copies` layers in rotation (each layer's state S is heads x 64 KB); one launch per step."""
    torch, mk, ctx, dev = _side_ctx()
    if args.kda_smem:
        ctx.set_option("kda_smem", 1)
    H, D = args.heads, 128
    proj = H * D
    rng = np.random.default_rng(5)
    layers = []
    for _ in range(args.copies):
        cw = [(rng.standard_normal((proj, 4)) * 0.5).astype(np.float32) for _ in range(3)]
        layers.append(mk.KdaLayer(H, D, *cw, np.log(rng.uniform(1, 16, D)).astype(np.float32),
                                  (rng.standard_normal(proj) * 0.3).astype(np.float32), np.ones(D, np.float32), ctx=ctx))
    gen = torch.Generator(device=dev)
    gen.manual_seed(9)
    ins = [torch.randn(n, dtype=torch.float32, device=dev, generator=gen) for n in (proj, proj, proj, proj, H, proj)]
    ms_call = _timed(torch, lambda i: layers[i % args.copies].step(*ins), args.steps, args.warmup)
    # one launch per call: the loop above is bound by the host's call overhead, so the kernel itself is timed
    # by the library's event pairs around each launch
    ctx.prof_enable(True)
    _timed(torch, lambda i: layers[i % args.copies].step(*ins), args.steps, 0)
    n_k, ms_k = ctx.prof_read("other")
    ctx.prof_enable(False)
    ms = ms_k / max(n_k, 1)
    alg = H * D * D * 8 + 10 * proj * 4
    print(json.dumps({"case": "kda_step", "form": "shared memory" if args.kda_smem else "registers", "heads": H, "dim": D,
                      "copies": args.copies, "kernel_us": ms * 1e3, "call_us_host_loop": ms_call * 1e3, "algorithmic_bytes": alg,
                      "status_word": ctx.status_word(), "roofline": _roof(alg, ms, "latency-bound: one CTA per head")}), flush=True)


def run_case_decode(args):
    """The whole-token decode alone (one GPU, or under torchrun expert-parallel over the ranks)."""
    import torch

    import microkimi_b200 as mk
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29534")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), rank=rank, world_size=world)
    res = measure_decode(torch, mk, torch.device("cuda", local), local, world, rank, dist, n_new=args.decode_steps,
                         cpu_tokens=0 if args.no_cpu else 8, profile_prefill=args.profile_prefill)
    if rank == 0:
        print(json.dumps({"case": "decode", "n_gpus": world, **res}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_case_mla(args):
    torch, mk, ctx, dev = _side_ctx()
    print(json.dumps({"case": "mla", **measure_mla(torch, mk, ctx, dev, args.layout, args.ctx, args.batch, args.steps, args.warmup)}),
          flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="lm_head", choices=["lm_head", "mxfp4_gemv", "moe", "moe_ep", "mla", "kda", "decode"],
                    help="lm_head is the benchmark proper; the others run one of the side workloads alone")
    ap.add_argument("--rows", type=int, default=7168)
    ap.add_argument("--cols", type=int, default=2048)
    ap.add_argument("--copies", type=int, default=1)
    ap.add_argument("--act", default="q8", choices=["q8", "q8x2"])
    ap.add_argument("--experts", type=int, default=384)
    ap.add_argument("--moe-act", default="q8", choices=["q8", "fp4x6"], help="--case moe: fp4x6 = block-scaled tcgen05 experts for calls of >= 4 rows")
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=4, help="--case kda: KDA heads of width 128")
    ap.add_argument("--kda-smem", action="store_true", help="--case kda: the shared-memory form of the step kernel (default at width 128: registers)")
    ap.add_argument("--layout", default="absorbed", choices=["absorbed", "per_head"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps each; the value is their median")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the side workloads that follow the headline measurement")
    ap.add_argument("--decode-steps", type=int, default=256, help="--case decode: greedy steps after the prompt")
    ap.add_argument("--profile-prefill", action="store_true",
                    help="--case decode: cudaProfilerStart / Stop around the timed prefill (for a profiler that starts with profiling off)")
    ap.add_argument("--graph", action="store_true", help="--case mxfp4_gemv / moe: also time the ring of calls as one CUDA graph")
    ap.add_argument("--collective", default="peer", choices=["peer", "nccl"],
                    help="N > 1: logits by one peer-memory exchange kernel after the matvec (default) or by an NCCL all-gather")
    ap.add_argument("--token-only", action="store_true",
                    help="N > 1: the timed step is the token-only step of greedy decode (the ranks exchange (maximum, index) pairs, the logits "
                         "stay sharded); default: the complete logits on every rank.  The other form is timed beside it either way")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    if args.impl == "reference":
        run_reference(args)
    elif args.case == "mxfp4_gemv":
        run_case_mxfp4(args)
    elif args.case == "moe":
        run_case_moe(args)
    elif args.case == "moe_ep":
        run_case_moe_ep(args)
    elif args.case == "mla":
        run_case_mla(args)
    elif args.case == "kda":
        run_case_kda(args)
    elif args.case == "decode":
        run_case_decode(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
