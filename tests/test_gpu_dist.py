"""Multi-GPU tests (NCCL, one process per GPU): the vocab-sharded lm_head and the
expert-parallel MoE must give the bits a single GPU gives.  Skipped with fewer than 2 GPUs."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    import microkimi_b200 as mk
    from microkimi_b200 import dist as mkd
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        ctx = mk.Context(rank)
        mk.Context._default = ctx
        ctx.use_torch_stream()
        g = torch.Generator(device="cpu").manual_seed(7)
        # ---- lm_head, vocab-sharded
        vocab, d, batch = 4096, 512, 3
        wf = (torch.randn((vocab, d), generator=g) * 0.02).numpy()
        x = torch.randn((batch, d), generator=g)
        lo, hi = mkd.vocab_shard(vocab, world, rank)
        head = mk.Q8Head.from_f32(np.ascontiguousarray(wf[lo:hi]), hi - lo, d, ctx=ctx)
        full = mkd.gather_logits(head.matvec(x.to(dev)), vocab)
        single = mk.Q8Head.from_f32(wf, vocab, d, ctx=ctx).matvec(x.to(dev))
        torch.cuda.synchronize()
        ok_head = torch.equal(full, single) and torch.equal(mkd.greedy_token(full).cpu().long(), single.argmax(1).cpu())
        # ---- the same head with the logits stored straight into every rank's gather buffer (peer memory),
        # several steps in a row (the buffers alternate by step parity), batch 1 and 2
        fused = mkd.FusedVocabHead(head, vocab, max_batch=2)
        xd = x.to(dev)
        for step in range(5):
            nb = 1 + step % 2
            xin = (xd[:nb] * float(step + 1)).contiguous()
            ptr, am = fused.matvec(xin)
            got = fused.logits_tensor(ptr, nb)
            want = mk.Q8Head.from_f32(wf, vocab, d, ctx=ctx).matvec(xin)
            torch.cuda.synchronize()
            ok_head = ok_head and torch.equal(got, want) and torch.equal(am.cpu().long(), want.argmax(1).cpu())
            # the token-only step in between (only the ranks' (maximum, index) pairs cross): the same token on every rank,
            # this rank's rows where the call says they are
            xin2 = (xin * -0.75).contiguous()
            ptr2, am2 = fused.matvec(xin2, want_logits=False)
            mine2 = fused.local_rows_tensor(ptr2, nb)
            want2 = mk.Q8Head.from_f32(wf, vocab, d, ctx=ctx).matvec(xin2)
            torch.cuda.synchronize()
            ok_head = ok_head and torch.equal(mine2, want2[:, lo:hi]) and torch.equal(am2.cpu().long(), want2.argmax(1).cpu())
        ok_head = ok_head and ctx.status_word() == 0
        dist.barrier()
        fused.free()
        # ---- MoE, expert-parallel, tokens sharded
        E, k, dm, inter, n_tok = 16, 4, 256, 128, 11
        gw = (torch.randn((E, dm), generator=g) * 0.02).numpy()

        def rw(rows, cols):
            p = torch.randint(0, 256, (rows, cols // 2), generator=g, dtype=torch.uint8).numpy()
            s = torch.randint(118, 124, (rows, cols // 32), generator=g, dtype=torch.uint8).numpy()
            return mk.MxFp4Weight(p, s, rows, cols, ctx=ctx)
        experts = [(rw(inter, dm), rw(dm, inter), rw(inter, dm)) for _ in range(E + 1)]
        xt = torch.randn((n_tok, dm), generator=g).to(dev)
        whole = mk.MoeLayer(gw, None, experts[:-1], experts[-1], k, ctx=ctx)
        ref = whole.moe_forward(xt)
        elo, ehi = mkd.local_expert_range(E, world, rank)
        mine = [experts[e] if elo <= e < ehi else None for e in range(E)]
        ep = mkd.EpMoeLayer(mk.MoeLayer(gw, None, mine, experts[-1], k, ctx=ctx))
        tlo, thi = mkd.shard_tokens(n_tok, world, rank)
        out = ep.forward(xt[tlo:thi].contiguous())
        torch.cuda.synchronize()
        ok_moe = torch.equal(out, ref[tlo:thi]) and ctx.status_word() == 0
        # ---- the decode form: rows replicated, outputs exchanged by peer-memory stores; several calls in a
        # row (the table alternates by step parity) and several row counts
        pep = mkd.PeerEpMoeLayer(mk.MoeLayer(gw, None, mine, experts[-1], k, ctx=ctx), max_tokens=16)
        for step, nrows in enumerate((1, 2, 5, 11, 1, 3)):
            xin = (xt[:nrows] * float(1 + step % 3)).contiguous()
            got = pep.forward(xin)
            want = whole.moe_forward(xin)
            torch.cuda.synchronize()
            ok_moe = ok_moe and torch.equal(got, want)
        ok_moe = ok_moe and ctx.status_word() == 0
        dist.barrier()
        pep.free()
        ret[rank] = (bool(ok_head), bool(ok_moe))
    finally:
        dist.destroy_process_group()


def _decode_worker(rank, world, port, path, ret):
    import torch.distributed as dist

    import microkimi_b200 as mk
    from microkimi_b200 import model as M
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = torch.device("cuda", rank)
        ctx = mk.Context(rank)
        stream = torch.cuda.Stream(device=dev)           # a real stream: the token can be recorded
        prompt = np.array([5, 900, 17, 1203, 44], np.int32)
        with torch.cuda.stream(stream):
            ctx.use_torch_stream()
            whole = M.Model(path, 40, use_graph=False, ctx=ctx)          # one GPU, launched kernel by kernel
            want = whole.generate(prompt, 14)
            split = M.Model(path, 40, use_graph=True, rank=rank, world=world, ctx=ctx)
            split.connect()
            got = split.generate(prompt, 14)             # eager token, one recording per exchange parity, replays
            torch.cuda.synchronize()
            ret[rank] = (bool(np.array_equal(got, want)), int(ctx.status_word()))
            dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_decode_with_experts_and_vocabulary_split_over_the_ranks_equals_one_gpu(world, tmp_path):
    """The whole decode token with the routed experts block-partitioned over the ranks and the lm_head rows sharded,
    replayed as a CUDA graph (the exchange kernels keep their step numbers on the device): the greedy continuation of a
    prompt is the one a single GPU produces (every partial result is bit-identical, so the token ids are)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    from oracle import oracle as O
    path = str(tmp_path / "split.bin")
    O.build_bin(path, O.Config.microkimi(n_layers=5, vocab=2048, n_experts=32, top_k=4, attn_res_block=2))
    ret = mp.Manager().dict()
    mp.spawn(_decode_worker, args=(world, _free_port(), path, ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r] == (True, 0), f"rank {r}: {ret[r]}"


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_lm_head_and_expert_parallel_moe_match_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r] == (True, True), f"rank {r}: {ret[r]}"


def test_second_context_on_another_gpu_of_the_same_process():
    """Kernels that opt in to more than 48 KB of dynamic shared memory must do so on every device a
    process uses: the MoE router, both MLA layouts, the KDA step and the f32 matvec run on GPU 1 after
    GPU 0 has used them, and give the same bits there."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import microkimi_b200 as mk
    rng = np.random.default_rng(3)
    E, k, d, inter = 16, 4, 256, 128
    gw = (rng.standard_normal((E, d)) * 0.02).astype(np.float32)
    blobs = [[(rng.integers(0, 256, (r, c // 2), dtype=np.uint8), rng.integers(118, 124, (r, c // 32), dtype=np.uint8), r, c)
              for r, c in ((inter, d), (d, inter), (inter, d))] for _ in range(E + 1)]
    x = rng.standard_normal((3, d)).astype(np.float32)
    rows = rng.standard_normal((300, 576)).astype(np.float32)
    q = rng.standard_normal((64, 576)).astype(np.float32)
    kk = rng.standard_normal((40, 8, 192)).astype(np.float32)
    kk[:, 1:, 128:] = kk[:, :1, 128:]
    vv = rng.standard_normal((40, 8, 128)).astype(np.float32)
    qp = rng.standard_normal((8, 192)).astype(np.float32)
    fw = (rng.standard_normal((96, 512)) * 0.05).astype(np.float32)
    fx = rng.standard_normal(512).astype(np.float32)
    kp = 2 * 96
    kw = [(rng.standard_normal((kp, 4)) * 0.5).astype(np.float32) for _ in range(3)]
    kw += [np.log(rng.uniform(1, 16, 96)).astype(np.float32), (rng.standard_normal(kp) * 0.3).astype(np.float32), np.ones(96, np.float32)]
    kin = [rng.standard_normal(n).astype(np.float32) for n in (kp, kp, kp, kp, 2, kp)]
    outs = []
    for device in (0, 1):
        ctx = mk.Context(device)
        with torch.cuda.device(device):
            ex = [tuple(mk.MxFp4Weight(*b, ctx=ctx) for b in tri) for tri in blobs]
            layer = mk.MoeLayer(gw, None, ex[:-1], ex[-1], k, ctx=ctx)
            o_moe = layer.moe_forward(x)
            ca = mk.MlaCache(64, 576, 0, 512, 300, layout="absorbed", ctx=ctx)
            ca.push(rows)
            o_abs = ca.mla_attn_flash_q8_mqa(q, 299, 1.0 / np.sqrt(192.0))
            cp = mk.MlaCache(8, 128, 64, 128, 40, ctx=ctx)
            cp.push(kk, vv)
            o_ph = cp.mla_attn_flash_q8_mqa(qp, 39, 1.0 / np.sqrt(192.0))
            o_f32 = mk.matvec(fw, 96, 512, fx, ctx=ctx)
            kda = mk.KdaLayer(2, 96, *kw, ctx=ctx)                       # width 96: the shared-memory form of the step
            o_kda = kda.step(*[torch.from_numpy(a).to(f"cuda:{device}") for a in kin]).cpu().numpy()
            assert ctx.status_word() == 0
            outs.append((o_moe, o_abs, o_ph, o_f32, o_kda))
            layer.free(); ca.free(); cp.free(); kda.free()
        ctx.close()
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
