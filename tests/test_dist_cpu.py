"""CPU (gloo, world_size 2 and 3) tests of the multi-GPU host logic: the vocab-sharded
logits gather and the expert-parallel token exchange must reproduce the single-rank
result exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from microkimi_b200 import dist as mkd


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _fake_expert(rows, pair_row, pair_expert, pair_weight):
    """Deterministic stand-in for the resident-experts kernel: depends on row, expert id and weight."""
    e = pair_expert.to(torch.float32)[:, None]
    return (rows[pair_row.long()] * (e + 1.0)).sin() * pair_weight[:, None] + e


def _combine(outs, n, slots):
    o = torch.zeros((n, outs.shape[1]), dtype=outs.dtype)
    v = outs.view(n, slots, -1)
    for s in range(slots):          # fixed slot order
        o = o + v[:, s]
    return o


def _worker(rank, world, port, n_tokens, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(123)
        n_experts, k, d, vocab = 12, 3, 16, 50
        x = torch.randn((n_tokens, d), generator=g)
        ids = torch.stack([torch.randperm(n_experts, generator=g)[:k] for _ in range(n_tokens)]).to(torch.int32)
        w = torch.rand((n_tokens, k), generator=g)
        lo, hi = mkd.shard_tokens(n_tokens, world, rank)
        elo, ehi = mkd.local_expert_range(n_experts, world, rank)

        def experts_here(rows, pr, pe, pw):
            ok = ((pe >= elo) & (pe < ehi)) | (pe == n_experts)
            assert bool(ok.all()), "a pair reached a rank that does not own its expert"
            return _fake_expert(rows, pr, pe, pw)

        out = mkd.ep_moe_forward(x[lo:hi], ids[lo:hi], w[lo:hi], n_experts, experts_here, _combine)
        # single-rank reference of the same rows
        slots = k + 1
        pe = torch.cat([ids, torch.full((n_tokens, 1), n_experts, dtype=torch.int32)], 1).reshape(-1)
        pw = torch.cat([w, torch.ones((n_tokens, 1))], 1).reshape(-1)
        pr = torch.arange(n_tokens, dtype=torch.int32).repeat_interleave(slots)
        ref = _combine(_fake_expert(x, pr, pe, pw), n_tokens, slots)
        ok_moe = torch.equal(out, ref[lo:hi])

        # vocab-sharded logits
        full = torch.randn((3, vocab), generator=g)
        vlo, vhi = mkd.vocab_shard(vocab, world, rank)
        got = mkd.gather_logits(full[:, vlo:vhi].contiguous(), vocab)
        ok_gather = torch.equal(got, full)
        tie = full.clone()
        tie[0, 7] = tie[0, 31] = 100.0
        ok_argmax = mkd.greedy_token(tie)[0].item() == 7 and torch.equal(mkd.greedy_token(full).long(), full.argmax(1))
        ret[rank] = (ok_moe, ok_gather, ok_argmax)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_tokens", [(2, 8), (2, 1), (3, 7)])
def test_expert_parallel_exchange_and_logits_gather(world, n_tokens):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), n_tokens, ret), nprocs=world, join=True)
    assert len(ret) == world
    for r in range(world):
        assert ret[r] == (True, True, True), f"rank {r}: {ret[r]}"


def test_partitions_cover_everything():
    for world in (1, 2, 3, 4, 8):
        for total in (1, 7, 384, 163840):
            cuts = [mkd.vocab_shard(total, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == total
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
        e = torch.arange(384)
        own = mkd.expert_owner(e, 384, world)
        for r in range(world):
            lo, hi = mkd.local_expert_range(384, world, r)
            assert bool((own[lo:hi] == r).all())


def _coverage_worker(rank, world, port, maps, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        try:
            mkd.check_expert_coverage(maps[rank])
            ret[rank] = "ok"
        except ValueError as exc:
            ret[rank] = str(exc)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("maps,expect", [
    ([[True, True, False, False], [False, False, True, True]], "ok"),
    ([[True, True, False, False], [False, False, False, True]], "resident nowhere [2]"),
    ([[True, True, True, False], [False, False, True, True]], "on several ranks [2]"),
])
def test_expert_partition_must_cover_every_routed_expert_once(maps, expect):
    """A mis-partitioned expert-parallel layer is refused on every rank when the peer exchange is set up."""
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_coverage_worker, args=(2, port, maps, ret), nprocs=2, join=True)
    for r in range(2):
        assert expect in ret[r], ret[r]
