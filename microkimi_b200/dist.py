"""Multi-GPU host logic for the two paths that shard: the vocab-sharded q8_0
lm_head (logits all-gather) and expert-parallel MoE (all-to-all token dispatch).

One process per GPU, `torch.distributed` for the plumbing (NCCL on GPUs, gloo in
the CPU tests).  The reference engine is single-process (no rank concept
anywhere), so there is no reference code for this file; what it must preserve is
the single-GPU RESULT: the gathered logits and the combined MoE output are the
bits a single GPU would produce, because every (row, expert) pair is computed by
the same kernels and combined in slot order on the token's home rank.

The functions take plain callables for the per-rank compute so that the exchange
logic can be exercised on CPU ranks.
"""
import torch
import torch.distributed as dist


# ---------------------------------------------------------------- vocab-sharded lm_head
def vocab_shard(vocab, world, rank):
    """Rows [lo, hi) of the lm_head owned by `rank` (block partition, remainder to the first ranks)."""
    base, rem = divmod(vocab, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def gather_logits(local_logits, vocab, group=None):
    """local_logits [batch, rows_of_this_rank] -> full logits [batch, vocab] on every rank."""
    world = dist.get_world_size(group)
    batch = local_logits.shape[0]
    sizes = [vocab_shard(vocab, world, r) for r in range(world)]
    if all(hi - lo == sizes[0][1] - sizes[0][0] for lo, hi in sizes):
        rows = sizes[0][1] - sizes[0][0]
        if batch == 1:
            full = torch.empty((1, vocab), dtype=local_logits.dtype, device=local_logits.device)
            dist.all_gather_into_tensor(full.view(-1), local_logits.contiguous().view(-1), group=group)
            return full
        stacked = torch.empty((world, batch, rows), dtype=local_logits.dtype, device=local_logits.device)
        dist.all_gather_into_tensor(stacked.view(-1), local_logits.contiguous().view(-1), group=group)
        return stacked.permute(1, 0, 2).reshape(batch, vocab)
    # uneven shards: pad every shard to the widest one, gather, cut the padding off
    widest = max(hi - lo for lo, hi in sizes)
    padded = torch.zeros((batch, widest), dtype=local_logits.dtype, device=local_logits.device)
    padded[:, :local_logits.shape[1]] = local_logits
    stacked = torch.empty((world, batch, widest), dtype=local_logits.dtype, device=local_logits.device)
    dist.all_gather_into_tensor(stacked.view(-1), padded.view(-1), group=group)
    return torch.cat([stacked[r, :, :hi - lo] for r, (lo, hi) in enumerate(sizes)], dim=1)


def greedy_token(full_logits):
    """First index of the maximum per row (the engine's greedy pick, src/model.rs:3277-3290)."""
    mx = full_logits.max(dim=1, keepdim=True).values
    idx = torch.arange(full_logits.shape[1], device=full_logits.device).expand_as(full_logits)
    big = torch.full_like(idx, full_logits.shape[1])
    return torch.where(full_logits == mx, idx, big).min(dim=1).values.to(torch.int32)


class FusedVocabHead:
    """Vocabulary-sharded q8_0 lm_head whose logits reach every rank by peer-memory stores over NVLink
    (one exchange kernel per token after the matvec: push, signal, bounded wait, token pick) - no
    collective library call per token.

    `head` is this rank's ops.Q8Head over rows vocab_shard(vocab, world, rank).  Construction
    exchanges the buffer handles once (all_gather over the process group)."""

    def __init__(self, head, vocab, group=None, max_batch=1):
        import ctypes as C
        from . import lib as _l
        self.head, self.vocab, self.ctx = head, int(vocab), head.ctx
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.row0, hi = vocab_shard(vocab, self.world, self.rank)
        assert hi - self.row0 == head.rows, "the head must hold exactly this rank's vocabulary rows"
        self.max_batch = int(max_batch)
        L = self.ctx._L
        h = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        _l.check(L.mk_gather_create(self.ctx._h, self.rank, self.world, self.vocab, self.max_batch, C.byref(h), handle))
        self._h = h
        dev = torch.device("cuda", self.ctx.device)
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
        allh = torch.empty((self.world, 64), dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allh.view(-1), mine, group=group)
        buf = (C.c_uint8 * (64 * self.world)).from_buffer_copy(bytes(allh.cpu().numpy().tobytes()))
        # every rank learns whether all ranks could open all buffers, so that all of them raise or none does
        ok = torch.ones(1, dtype=torch.int32, device=dev)
        err = None
        try:
            _l.check(L.mk_gather_connect(self.ctx._h, self._h, buf))
        except Exception as exc:
            err = exc
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            self.free()
            raise RuntimeError(f"peer gather buffers could not be connected on every rank ({err})")
        self._am = torch.empty((self.max_batch,), dtype=torch.int32, device=dev)

    def matvec(self, x, want_argmax=True, head=None, want_logits=True):
        """x [batch, cols] (torch CUDA, identical on every rank) -> (device address of the complete logits
        [batch, vocab] in this rank's gather buffer, valid until the call after next; argmax int32 [batch]).
        `head`: another Q8Head over the same rows (every rank must pass its counterpart).
        want_logits=False: the token-only step of greedy decode - the ranks exchange their (maximum, index)
        pairs instead of the rows; returns (device address of THIS rank's rows of the logits, [batch] rows `vocab`
        floats apart, argmax)."""
        import ctypes as C
        from . import lib as _l
        head = head or self.head
        assert head.rows == self.head.rows and head.cols == self.head.cols
        xs = x.reshape(-1, self.head.cols)
        assert xs.dtype == torch.float32 and xs.is_contiguous() and xs.shape[0] <= self.max_batch
        self.ctx._follow_torch()
        batch = xs.shape[0]
        ptr = C.c_void_p()
        if want_logits:
            _l.check(self.ctx._L.mk_matvec_q8_gather_dev(self.ctx._h, head._h, self._h, C.c_void_p(xs.data_ptr()), batch, self.row0,
                                                        C.byref(ptr), C.c_void_p(self._am.data_ptr()) if want_argmax else None))
        else:
            assert want_argmax, "the token-only step returns the token"
            _l.check(self.ctx._L.mk_matvec_q8_gather_token_dev(self.ctx._h, head._h, self._h, C.c_void_p(xs.data_ptr()), batch, self.row0,
                                                              C.byref(ptr), C.c_void_p(self._am.data_ptr())))
        self._last_ptr = ptr.value
        return ptr.value, (self._am[:batch] if want_argmax else None)

    def local_rows_tensor(self, ptr, batch):
        """Copies this rank's rows behind the pointer of a token-only step into a fresh torch tensor [batch, rows]."""
        import ctypes as C
        from . import lib as _l
        out = torch.empty((batch, self.head.rows), dtype=torch.float32, device=torch.device("cuda", self.ctx.device))
        for b in range(batch):
            _l.check(self.ctx._L.mk_memcpy_dev(self.ctx._h, C.c_void_p(out[b].data_ptr()), C.c_void_p(ptr + b * self.vocab * 4), self.head.rows * 4))
        return out

    def logits_tensor(self, ptr, batch):
        """Copies the complete logits behind `ptr` into a fresh torch tensor [batch, vocab]."""
        import ctypes as C
        from . import lib as _l
        out = torch.empty((batch, self.vocab), dtype=torch.float32, device=torch.device("cuda", self.ctx.device))
        _l.check(self.ctx._L.mk_memcpy_dev(self.ctx._h, C.c_void_p(out.data_ptr()), C.c_void_p(ptr), batch * self.vocab * 4))
        return out

    def free(self):
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._L.mk_gather_free(self.ctx._h, self._h)
        self._h = None


def check_expert_coverage(resident, group=None, device=None):
    """`resident`: bool per routed expert, True where this rank holds the expert.  All-gathers the maps and raises on every
    rank unless each routed expert is resident on exactly one rank: an expert nobody holds would leave its (token, slot)
    row of the exchange table unwritten and the combine would sum a stale row."""
    mine = torch.as_tensor(resident, dtype=torch.uint8, device=device).contiguous().view(-1)
    world = dist.get_world_size(group)
    allm = torch.empty((world, mine.numel()), dtype=torch.uint8, device=mine.device)
    dist.all_gather_into_tensor(allm.view(-1), mine, group=group)
    count = allm.to(torch.int32).sum(0).cpu()
    missing = torch.nonzero(count == 0).view(-1).tolist()
    doubled = torch.nonzero(count > 1).view(-1).tolist()
    if missing or doubled:
        raise ValueError(f"expert partition is not a cover: resident nowhere {missing[:8]}, on several ranks {doubled[:8]}")


class PeerEpMoeLayer:
    """Expert-parallel MoE for decode without a collective library call per layer: token rows are
    replicated on every rank (<= 16), each rank runs the pairs of its resident experts and the
    output rows travel by peer-memory stores (mk_moe_forward_ep_dev).  `layer` is an ops.MoeLayer
    built with None for the routed experts that live on other ranks (local_expert_range) and with
    the shared expert on every rank."""

    def __init__(self, layer, group=None, max_tokens=16):
        import ctypes as C
        from . import lib as _l
        self.layer, self.ctx = layer, layer.ctx
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        check_expert_coverage(layer.resident, group, torch.device("cuda", self.ctx.device))
        L = self.ctx._L
        h = C.c_void_p()
        handle = (C.c_uint8 * 64)()
        _l.check(L.mk_moe_ep_create(self.ctx._h, layer._h, self.rank, self.world, int(max_tokens), C.byref(h), handle))
        self._h = h
        dev = torch.device("cuda", self.ctx.device)
        mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
        allh = torch.empty((self.world, 64), dtype=torch.uint8, device=dev)
        dist.all_gather_into_tensor(allh.view(-1), mine, group=group)
        buf = (C.c_uint8 * (64 * self.world)).from_buffer_copy(bytes(allh.cpu().numpy().tobytes()))
        ok = torch.ones(1, dtype=torch.int32, device=dev)
        err = None
        try:
            _l.check(L.mk_moe_ep_connect(self.ctx._h, self._h, buf))
        except Exception as exc:
            err = exc
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            self.free()
            raise RuntimeError(f"peer exchange buffers could not be connected on every rank ({err})")

    def forward(self, x):
        """x [n, d] (torch CUDA, n <= max_tokens, the same rows on every rank) -> [n, d], the same on every rank."""
        import ctypes as C
        from . import lib as _l
        xs = x.reshape(-1, self.layer.dx)
        assert xs.dtype == torch.float32 and xs.is_contiguous()
        self.ctx._follow_torch()
        out = torch.empty_like(xs)
        _l.check(self.ctx._L.mk_moe_forward_ep_dev(self.ctx._h, self.layer._h, self._h, C.c_void_p(xs.data_ptr()), xs.shape[0],
                                                  C.c_void_p(out.data_ptr()), None, None))
        return out.reshape(x.shape)

    def free(self):
        if getattr(self, "_h", None) and getattr(self.ctx, "_h", None):
            self.ctx._L.mk_moe_ep_free(self.ctx._h, self._h)
        self._h = None


# ---------------------------------------------------------------- expert-parallel MoE
def expert_owner(expert, n_experts, world):
    """Block partition of the routed experts: expert e lives on rank e // (n_experts / world)."""
    per = n_experts // world
    return torch.clamp(expert // per, max=world - 1)


def local_expert_range(n_experts, world, rank):
    per = n_experts // world
    lo = rank * per
    return lo, (n_experts if rank == world - 1 else lo + per)


def ep_moe_forward(x, ids, weights, n_experts, experts_fn, combine_fn, group=None, shared_expert=True):
    """Expert-parallel MoE for the token rows this rank owns.

    x        [n, d]      the rank's own token rows (n may be 0)
    ids      [n, k] i32  routed expert ids in slot order (router is replicated, so every
    weights  [n, k] f32  rank computes the routing of its own tokens itself)
    experts_fn(rows [m, d], pair_row [m] i32, pair_expert [m] i32, pair_weight [m] f32) -> [m, d]
             runs the experts RESIDENT ON THIS RANK on explicit (row, expert, weight) pairs
    combine_fn(outs [n * slots, d], n, slots) -> [n, d]   slot-order sum
    The shared expert (id n_experts, weight 1) runs on the token's home rank.

    Exchange: one all-to-all of per-destination pair counts, one of the activation
    rows (+ expert ids and weights), one back with the expert outputs.  The payload
    lands in local memory before any kernel reads it.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n, d = x.shape
    k = ids.shape[1]
    slots = k + (1 if shared_expert else 0)
    dev = x.device

    pe = ids.to(torch.int64)
    pw = weights
    if shared_expert:
        pe = torch.cat([pe, torch.full((n, 1), n_experts, dtype=torch.int64, device=dev)], dim=1)
        pw = torch.cat([pw, torch.ones((n, 1), dtype=weights.dtype, device=dev)], dim=1)
    pe = pe.reshape(-1)                         # pair p = token * slots + slot
    pw = pw.reshape(-1)
    prow = torch.arange(n, device=dev).repeat_interleave(slots)
    dest = expert_owner(pe, n_experts, world)
    if shared_expert:
        dest = torch.where(pe == n_experts, torch.full_like(dest, rank), dest)

    order = torch.argsort(dest, stable=True)    # pairs grouped by destination rank
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    s_list, r_list = send_counts.tolist(), recv_counts.tolist()
    m = int(sum(r_list))

    send_rows = x[prow[order]].contiguous()
    send_meta = torch.stack([pe[order].to(torch.float64), pw[order].to(torch.float64)], dim=1).contiguous()
    recv_rows = torch.empty((m, d), dtype=x.dtype, device=dev)
    recv_meta = torch.empty((m, 2), dtype=torch.float64, device=dev)
    dist.all_to_all_single(recv_rows, send_rows, r_list, s_list, group=group)
    dist.all_to_all_single(recv_meta, send_meta, r_list, s_list, group=group)

    if m > 0:
        outs_here = experts_fn(recv_rows, torch.arange(m, dtype=torch.int32, device=dev),
                               recv_meta[:, 0].to(torch.int32), recv_meta[:, 1].to(torch.float32))
    else:
        outs_here = torch.empty((0, d), dtype=x.dtype, device=dev)

    back = torch.empty((n * slots, d), dtype=x.dtype, device=dev)
    dist.all_to_all_single(back, outs_here.contiguous(), s_list, r_list, group=group)
    outs = torch.empty_like(back)
    outs[order] = back                          # undo the grouping: outs[token * slots + slot]
    if n == 0:
        return torch.empty((0, d), dtype=x.dtype, device=dev)
    return combine_fn(outs, n, slots)


def shard_tokens(n_tokens, world, rank):
    """Token rows [lo, hi) whose home is `rank` (tokens are sharded, not replicated)."""
    base, rem = divmod(n_tokens, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class EpMoeLayer:
    """Expert-parallel MoE layer on this rank's GPU: the router is replicated, routed experts
    are block-partitioned over the ranks, the shared expert lives on every rank and serves
    the rank's own tokens.  `layer` is an ops.MoeLayer built with None for the experts that
    are not resident here."""

    def __init__(self, layer, group=None):
        self.layer, self.group = layer, group

    def forward(self, x_local):
        """x_local [n, d] (torch CUDA, the token rows whose home is this rank) -> [n, d]."""
        layer = self.layer
        if x_local.shape[0] > 0:
            ids, w = layer.route(x_local)
        else:
            ids = torch.empty((0, layer.top_k), dtype=torch.int32, device=x_local.device)
            w = torch.empty((0, layer.top_k), dtype=torch.float32, device=x_local.device)
        return ep_moe_forward(x_local, ids, w, layer.n_experts, layer.experts_dev,
                              lambda outs, n, slots: layer.combine_dev(outs, n, slots),
                              group=self.group, shared_expert=layer.has_shared)
