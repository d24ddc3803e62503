"""Failure detection on the GPU without a fault: a rank that never joined.

The multi-GPU exchange kernels wait for the other ranks' flags with a bounded poll loop (about half a second);
when it runs out they record MK_ERR_TIMEOUT in the context's status word and return, so the host reads a status
and the context stays usable.  Here one process plays rank 0 of a world of 2 whose rank 1 never joined: its
buffer handle is all zeros, which mk_*_connect turns into a local stand-in buffer that nobody signals.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture()
def own_ctx():
    """A context of its own, so that the status word of the shared default context stays clean."""
    import microkimi_b200 as mk
    ctx = mk.Context(0)
    ctx.use_torch_stream()
    yield mk, ctx
    ctx.close()


def test_lm_head_gather_with_absent_rank_reports_timeout(own_ctx):
    import torch
    from microkimi_b200 import lib as L
    mk, ctx = own_ctx
    rng = np.random.default_rng(1)
    rows, cols, vocab = 256, 128, 512
    head = mk.Q8Head.from_f32((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32), rows, cols, ctx=ctx)
    g, handles = C.c_void_p(), (C.c_uint8 * 128)()
    mine = (C.c_uint8 * 64)()
    L.check(ctx._L.mk_gather_create(ctx._h, 0, 2, vocab, 1, C.byref(g), mine))
    handles[0:64] = mine[:]                      # rank 1's handle stays all zeros: it never joined
    L.check(ctx._L.mk_gather_connect(ctx._h, g, handles))
    x = torch.from_numpy(rng.standard_normal((1, cols)).astype(np.float32)).cuda()
    am = torch.zeros(1, dtype=torch.int32, device="cuda")
    ptr = C.c_void_p()
    try:
        L.check(ctx._L.mk_matvec_q8_gather_dev(ctx._h, head._h, g, C.c_void_p(x.data_ptr()), 1, 0, C.byref(ptr), C.c_void_p(am.data_ptr())))
        torch.cuda.synchronize()                 # returns: the wait gave up by itself
        assert ctx.status_word() == L.MK_ERR_TIMEOUT
        assert ctx.status_word() == 0            # reading clears the word
        # the context is usable afterwards, and this rank's own rows are in its buffer
        y = head.matvec(x)
        got = torch.empty((1, vocab), dtype=torch.float32, device="cuda")
        L.check(ctx._L.mk_memcpy_dev(ctx._h, C.c_void_p(got.data_ptr()), ptr, vocab * 4))
        torch.cuda.synchronize()
        assert torch.equal(got[:, :rows], y)
        assert ctx.status_word() == 0
    finally:
        L.check(ctx._L.mk_gather_free(ctx._h, g))
        head.free()


def test_expert_parallel_moe_with_absent_rank_reports_timeout(own_ctx):
    import torch
    from microkimi_b200 import lib as L
    from oracle import oracle as O
    mk, ctx = own_ctx
    rng = np.random.default_rng(2)
    E, k, d, inter = 8, 2, 128, 64
    gate_w = (rng.standard_normal((E, d)) * 0.02).astype(np.float32)

    def tri():
        out = []
        for r, c in ((inter, d), (d, inter), (inter, d)):
            p, s = O.mxfp4_quantize((rng.standard_normal((r, c)) * 0.02).astype(np.float32))
            out.append(mk.MxFp4Weight(p, s, r, c, ctx=ctx))
        return tuple(out)

    experts = [tri() if e < E // 2 else None for e in range(E)]      # rank 0 of 2 holds the first half
    layer = mk.MoeLayer(gate_w, None, experts, tri(), k, ctx=ctx)
    ep, handles, mine = C.c_void_p(), (C.c_uint8 * 128)(), (C.c_uint8 * 64)()
    L.check(ctx._L.mk_moe_ep_create(ctx._h, layer._h, 0, 2, 16, C.byref(ep), mine))
    handles[0:64] = mine[:]
    L.check(ctx._L.mk_moe_ep_connect(ctx._h, ep, handles))
    x = torch.from_numpy(rng.standard_normal((3, d)).astype(np.float32)).cuda()
    out = torch.empty_like(x)
    try:
        L.check(ctx._L.mk_moe_forward_ep_dev(ctx._h, layer._h, ep, C.c_void_p(x.data_ptr()), 3, C.c_void_p(out.data_ptr()), None, None))
        torch.cuda.synchronize()
        assert ctx.status_word() == L.MK_ERR_TIMEOUT
        assert ctx.status_word() == 0
    finally:
        L.check(ctx._L.mk_moe_ep_free(ctx._h, ep))
