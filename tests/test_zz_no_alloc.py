"""The entry point that allocates nothing (mk_matvec_mxfp4_noalloc_dev).

It is for hosts that cannot call cudaMalloc once they are running - all device memory
already given to their own pools, or no tolerance for the synchronization an allocation
implies.  Its scratch is one fixed array shared by every call, so the test runs two calls
in a row with different inputs and shapes of batch and checks each against the regular
entry point (same kernels, so the bits must be equal).  Collected last on purpose.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_noalloc_matvec_matches_regular_entry_point_twice_in_a_row():
    import torch

    import microkimi_b200 as mk
    ctx = mk.Context.default()
    ctx.use_torch_stream()
    dev = torch.device("cuda", ctx.device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    rows, cols = 1000, 2048 + 32          # ragged: rows % 16 != 0, blocks % 4 != 0 (padding path)
    p = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device=dev, generator=gen)
    s = torch.randint(110, 130, (rows, cols // 32), dtype=torch.uint8, device=dev, generator=gen)
    w = mk.MxFp4Weight(p, s, rows, cols)
    x1 = torch.randn((5, cols), dtype=torch.float32, device=dev, generator=gen)
    x2 = torch.randn((1, cols), dtype=torch.float32, device=dev, generator=gen) * 3.0
    for x in (x1, x2, x1[:2].contiguous()):            # back to back, the second call sees the first one's scratch
        got = w.matvec_noalloc(x)
        want = w.matvec(x)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
    got = w.matvec_noalloc(x2, act="q8x2")
    assert torch.equal(got, w.matvec(x2, act="q8x2"))
    got = w.matvec_noalloc(x1, strict=True)
    assert torch.equal(got, w.matvec(x1, strict=True))
    # the call itself allocates nothing: with the result buffer made beforehand, neither the driver's free
    # memory nor torch's allocator moves across two calls through the C ABI
    import ctypes as C
    y = torch.empty((5, rows), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    free0, alloc0, reserved0 = torch.cuda.mem_get_info(dev)[0], torch.cuda.memory_allocated(dev), torch.cuda.memory_reserved(dev)
    for x in (x1, x2):
        mk.lib.check(ctx._L.mk_matvec_mxfp4_noalloc_dev(ctx._h, w._h, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()),
                                                        x.shape[0], mk.lib.MK_ACT_Q8))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(dev)[0] == free0
    assert torch.cuda.memory_allocated(dev) == alloc0 and torch.cuda.memory_reserved(dev) == reserved0
    assert torch.equal(y[:1], w.matvec(x2))
    # beyond the fixed scratch: a clear error, nothing launched
    with pytest.raises(mk.lib.MkError) as e:
        w.matvec_noalloc(torch.zeros((9, cols), dtype=torch.float32, device=dev))
    assert e.value.code == -1 and "fixed scratch" in str(e.value)
    wide = mk.MxFp4Weight(torch.zeros((16, 16416 // 2), dtype=torch.uint8, device=dev),
                          torch.zeros((16, 16416 // 32), dtype=torch.uint8, device=dev), 16, 16416)
    with pytest.raises(mk.lib.MkError):
        wide.matvec_noalloc(torch.zeros((1, 16416), dtype=torch.float32, device=dev))
    assert ctx.status_word() == 0
