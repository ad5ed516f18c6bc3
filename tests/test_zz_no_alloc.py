"""The allocation-free routing-index entry point, called through its exported C symbol.

``fluxb_moe_index_build_static`` is for host programs that cannot allocate device memory
(everything already sits in their own pool, or cudaMalloc's device-wide synchronisation is not
acceptable in their request loop): it keeps its scratch in a fixed 1 MiB array inside the
library instead of taking a scratch buffer. Its results must equal those of
``fluxb_moe_index_build`` on the same input, also on the second of two calls in a row, since
the array is shared by all calls and keeps the previous call's contents. Collected last, so a
run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_ELEMS = 256 * 1024


def _call_static(lib, ce, E, topk):
    dev = ce.device
    n = ce.numel()
    outs = [torch.full((E,), -1, dtype=torch.int32, device=dev),
            torch.full((E + 1,), -1, dtype=torch.int32, device=dev),
            torch.full((n,), -1, dtype=torch.int32, device=dev),
            torch.full((n,), -1, dtype=torch.int32, device=dev),
            torch.full((n,), -1, dtype=torch.int32, device=dev)]
    fn = lib.fluxb_moe_index_build_static
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_void_p(ce.data_ptr()), ctypes.c_int64(n), ctypes.c_int(E), ctypes.c_int(topk),
            *[ctypes.c_void_p(t.data_ptr()) for t in outs],
            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    return rc, outs


def test_static_scratch_entry_matches_allocating_entry():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from tempname_new_b200 import _native
    from tempname_new_b200.ops.misc import moe_index_build
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(11)
    # two calls in a row with different sizes and expert counts: the second one runs on top of
    # whatever the first left in the shared array
    for tokens, topk, E in [(20000, 8, 64), (3000, 2, 16)]:
        ce = torch.randint(0, E, (tokens, topk), device=dev, generator=g, dtype=torch.int32)
        flat = ce.reshape(-1).contiguous()
        rc, got = _call_static(lib, flat, E, topk)
        assert rc == 0, lib.fluxb_last_error().decode()
        ref = moe_index_build(ce, E)
        torch.cuda.synchronize()
        names = ["splits", "offsets", "scatter_index", "gather_index", "topk_index"]
        for name, a, b in zip(names, got, ref):
            assert torch.equal(a.reshape(-1), b.reshape(-1)), name
        # and, independently of the other entry point, against the plain statement of the routing
        # tensors: counts per expert and the stable expert-sorted order
        order = torch.argsort(flat.long(), stable=True)
        scatter_ref = torch.empty_like(order)
        scatter_ref[order] = torch.arange(order.numel(), device=dev)
        assert torch.equal(got[0].long(), torch.bincount(flat.long(), minlength=E))
        assert torch.equal(got[2].long(), scatter_ref)
        assert torch.equal(got[3].long(), order // topk)
        assert torch.equal(got[4].long(), order % topk)


def test_static_scratch_entry_refuses_oversized_problem():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from tempname_new_b200 import _native
    lib = _native.lib()
    dev = torch.device("cuda", 0)
    E = 512
    n = 4096 * (STATIC_ELEMS // E) + 1        # one block more than the array holds
    ce = torch.zeros(n, dtype=torch.int32, device=dev)
    rc, _ = _call_static(lib, ce, E, 1)
    assert rc == 1
    assert "exceeds the built-in scratch" in lib.fluxb_last_error().decode()
    # and a fitting problem still works afterwards
    rc, outs = _call_static(lib, ce[:4096], E, 1)
    torch.cuda.synchronize()
    assert rc == 0 and int(outs[0][0]) == 4096
