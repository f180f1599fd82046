"""The allocation-free plan entry point, called through its exported C symbol.

Some users of this library cannot allocate device memory at call time (a serving loop
with all memory pre-sized, a callback running under a framework allocator that must not
be re-entered, a host program that only hands over raw buffers).  ``b200_plan_noalloc``
gives them the dispatch plan with its temporary held in a fixed array inside the library.
This test calls it twice in a row through ``ctypes`` and checks every output against the
regular entry point ``b200_plan``; the second call uses different routing so that stale
contents of the shared array would show.  It lives in a file that pytest collects last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(lib, idx, E, stream):
    n = idx.numel()
    i32 = dict(dtype=torch.int32, device=idx.device)
    rank, counts, start = torch.empty(n, **i32), torch.empty(E, **i32), torch.empty(E + 1, **i32)
    order, slot = torch.empty(n, **i32), torch.empty(n, **i32)
    lib.b200_plan.argtypes = [C.c_void_p] * 1 + [C.c_int, C.c_int] + [C.c_void_p] * 7
    lib.b200_plan.restype = C.c_int
    rc = lib.b200_plan(idx.data_ptr(), n, E, rank.data_ptr(), counts.data_ptr(), start.data_ptr(),
                       order.data_ptr(), slot.data_ptr(), None, stream)
    assert rc == 0
    return counts, start, order, slot


def test_plan_noalloc_matches_regular_entry_point_twice():
    from iris_testing_b200 import _native
    lib = _native.lib()
    fn = lib.b200_plan_noalloc
    fn.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    lib.b200_plan_noalloc_max.restype = C.c_int
    limit = lib.b200_plan_noalloc_max()
    assert limit == 1 << 20
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    g = torch.Generator(device="cpu").manual_seed(7)
    cases = [(4096, 8, 64), (1000, 2, 8)]          # second call: fewer copies, other experts
    for T, k, E in cases:
        idx = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32).to(dev)
        n = T * k
        i32 = dict(dtype=torch.int32, device=dev)
        counts, start = torch.empty(E, **i32), torch.empty(E + 1, **i32)
        order, slot = torch.empty(n, **i32), torch.empty(n, **i32)   # outputs, made by the caller
        rc = fn(idx.data_ptr(), n, E, counts.data_ptr(), start.data_ptr(), order.data_ptr(),
                slot.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        r_counts, r_start, r_order, r_slot = _regular(lib, idx, E, stream)
        torch.cuda.synchronize()
        assert torch.equal(counts, r_counts) and torch.equal(start, r_start)
        assert torch.equal(order, r_order) and torch.equal(slot, r_slot)
    # dst_slot is optional: without it the other outputs are unchanged
    order2 = torch.empty(n, **i32)
    assert fn(idx.data_ptr(), n, E, counts.data_ptr(), start.data_ptr(), order2.data_ptr(), None, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(order2, r_order) and torch.equal(counts, r_counts)
    # no routed copies at all: zero counts, an all-zero scan, nothing else touched
    assert fn(idx.data_ptr(), 0, E, counts.data_ptr(), start.data_ptr(), order2.data_ptr(), None, stream) == 0
    torch.cuda.synchronize()
    assert int(counts.abs().sum()) == 0 and int(start.abs().sum()) == 0
    assert torch.equal(order2, r_order)
    # beyond the stated maximum: a clear error and nothing launched
    assert fn(idx.data_ptr(), limit + 1, 8, counts.data_ptr(), start.data_ptr(), order.data_ptr(),
              slot.data_ptr(), stream) == -20
    assert fn(None, 8, 8, counts.data_ptr(), start.data_ptr(), order.data_ptr(), None, stream) == -21
