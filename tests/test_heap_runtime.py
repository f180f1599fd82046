"""Symmetric-heap runtime: the offset allocator and the file-descriptor channel run on CPU;
heap creation, growth and release run on one GPU (the multi-GPU pattern test is part of
``unit_tests.py``)."""
import ctypes as C
import os

import pytest
import torch

from conftest import run_gloo


def test_offset_allocator_first_fit_coalesce_and_determinism():
    from iris_testing_b200.parallel.symm import OffsetAllocator
    a = OffsetAllocator(1024)
    o1, o2, o3 = a.alloc(100), a.alloc(5000), a.alloc(1024)
    assert (o1, o2, o3) == (0, 1024, 1024 + 5120) and a.top == 7168
    a.free(o2)                                  # a hole of 5 KiB
    assert a.alloc(2048) == 1024                # first fit, splits the hole
    assert a.alloc(4096) == 7168                # does not fit the remaining 3 KiB: bump
    a.free(o1)
    assert a.alloc(1) == 0
    with pytest.raises(ValueError):
        a.free(12345)
    # freeing everything in any order returns the allocator to empty
    for off in list(a.live):
        a.free(off)
    assert a.top == 0 and a.holes == [] and a.bytes_in_use == 0
    # two ranks making the same calls get the same offsets
    b, c = OffsetAllocator(), OffsetAllocator()
    seq = [("a", 3000), ("a", 70000), ("f", 0), ("a", 1024), ("a", 2048), ("f", 1), ("a", 50000)]
    outs = []
    for alloc in (b, c):
        offs, got = [], []
        for op, v in seq:
            if op == "a":
                offs.append(alloc.alloc(v))
                got.append(offs[-1])
            else:
                alloc.free(offs[v])
        outs.append(got)
    assert outs[0] == outs[1]


def _fd_worker(rank, world, tag):
    """Each rank sends a pipe's read end to its neighbour and writes its own rank into the pipe;
    the neighbour reads the rank back through the descriptor it received."""
    from iris_testing_b200 import _native
    lib = _native.lib()
    vp = C.c_void_p
    lib.b200_fdchan_open.argtypes = [C.c_char_p, C.c_int, C.c_int, C.POINTER(vp)]
    lib.b200_fdchan_send.argtypes = [vp, C.c_int, C.c_int, C.c_uint, C.c_ulonglong]
    lib.b200_fdchan_recv.argtypes = [vp, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_uint),
                                     C.POINTER(C.c_ulonglong)]
    lib.b200_fdchan_close.argtypes = [vp]
    import torch.distributed as dist
    chan = vp()
    assert lib.b200_fdchan_open(f"b200test-{tag}".encode(), rank, 5000, C.byref(chan)) == 0
    dist.barrier()                                       # every socket is bound
    r, w = os.pipe()
    os.write(w, bytes([40 + rank]))
    assert lib.b200_fdchan_send(chan, (rank + 1) % world, r, 7, 4096 + rank) == 0
    frm, fd, gen, nbytes = C.c_int(-1), C.c_int(-1), C.c_uint(0), C.c_ulonglong(0)
    assert lib.b200_fdchan_recv(chan, C.byref(frm), C.byref(fd), C.byref(gen), C.byref(nbytes)) == 0
    got = os.read(fd.value, 1)[0]
    # nothing else is queued: the next receive runs into the channel's time limit
    lib.b200_fdchan_close(chan)
    chan2 = vp()
    assert lib.b200_fdchan_open(f"b200test-{tag}-idle".encode(), rank, 200, C.byref(chan2)) == 0
    timeout_rc = lib.b200_fdchan_recv(chan2, C.byref(frm), C.byref(C.c_int()), C.byref(gen), C.byref(nbytes))
    lib.b200_fdchan_close(chan2)
    return dict(frm=frm.value, got=got, gen=gen.value, nbytes=nbytes.value, timeout_rc=timeout_rc)


def test_fd_channel_passes_descriptors_between_processes():
    import uuid
    res = run_gloo(_fd_worker, world=2, args=(uuid.uuid4().hex,))
    for rank, r in enumerate(res):
        src = (rank - 1) % 2
        assert r["frm"] == src and r["got"] == 40 + src and r["gen"] == 7 and r["nbytes"] == 4096 + src
        assert r["timeout_rc"] == -34                   # time limit, not a hang


@pytest.mark.gpu
@pytest.mark.parametrize("backend", ["vmm", "ipc"])
def test_heap_create_close_leaves_memory_flat(backend):
    from iris_testing_b200.parallel.symm import SymmetricHeap
    torch.cuda.set_device(0)
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for i in range(50):
        heap = SymmetricHeap(64 << 20, backend=backend)
        assert heap.backend == backend
        t = heap.zeros((1024,), torch.int32)
        t += i
        assert int(t[5]) == i
        del t
        heap.close()
        assert heap.closed
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert abs(free1 - free0) <= (8 << 20), (free0, free1)
    # a heap that is merely dropped is released once its last tensor dies
    heap = SymmetricHeap(64 << 20, backend=backend)
    t = heap.zeros((16,), torch.int32)
    del heap
    assert int(t.sum()) == 0                             # memory still valid through the tensor
    del t
    torch.cuda.synchronize()
    free2, _ = torch.cuda.mem_get_info()
    assert abs(free2 - free0) <= (8 << 20), (free0, free2)


@pytest.mark.gpu
def test_vmm_heap_grows_without_moving_and_reports_capabilities():
    from iris_testing_b200.parallel.symm import SymmetricHeap
    torch.cuda.set_device(0)
    heap = SymmetricHeap(8 << 20, backend="vmm", max_bytes=256 << 20)
    caps = heap.capabilities
    assert caps["vmm"] == 1 and caps["granularity"] > 0 and caps["multicast"] in (0, 1)
    a = heap.zeros((1 << 20,), torch.int32)              # 4 MiB
    a.fill_(3)
    addr, size0 = a.data_ptr(), heap.size
    b = heap.zeros((16 << 20,), torch.int32)             # 64 MiB: does not fit -> the heap grows
    assert heap.size > size0 and a.data_ptr() == addr and int(a[12345]) == 3
    b.fill_(9)
    assert int(b[-1]) == 9 and heap.peer_ptr(b, 0) == b.data_ptr()
    # copies through the peer table (on one GPU the peer is this GPU)
    src = torch.arange(64, dtype=torch.int32, device=heap.device)
    heap.copy_to_peer(a, 0, src)
    assert torch.equal(heap.copy_from_peer(a, 0)[:64], src)
    heap.free(b)
    c = heap.zeros((1024,), torch.int32)
    assert c.data_ptr() == b.data_ptr()                  # freed space is reused
    with pytest.raises(MemoryError):
        heap.zeros((128 << 20,), torch.int32)            # 512 MiB > max_bytes
    del a, b, c
    heap.close()
