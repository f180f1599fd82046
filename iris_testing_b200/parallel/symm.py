"""Symmetric heap over NVLink peer memory (one per process / GPU).

``SymmetricHeap`` is this library's counterpart of the ``iris.iris(heap_size)``
context the reference project builds on (benchmark.py:38-42): a fixed-size
device heap with a bump allocator that returns the *same offsets on every
rank*, a table of every rank's heap base as mapped into this process
(``get_heap_bases``), ``zeros`` / ``empty`` allocation and a ``barrier``.

Heaps are created natively (cudaMalloc + CUDA IPC, csrc/symm_heap.cu); only the
64-byte handles travel through ``torch.distributed``.  With ``world_size == 1``
no process group is needed and "peer" addresses are local addresses, so every
kernel runs unchanged on a single GPU.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import _native as nv

_ALIGN = 1024


class _DeviceSpan:
    """Adapter exposing raw device memory through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner) -> None:
        self._owner = owner   # keeps the heap alive while tensors exist
        self.__cuda_array_interface__ = {
            "shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False),
            "version": 3, "strides": None,
        }


def _declare_once() -> None:
    if getattr(_declare_once, "done", False):
        return
    vp, i32, u64 = C.c_void_p, C.c_int, C.c_ulonglong
    nv.declare("b200_heap_create", [i32, u64, C.POINTER(vp)])
    nv.declare("b200_heap_destroy", [i32, vp])
    nv.declare("b200_heap_handle_bytes", [])
    nv.declare("b200_heap_export", [i32, vp, C.c_char_p])
    nv.declare("b200_heap_open", [i32, C.c_char_p, C.POINTER(vp)])
    nv.declare("b200_heap_close", [i32, vp])
    nv.declare("b200_memset_async", [vp, i32, u64, vp])
    nv.declare("b200_barrier", [C.POINTER(u64), vp, i32, i32, C.c_uint, vp, u64, vp])
    nv.declare("b200_error_string", [i32], C.c_char_p)
    _declare_once.done = True


def cuda_check(code: int, what: str) -> None:
    if code != 0:
        msg = nv.lib().b200_error_string(code).decode() if code > 0 else "argument error"
        raise nv.NativeError(f"{what}: error {code} ({msg})")


class SymmetricHeap:
    """Fixed-size symmetric device heap shared by the ranks of one node."""

    def __init__(self, size_bytes: int, group: Optional[dist.ProcessGroup] = None,
                 device: Optional[torch.device] = None, wait_budget_ms: float = 2000.0) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("SymmetricHeap needs a CUDA device")
        _declare_once()
        self.lib = nv.lib()
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        if self.world > nv.MAX_WORLD:
            raise ValueError(f"at most {nv.MAX_WORLD} ranks per node are supported")
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self.dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.size = (int(size_bytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        self.wait_budget_ns = int(wait_budget_ms * 1e6)
        base = C.c_void_p()
        cuda_check(self.lib.b200_heap_create(self.dev_index, self.size, C.byref(base)), "heap create")
        self.base = int(base.value)
        self._mapped: List[int] = []
        self.peer_bases: List[int] = [self.base] * self.world
        if self.world > 1:
            self._exchange_handles()
        self._bytes = torch.as_tensor(_DeviceSpan(self.base, self.size, self), device=self.device)
        self._top = 0
        self._closed = False
        # control block: status word + barrier flags, allocated first so offsets are fixed
        self.status = self.zeros((4,), torch.int32)
        self._barrier_flags = self.zeros((nv.MAX_WORLD,), torch.int32)
        self._barrier_epoch = 0
        self._heap_bases_t = torch.tensor(self.peer_bases, dtype=torch.int64, device=self.device)

    # ------------------------------------------------------------------ set-up
    def _exchange_handles(self) -> None:
        n = self.lib.b200_heap_handle_bytes()
        buf = C.create_string_buffer(n)
        cuda_check(self.lib.b200_heap_export(self.dev_index, C.c_void_p(self.base), buf), "heap export")
        mine = bytes(buf.raw)
        handles: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(handles, mine, group=self.group)
        for r, h in enumerate(handles):
            if r == self.rank:
                continue
            mapped = C.c_void_p()
            cuda_check(self.lib.b200_heap_open(self.dev_index, h, C.byref(mapped)), f"heap open (rank {r})")
            self.peer_bases[r] = int(mapped.value)
            self._mapped.append(int(mapped.value))
        dist.barrier(group=self.group)

    # -------------------------------------------------------------- allocation
    def _alloc(self, nbytes: int) -> Tuple[int, torch.Tensor]:
        off = (self._top + _ALIGN - 1) // _ALIGN * _ALIGN
        if off + nbytes > self.size:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} B at offset {off}, size {self.size}")
        self._top = off + nbytes
        return off, self._bytes[off:off + nbytes]

    def empty(self, shape: Sequence[int], dtype: torch.dtype, device=None) -> torch.Tensor:
        """Allocate at the next offset (identical on every rank if all ranks make the same calls)."""
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        _, raw = self._alloc(max(nbytes, 1))
        return raw[:nbytes].view(dtype).view(*shape) if nbytes else torch.empty(shape, dtype=dtype, device=self.device)

    def zeros(self, shape: Sequence[int], dtype: torch.dtype, device=None) -> torch.Tensor:
        t = self.empty(shape, dtype)
        t.zero_()
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self.size:
            raise ValueError("tensor does not live in this symmetric heap")
        return off

    def peer_ptr(self, t: torch.Tensor, rank: int) -> int:
        """Address of rank ``rank``'s copy of symmetric tensor ``t`` in this process."""
        return self.peer_bases[rank] + self.offset_of(t)

    def peer_ptrs(self, t: torch.Tensor):
        arr = (C.c_ulonglong * nv.MAX_WORLD)()
        off = self.offset_of(t)
        for r in range(self.world):
            arr[r] = self.peer_bases[r] + off
        return arr

    def get_heap_bases(self) -> torch.Tensor:
        """int64 [world]: every rank's heap base as mapped here (cf. utils.py:72)."""
        return self._heap_bases_t

    # ------------------------------------------------------------ coordination
    def barrier(self, stream: Optional[torch.cuda.Stream] = None, host_sync: bool = True) -> None:
        """Device-side barrier across the ranks (bounded wait), then optional host sync.

        Counterpart of ``shmem.barrier()`` (benchmark.py:194).  Every rank must call it
        the same number of times.
        """
        self._barrier_epoch += 1
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        cuda_check(self.lib.b200_barrier(self.peer_ptrs(self._barrier_flags),
                                         C.c_void_p(self._barrier_flags.data_ptr()), self.rank,
                                         self.world, self._barrier_epoch,
                                         C.c_void_p(self.status.data_ptr()), self.wait_budget_ns,
                                         C.c_void_p(st.cuda_stream)), "barrier launch")
        if host_sync:
            st.synchronize()
            self.check_status()

    def check_status(self, reset: bool = True) -> None:
        """Raise if any kernel recorded an error (timeout, overflow, bad index) on this rank."""
        st = self.status.tolist()
        code = int(st[0])
        if code != 0:
            if reset:
                self.status.zero_()
            extra = f" (rows needed on this rank: {st[1]})" if code == 10 and st[1] > 0 else ""
            raise nv.NativeError(f"rank {self.rank}: device status {code}: {nv.status_message(code)}{extra}")

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        for m in self._mapped:
            self.lib.b200_heap_close(self.dev_index, C.c_void_p(m))
        self._mapped = []

    def __del__(self):  # the allocation itself lives until process exit: tensors may still view it
        try:
            self.close()
        except Exception:
            pass
