"""Symmetric heap over NVLink peer memory (one per process / GPU).

``SymmetricHeap`` is this library's counterpart of the ``iris.iris(heap_size)``
context the reference project builds on (benchmark.py:38-42): a device heap whose
allocator returns the *same offsets on every rank*, a table of every rank's heap
base as mapped into this process (``get_heap_bases``), ``zeros`` / ``empty``
allocation, ``free`` and a ``barrier``.

Two native back-ends (``backend=`` or ``B200_HEAP_BACKEND``; default ``auto``):

``vmm``   csrc/vmm_heap.cu -- ``cuMemCreate`` chunks exported as POSIX file descriptors,
          passed between the ranks over Unix sockets and mapped with ``cuMemMap`` into
          one reserved address window that holds every peer.  The heap can ``grow``
          (a collective call) up to ``max_bytes`` without moving anything.
``ipc``   csrc/symm_heap.cu -- one ``cudaMalloc`` per rank shared through CUDA IPC
          handles (fixed size).  Used when the virtual-memory API or descriptor
          export is not available; ``auto`` falls back to it after a failed ``vmm``
          set-up on any rank.

With ``world_size == 1`` no process group is needed and "peer" addresses are local
addresses, so every kernel runs unchanged on a single GPU.  ``close()`` unmaps and
frees everything; tensors handed out by the heap must not be used afterwards.
"""
from __future__ import annotations

import ctypes as C
import os
import uuid
import weakref
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import _native as nv

_ALIGN = 1024


class _DeviceSpan:
    """Adapter exposing raw device memory through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner) -> None:
        self._owner = owner   # keeps the native memory alive while tensors exist
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
    nv.declare("b200_memcpy_async", [vp, vp, u64, vp])
    nv.declare("b200_barrier", [C.POINTER(u64), vp, i32, i32, C.c_uint, vp, u64, vp])
    nv.declare("b200_error_string", [i32], C.c_char_p)
    nv.declare("b200_vmm_probe", [i32, C.POINTER(C.c_longlong)])
    nv.declare("b200_vmm_create", [i32, i32, i32, u64, C.c_char_p, i32, C.POINTER(vp)])
    nv.declare("b200_vmm_grow", [vp, u64, C.POINTER(u64)])
    nv.declare("b200_vmm_base", [vp, i32], u64)
    nv.declare("b200_vmm_mapped_bytes", [vp], u64)
    nv.declare("b200_vmm_slot_bytes", [vp], u64)
    nv.declare("b200_vmm_destroy", [vp])
    _declare_once.done = True


def cuda_check(code: int, what: str) -> None:
    if code != 0:
        msg = nv.lib().b200_error_string(code).decode() if code > 0 else "argument / set-up error"
        raise nv.NativeError(f"{what}: error {code} ({msg})")


def probe_capabilities(device_index: int) -> Dict[str, int]:
    """What the device offers for symmetric memory (queries only): virtual memory management,
    POSIX descriptor export, NVLink multicast objects (NVLS / ``multimem``), granularity."""
    _declare_once()
    out = (C.c_longlong * 4)()
    rc = nv.lib().b200_vmm_probe(device_index, out)
    return dict(probe_rc=int(rc), vmm=int(out[0]), posix_fd=int(out[1]), multicast=int(out[2]),
                granularity=int(out[3]))


class OffsetAllocator:
    """First-fit offset allocator with coalescing.  Deterministic: ranks that make the same
    sequence of calls get the same offsets, which is what makes the heap symmetric."""

    def __init__(self, align: int = _ALIGN) -> None:
        self.align = align
        self.top = 0                                  # bump pointer: everything above is unused
        self.holes: List[Tuple[int, int]] = []        # (offset, nbytes) below ``top``, sorted, coalesced
        self.live: Dict[int, int] = {}                # offset -> nbytes

    def alloc(self, nbytes: int) -> int:
        need = (max(int(nbytes), 1) + self.align - 1) // self.align * self.align
        for i, (off, sz) in enumerate(self.holes):
            if sz >= need:
                if sz == need:
                    self.holes.pop(i)
                else:
                    self.holes[i] = (off + need, sz - need)
                self.live[off] = need
                return off
        off = self.top
        self.top = off + need
        self.live[off] = need
        return off

    def free(self, off: int) -> None:
        size = self.live.pop(off, None)
        if size is None:
            raise ValueError("not the start of a live allocation")
        self.holes.append((off, size))
        self.holes.sort()
        merged: List[Tuple[int, int]] = []
        for o, sz in self.holes:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + sz)
            else:
                merged.append((o, sz))
        while merged and merged[-1][0] + merged[-1][1] == self.top:   # the tail goes back to the bump pointer
            self.top = merged.pop()[0]
        self.holes = merged

    @property
    def bytes_in_use(self) -> int:
        return sum(self.live.values())


class _HeapMemory:
    """Owns the native allocation.  Tensors carved from the heap keep this object (not the
    ``SymmetricHeap``) alive, so a heap that nobody references any more is released as soon
    as its last tensor dies, and ``close()`` releases it at once."""

    def __init__(self, lib, dev_index: int) -> None:
        self.lib, self.dev_index = lib, dev_index
        self.vmm_handle: Optional[int] = None     # vmm back-end
        self.ipc_base: Optional[int] = None       # ipc back-end
        self.ipc_mapped: List[int] = []
        self.closed = False

    def release(self) -> None:
        if self.closed:
            return
        self.closed = True
        try:
            torch.cuda.synchronize(self.dev_index)
        except Exception:
            pass
        if self.vmm_handle is not None:
            self.lib.b200_vmm_destroy(C.c_void_p(self.vmm_handle))
            self.vmm_handle = None
        for m in self.ipc_mapped:
            self.lib.b200_heap_close(self.dev_index, C.c_void_p(m))
        self.ipc_mapped = []
        if self.ipc_base is not None:
            self.lib.b200_heap_destroy(self.dev_index, C.c_void_p(self.ipc_base))
            self.ipc_base = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class SymmetricHeap:
    """Symmetric device heap shared by the ranks of one node.

    ``size_bytes`` is mapped at once; ``max_bytes`` (vmm back-end) is the address space
    reserved per rank, up to which :meth:`grow` can extend the heap later."""

    def __init__(self, size_bytes: int, group: Optional[dist.ProcessGroup] = None,
                 device: Optional[torch.device] = None, wait_budget_ms: float = 2000.0,
                 backend: Optional[str] = None, max_bytes: Optional[int] = None) -> None:
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
        self.device = torch.device("cuda", self.dev_index)
        self.wait_budget_ns = int(wait_budget_ms * 1e6)
        want = (backend or os.getenv("B200_HEAP_BACKEND", "auto")).lower()
        if want not in ("auto", "vmm", "ipc"):
            raise ValueError("backend must be 'auto', 'vmm' or 'ipc'")
        self.capabilities = probe_capabilities(self.dev_index)
        self._mem = _HeapMemory(self.lib, self.dev_index)
        size = (int(size_bytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        reserve = max(size, int(max_bytes) if max_bytes is not None else 4 * size)
        self.backend = None
        if want in ("auto", "vmm"):
            err = self._setup_vmm(size, reserve)
            if err is not None and want == "vmm":
                raise nv.NativeError(f"vmm heap set-up failed: {err}")
            if err is None:
                self.backend = "vmm"
        if self.backend is None:
            self._setup_ipc(size)
            self.backend = "ipc"
        self.capabilities["backend"] = self.backend
        self.base = self.peer_bases[self.rank]
        self._bytes = torch.as_tensor(_DeviceSpan(self.base, self._span, self._mem), device=self.device)
        self._allocator = OffsetAllocator(_ALIGN)
        # control block: status word + barrier flags, allocated first so offsets are fixed
        self.status = self.zeros((4,), torch.int32)
        self._barrier_flags = self.zeros((nv.MAX_WORLD,), torch.int32)
        self._barrier_epoch = 0
        self._heap_bases_t = torch.tensor(self.peer_bases, dtype=torch.int64, device=self.device)
        self._heap_bases_t._b200_heap = weakref.ref(self)    # lets ops find the heap from the table

    # ------------------------------------------------------------------ set-up
    def _agree(self, ok: bool) -> bool:
        """True when ``ok`` holds on every rank."""
        if self.world == 1:
            return ok
        flags: List[Optional[bool]] = [None] * self.world
        dist.all_gather_object(flags, bool(ok), group=self.group)
        return all(flags)

    def _setup_vmm(self, size: int, reserve: int) -> Optional[str]:
        caps = self.capabilities
        err = None
        if caps["probe_rc"] != 0 or not caps["vmm"] or (self.world > 1 and not caps["posix_fd"]):
            err = f"not supported on this device ({caps})"
        tag = [uuid.uuid4().hex if self.rank == 0 else None]
        if self.world > 1:
            dist.broadcast_object_list(tag, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                                       group=self.group)
        handle = C.c_void_p()
        if err is None:
            rc = self.lib.b200_vmm_create(self.dev_index, self.world, self.rank, reserve,
                                          f"b200heap-{tag[0]}".encode(), 30000, C.byref(handle))
            if rc != 0:
                err = f"create returned {rc}"
        if not self._agree(err is None):          # also: every socket is bound before anyone sends
            if handle.value:
                self.lib.b200_vmm_destroy(handle)
            return err or "a peer could not set up its heap"
        self._mem.vmm_handle = int(handle.value)
        got = C.c_ulonglong()
        rc = self.lib.b200_vmm_grow(handle, size, C.byref(got))
        if not self._agree(rc == 0):
            self._mem.release()
            self._mem = _HeapMemory(self.lib, self.dev_index)
            return f"grow returned {rc}"
        self.size = int(self.lib.b200_vmm_mapped_bytes(handle))
        self._span = int(self.lib.b200_vmm_slot_bytes(handle))
        self.max_bytes = self._span
        self.peer_bases = [int(self.lib.b200_vmm_base(handle, r)) for r in range(self.world)]
        return None

    def _setup_ipc(self, size: int) -> None:
        base = C.c_void_p()
        cuda_check(self.lib.b200_heap_create(self.dev_index, size, C.byref(base)), "heap create")
        self._mem.ipc_base = int(base.value)
        self.size = self._span = self.max_bytes = size
        self.peer_bases = [int(base.value)] * self.world
        if self.world > 1:
            n = self.lib.b200_heap_handle_bytes()
            buf = C.create_string_buffer(n)
            cuda_check(self.lib.b200_heap_export(self.dev_index, base, buf), "heap export")
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(buf.raw), group=self.group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                mapped = C.c_void_p()
                cuda_check(self.lib.b200_heap_open(self.dev_index, h, C.byref(mapped)), f"heap open (rank {r})")
                self.peer_bases[r] = int(mapped.value)
                self._mem.ipc_mapped.append(int(mapped.value))
            dist.barrier(group=self.group)

    def grow(self, new_size_bytes: int) -> None:
        """Collective: extend the mapped heap to at least ``new_size_bytes`` on every rank
        (vmm back-end; addresses of existing allocations do not change)."""
        if new_size_bytes <= self.size:
            return
        if self.backend != "vmm":
            raise MemoryError("the ipc heap has a fixed size; create it large enough or use the vmm back-end")
        if new_size_bytes > self.max_bytes:
            raise MemoryError(f"heap can grow to {self.max_bytes} bytes at most (max_bytes)")
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(group=self.group)      # nobody is still inside an earlier grow
        got = C.c_ulonglong()
        rc = self.lib.b200_vmm_grow(C.c_void_p(self._mem.vmm_handle), new_size_bytes - self.size, C.byref(got))
        if not self._agree(rc == 0):
            raise nv.NativeError(f"rank {self.rank}: heap grow failed ({rc})")
        self.size = int(self.lib.b200_vmm_mapped_bytes(C.c_void_p(self._mem.vmm_handle)))

    # -------------------------------------------------------------- allocation
    def _alloc(self, nbytes: int) -> Tuple[int, torch.Tensor]:
        off = self._allocator.alloc(nbytes)
        end = off + self._allocator.live[off]
        if end > self.size:
            if self.backend == "vmm" and end <= self.max_bytes:
                self.grow(max(end, min(self.max_bytes, self.size + (self.size >> 1))))
            else:
                self._allocator.free(off)
                raise MemoryError(f"symmetric heap exhausted: need {nbytes} B at offset {off}, size {self.size}")
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

    def free(self, t: torch.Tensor) -> None:
        """Return an allocation made by :meth:`empty` / :meth:`zeros` (every rank must free the
        same buffers in the same order).  ``t`` must be the tensor that was returned, or a
        view starting at its first byte."""
        self._allocator.free(self.offset_of(t))

    @property
    def bytes_in_use(self) -> int:
        return self._allocator.bytes_in_use

    def offset_of(self, t: torch.Tensor) -> int:
        off = t.data_ptr() - self.base
        if off < 0 or off >= self._span:
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

    def copy_to_peer(self, t: torch.Tensor, rank: int, src: torch.Tensor) -> None:
        """Copy local tensor ``src`` into rank ``rank``'s copy of symmetric tensor ``t`` (one
        asynchronous device copy on the current stream; goes over NVLink for a peer)."""
        nbytes = src.numel() * src.element_size()
        if nbytes > t.numel() * t.element_size() or not src.is_contiguous():
            raise ValueError("src must be contiguous and fit into the symmetric tensor")
        st = torch.cuda.current_stream(self.device)
        cuda_check(self.lib.b200_memcpy_async(C.c_void_p(self.peer_ptr(t, rank)), C.c_void_p(src.data_ptr()),
                                              nbytes, C.c_void_p(st.cuda_stream)), "copy to peer")

    def copy_from_peer(self, t: torch.Tensor, rank: int) -> torch.Tensor:
        """A local copy of rank ``rank``'s copy of symmetric tensor ``t`` (asynchronous)."""
        out = torch.empty(t.shape, dtype=t.dtype, device=self.device)
        st = torch.cuda.current_stream(self.device)
        cuda_check(self.lib.b200_memcpy_async(C.c_void_p(out.data_ptr()), C.c_void_p(self.peer_ptr(t, rank)),
                                              t.numel() * t.element_size(), C.c_void_p(st.cuda_stream)),
                   "copy from peer")
        return out

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
        """Unmap the peers and free this rank's memory now.  Collective in spirit: no rank may
        still be writing into a heap that a peer closes.  Tensors from this heap are dead."""
        self._mem.release()

    @property
    def closed(self) -> bool:
        return self._mem.closed
