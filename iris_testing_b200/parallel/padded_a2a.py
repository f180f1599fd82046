"""Re-usable padded all-to-all (dispatch, optional return + weighted sum) and the device-side
capacity rule.

``PaddedAllToAll`` owns the symmetric buffers of the reference's contract
(``token_buf[e_local, world, CAP, H]``, ``pca[e_local, world]``, ``counts_ready[1]``,
``token_sync[e_local]``: layers/all_to_all.py:19-45, utils.py:48-80) and drives them with an
epoch counter, so consecutive exchanges need neither the memsets nor the barrier the
reference's benchmark puts around every call (benchmark.py:247-272): flags are re-armed
inside the kernel, a sender writes only after the destination has announced the epoch, and
completion is a local device-side wait on the flags.  Rows travel as bulk copies
(csrc/exchange.cu ``padded_bulk_kernel``).

``CapacityProbe`` computes CAP (utils.py:118-121) and the per-pair message size M
(README.md:5-7) across all ranks on the device, without a host round trip.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as nv
from ..ops._common import declare, ptr, require, stream_ptr
from ..ops.combine import weighted_gather
from ..ops.dispatch import tile_rows
from ..ops.expert import sm_count
from ..utils.buffers import ReturnBuffers, ShmemBuffers


def _exchange_fn():
    u64p = C.POINTER(C.c_ulonglong)
    return declare("b200_padded_exchange",
                   [C.c_void_p, C.c_void_p, C.c_void_p, u64p, u64p, u64p, u64p, u64p, C.c_void_p, C.c_uint,
                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                    C.c_void_p, C.c_ulonglong, C.c_void_p])


class PaddedAllToAll:
    """Padded dispatch (and return) over one set of symmetric buffers, call after call.

    Every rank must construct it with the same arguments and make the same sequence of
    calls.  Between ``dispatch`` calls the caller's consumer of ``token_buf`` must have been
    enqueued on the same stream (stream order is what tells the next call that the buffers
    are free)."""

    def __init__(self, heap, e_local: int, capacity: int, hidden_dim: int, dtype: torch.dtype,
                 with_return: bool = False, num_blocks: Optional[int] = None,
                 wait_budget_ms: float = 2000.0, copy_mode: Optional[str] = None) -> None:
        self.heap, self.world, self.rank = heap, heap.world, heap.rank
        self.e_local, self.cap, self.H, self.dtype = int(e_local), int(capacity), int(hidden_dim), dtype
        self.esz = torch.empty((), dtype=dtype).element_size()
        require((self.H * self.esz) % 16 == 0, "rows must be a multiple of 16 bytes")
        W = self.world
        i32 = torch.int32
        self.buffers = ShmemBuffers(
            pca=heap.zeros((self.e_local, W), i32), counts_ready=heap.zeros((1,), i32),
            token_buf=heap.zeros((self.e_local, W, self.cap, self.H), dtype),
            token_sync=heap.zeros((self.e_local,), i32), heap_bases=heap.get_heap_bases())
        self.entered = heap.zeros((nv.MAX_WORLD,), i32)
        self.ret: Optional[ReturnBuffers] = None
        if with_return:
            self.ret = ReturnBuffers(ret_buf=heap.zeros((W, self.e_local, self.cap, self.H), dtype),
                                     ret_sync=heap.zeros((W,), i32))
            self._ticket = torch.zeros(1, dtype=i32, device=heap.device)
        self.epoch = 0
        # "stores": every thread moves 16-byte pieces (several blocks per SM); "bulk": one lane per warp
        # drives bulk copies through shared memory (one block per SM)
        self.copy_mode = (copy_mode or os.getenv("B200MOE_A2A_COPY", "stores")).lower()
        require(self.copy_mode in ("stores", "bulk"), "copy_mode must be 'stores' or 'bulk'")
        self._plain = int(self.copy_mode == "stores")
        per_sm = 4 if self._plain else 1
        self.blocks = int(num_blocks) if num_blocks else sm_count(heap.device) * per_sm
        self.budget_ns = int(wait_budget_ms * 1e6)
        torch.cuda.synchronize(heap.device)
        if W > 1:
            dist.barrier(group=heap.group)        # every rank's flags exist and are zero

    # -- reference field names, for code written against utils.alloc_shmem_buffers
    @property
    def token_buf(self): return self.buffers.token_buf
    @property
    def pca(self): return self.buffers.pca
    @property
    def counts_ready(self): return self.buffers.counts_ready
    @property
    def token_sync(self): return self.buffers.token_sync

    def dispatch(self, payload: torch.Tensor, send_counts: torch.Tensor, dst_offsets: torch.Tensor
                 ) -> torch.Tensor:
        """Send the packed ``payload`` (rows ordered by destination, then local expert).  Returns
        ``token_buf`` without waiting for remote arrival, like ``custom_a2a``."""
        require(send_counts.dtype == torch.int32 and dst_offsets.dtype == torch.int32,
                "send_counts and dst_offsets must be int32")
        require(payload.is_contiguous() and payload.dtype == self.dtype and payload.shape[-1] == self.H,
                "payload must be contiguous [rows, hidden_dim] of the buffer dtype")
        h, b = self.heap, self.buffers
        self.epoch += 1
        rc = _exchange_fn()(ptr(payload), ptr(send_counts), ptr(dst_offsets), h.peer_ptrs(b.pca),
                            h.peer_ptrs(b.token_buf), h.peer_ptrs(b.counts_ready), h.peer_ptrs(b.token_sync),
                            h.peer_ptrs(self.entered), ptr(self.entered), self.epoch, self.rank, self.world,
                            self.e_local, self.cap, self.H, self.esz, tile_rows(), 0, self.blocks, self._plain,
                            ptr(h.status), self.budget_ns, stream_ptr(payload))
        nv.check(rc, "padded dispatch launch")
        return b.token_buf

    def wait(self) -> None:
        """Device-side wait (bounded) until this rank has received everything of the current
        dispatch; later work on the stream may read ``token_buf`` and ``pca``."""
        b = self.buffers
        fn = declare("b200_padded_wait", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_void_p, C.c_ulonglong, C.c_void_p])
        nv.check(fn(ptr(b.pca), ptr(b.counts_ready), ptr(b.token_sync), self.world, self.e_local, self.cap,
                    tile_rows(), ptr(self.heap.status), self.budget_ns, stream_ptr(b.pca)), "padded wait launch")

    def send_back(self, out_buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Return the processed rows ``out_buf[e_local, world(src), CAP, H]`` (default: the received
        ``token_buf`` itself) to their source ranks.  Call after :meth:`wait` (the counts must
        have landed).  Returns ``ret_buf`` without waiting for remote arrival."""
        require(self.ret is not None, "constructed without with_return=True")
        h, b, r = self.heap, self.buffers, self.ret
        src = b.token_buf if out_buf is None else out_buf
        require(src.is_contiguous() and tuple(src.shape) == tuple(b.token_buf.shape), "out_buf has the wrong shape")
        rc = _exchange_fn()(ptr(src), ptr(b.pca), None, None, h.peer_ptrs(r.ret_buf), None,
                            h.peer_ptrs(r.ret_sync), None, None, self.epoch, self.rank, self.world,
                            self.e_local, self.cap, self.H, self.esz, tile_rows(), 1, self.blocks, self._plain,
                            ptr(h.status), self.budget_ns, stream_ptr(src))
        nv.check(rc, "padded return launch")
        return r.ret_buf

    def reduce(self, plan, topk_idx: torch.Tensor, topk_w: torch.Tensor) -> torch.Tensor:
        """Wait (bounded) for the returned rows and form ``y[t] = sum_slot w * row``; re-arms the
        return counters for the next exchange."""
        require(self.ret is not None, "constructed without with_return=True")
        return weighted_gather(self.ret.ret_buf, plan, topk_idx, topk_w, self.ret.ret_sync, self.world,
                               self.cap, status=self.heap.status, wait_budget_ms=self.budget_ns / 1e6,
                               rearm_ticket=self._ticket)


class _CapacityArgs(C.Structure):
    _fields_ = [("world", C.c_int), ("rank", C.c_int), ("e_local", C.c_int), ("epoch", C.c_uint32),
                ("peer_table", C.c_ulonglong * nv.MAX_WORLD), ("peer_flags", C.c_ulonglong * nv.MAX_WORLD),
                ("status", C.c_void_p), ("wait_budget_ns", C.c_ulonglong)]


class CapacityProbe:
    """CAP and M of a padded exchange, reduced over all ranks on the device.

    ``measure(send_counts)`` returns an int32 device tensor ``[CAP, M, max rows received by
    any rank, rows received by this rank]`` without synchronising the host; every rank must
    call it the same number of times."""

    def __init__(self, heap, e_local: int, wait_budget_ms: float = 2000.0) -> None:
        self.heap, self.e_local = heap, int(e_local)
        W = heap.world
        self.table = heap.zeros((2, W, W * self.e_local), torch.int32)
        self.flags = heap.zeros((2, W), torch.int32)
        self.epoch = 0
        self.budget_ns = int(wait_budget_ms * 1e6)
        torch.cuda.synchronize(heap.device)
        if W > 1:
            dist.barrier(group=heap.group)

    def measure(self, send_counts: torch.Tensor) -> torch.Tensor:
        h = self.heap
        require(send_counts.dtype == torch.int32 and send_counts.is_cuda and send_counts.is_contiguous()
                and send_counts.numel() == h.world * self.e_local, "send_counts must be int32 [world, e_local]")
        fn = declare("b200_capacity", [C.c_void_p, C.POINTER(_CapacityArgs), C.c_void_p, C.c_void_p])
        self.epoch += 1
        a = _CapacityArgs()
        a.world, a.rank, a.e_local, a.epoch = h.world, h.rank, self.e_local, self.epoch
        a.peer_table = h.peer_ptrs(self.table)
        a.peer_flags = h.peer_ptrs(self.flags)
        a.status = h.status.data_ptr()
        a.wait_budget_ns = self.budget_ns
        out = torch.empty(4, dtype=torch.int32, device=h.device)
        nv.check(fn(ptr(send_counts), C.byref(a), ptr(out), stream_ptr(send_counts)), "capacity launch")
        return out
