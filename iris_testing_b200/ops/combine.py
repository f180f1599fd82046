"""Combine: return all-to-all of expert outputs plus the top-k weighted sum.

The reference stops after dispatch (no return path, top-k weights discarded,
utils.py:201-202); this is the missing tail of its intended forward pass.
Unfused form: ``padded_return`` sends every (expert, src) cell of processed rows
back to ``src``; ``weighted_gather`` then forms ``y[t] = sum_slot w[t, slot] * row``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as nv
from ._common import declare, default_status, ptr, require, stream_ptr
from .dispatch import _heap_of, tile_rows


def padded_return(out_buf: torch.Tensor, pca: torch.Tensor, ret_buf: torch.Tensor,
                  ret_sync: torch.Tensor, heap_bases) -> torch.Tensor:
    """out_buf [e_local, world(src), CAP, H] on the expert rank -> ret_buf
    [world(expert rank), e_local, CAP, H] on each source rank (symmetric), with one
    count per tile added to ``ret_sync[expert rank]`` there.  Returns ``ret_buf``
    without waiting for remote arrival."""
    e_local, world, cap, H = out_buf.shape
    if not out_buf.is_cuda:
        send = out_buf.permute(1, 0, 2, 3).contiguous()     # [src, e, CAP, H]
        recv = torch.empty_like(send)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_to_all_single(recv, send)
        else:
            recv.copy_(send)
        ret_buf.copy_(recv)
        return ret_buf
    heap = _heap_of(heap_bases)
    require(out_buf.is_contiguous() and H % 8 == 0, "out_buf must be contiguous with hidden_dim % 8 == 0")
    fn = declare("b200_padded_return",
                 [C.c_void_p, C.c_void_p, C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), C.c_int,
                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p])
    rc = fn(ptr(out_buf), ptr(pca), heap.peer_ptrs(ret_buf), heap.peer_ptrs(ret_sync), heap.rank,
            heap.world, e_local, cap, H, tile_rows(), stream_ptr(out_buf))
    nv.check(rc, "padded return launch")
    return ret_buf


def weighted_gather(ret_buf: torch.Tensor, plan, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                    ret_sync: Optional[torch.Tensor], world: int, capacity: int,
                    status: Optional[torch.Tensor] = None, wait_budget_ms: float = 2000.0,
                    rearm_ticket: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[t] = sum_slot topk_w[t, slot] * ret_buf[cell of (t, slot)]   -> [T, H].

    ``plan`` is the :class:`~iris_testing_b200.ops.plan.Plan` used for the dispatch.  On CUDA
    the kernel first waits (bounded) until ``ret_sync`` shows every returned tile; with
    ``rearm_ticket`` (an int32 scratch counter that is zero between calls) it also zeroes
    ``ret_sync`` when done, so the next exchange needs no memset."""
    T, k = topk_idx.shape
    H = ret_buf.shape[-1]
    e_local = ret_buf.shape[1]
    if not ret_buf.is_cuda:
        flat_e = topk_idx.reshape(-1).long()
        m = plan.dst_slot.long() - plan.bucket_start.long()[flat_e]
        keep = (m < capacity)
        rows = ret_buf.reshape(-1, H)[(flat_e * capacity + m.clamp(max=capacity - 1))].float()
        rows = rows * (topk_w.reshape(-1, 1).float() * keep.unsqueeze(1))
        return rows.view(T, k, H).sum(dim=1).to(ret_buf.dtype)
    fn = declare("b200_weighted_gather",
                 [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                  C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                  C.c_void_p, C.c_ulonglong, C.c_void_p, C.c_void_p])
    y = torch.empty((T, H), dtype=ret_buf.dtype, device=ret_buf.device)
    if status is None:
        status = default_status(ret_buf.device)
    if ret_sync is None:   # nothing to wait for: an all-zero expectation is met by any counter
        ret_sync = torch.full((world,), 2 ** 30, dtype=torch.int32, device=ret_buf.device)
    rc = fn(ptr(ret_buf), ptr(plan.dst_slot), ptr(topk_idx), ptr(plan.bucket_start), ptr(topk_w),
            ptr(ret_sync), ptr(plan.counts), T, k, world, e_local, capacity, H, tile_rows(), ptr(y),
            ptr(status), int(wait_budget_ms * 1e6), ptr(rearm_ticket), stream_ptr(ret_buf))
    nv.check(rc, "weighted gather launch")
    return y
