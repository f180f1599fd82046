"""Dispatch plan: per-expert counts, stable bucket ranks, packed send order.

Replaces the reference's Python bucket loop (utils.py:204-246, one ``.item()``
per routed copy) and its offset helpers (utils.py:20-31, benchmark.py:44-49)
with two kernel launches.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _native as nv
from . import cpu_ref
from ._common import declare, ptr, require, stream_ptr, use_native


class PlanPushArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int), ("rank", C.c_int),
        ("epoch", C.c_uint32), ("need_iter_done", C.c_uint32),
        ("iter_done", C.c_void_p),
        ("peer_counts", C.c_ulonglong * nv.MAX_WORLD),
        ("peer_flags", C.c_ulonglong * nv.MAX_WORLD),
        ("status", C.c_void_p),
        ("wait_budget_ns", C.c_ulonglong),
        ("iter_ptr", C.c_void_p),
        ("stride_counts", C.c_ulonglong),
        ("stride_flags", C.c_ulonglong),
    ]


@dataclass
class Plan:
    counts: torch.Tensor          # int32 [E]
    bucket_start: torch.Tensor    # int32 [E+1]
    send_order: torch.Tensor      # int32 [T*k]
    dst_slot: torch.Tensor        # int32 [T*k]
    rank_in_bucket: torch.Tensor  # int32 [T*k]

    def send_counts(self, world: int) -> torch.Tensor:
        """[world, e_local] view of the counts (reference layout, layers/all_to_all.py:21)."""
        return self.counts.view(world, -1)


def _plan_fn():
    return declare("b200_plan", [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_void_p, C.POINTER(PlanPushArgs), C.c_void_p])


def make_plan(topk_idx: torch.Tensor, num_experts: int, out: Optional[Plan] = None,
              push: Optional[PlanPushArgs] = None) -> Plan:
    """topk_idx int32 [T, k] (global expert ids) -> :class:`Plan`.

    ``out`` lets a caller reuse preallocated buffers; ``push`` (fused engine only)
    makes the second kernel also publish the counts to every peer.
    """
    require(topk_idx.dtype == torch.int32, "topk_idx must be int32")
    n = topk_idx.numel()
    if not use_native(topk_idx):
        p = cpu_ref.plan_ref(topk_idx, num_experts)
        return Plan(p.counts, p.bucket_start, p.send_order, p.dst_slot, p.rank_in_bucket)
    require(num_experts <= nv.MAX_EXPERTS, f"at most {nv.MAX_EXPERTS} experts are supported")
    dev = topk_idx.device
    if out is None:
        i32 = dict(dtype=torch.int32, device=dev)
        out = Plan(torch.empty(num_experts, **i32), torch.empty(num_experts + 1, **i32),
                   torch.empty(n, **i32), torch.empty(n, **i32), torch.empty(n, **i32))
    idx = topk_idx if topk_idx.is_contiguous() else topk_idx.contiguous()
    rc = _plan_fn()(ptr(idx), n, num_experts, ptr(out.rank_in_bucket), ptr(out.counts),
                    ptr(out.bucket_start), ptr(out.send_order), ptr(out.dst_slot),
                    C.byref(push) if push is not None else None, stream_ptr(idx))
    if rc != 0:
        raise RuntimeError(f"plan launch failed ({rc})")
    return out


def pack_rows(x: torch.Tensor, send_order: torch.Tensor, topk: int) -> torch.Tensor:
    """payload[j] = x[send_order[j] // topk]: the packed send payload (dst-major, expert-major)."""
    if not use_native(x):
        return cpu_ref.pack_ref(x, send_order, topk)
    require(x.is_contiguous() and x.shape[1] % 8 == 0 and x.element_size() == 2,
            "pack_rows: x must be contiguous 16-bit with hidden_dim % 8 == 0")
    fn = declare("b200_pack_rows", [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                    C.c_void_p])
    out = torch.empty((send_order.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    rc = fn(ptr(x), ptr(send_order), send_order.numel(), topk, x.shape[1], ptr(out), stream_ptr(x))
    if rc != 0:
        raise RuntimeError(f"pack_rows launch failed ({rc})")
    return out
