"""Router: softmax over router logits, then top-k (indices and weights).

Reference: utils.py:201-202 computes ``softmax(tokens @ router)`` and keeps only
the top-k *indices*; this op also returns the top-k probabilities, which the
combine step needs.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import cpu_ref
from ._common import contiguous_bf16, declare, ptr, require, stream_ptr, use_native

MAX_TOPK = 8


def router_topk(x: torch.Tensor, w_router: torch.Tensor, topk: int,
                bias: Optional[torch.Tensor] = None, renormalize: bool = False,
                return_logits: bool = False):
    """x [T, D], w_router [D, E] -> (idx int32 [T, k], weight fp32 [T, k][, logits fp32 [T, E]])."""
    require(x.dim() == 2 and w_router.dim() == 2 and x.shape[1] == w_router.shape[0],
            "router_topk: x must be [T, D] and w_router [D, E]")
    T, D = x.shape
    E = w_router.shape[1]
    require(1 <= topk <= min(E, MAX_TOPK), f"topk must be in [1, min(E, {MAX_TOPK})]")
    if not use_native(x):
        idx, w = cpu_ref.router_topk_ref(x, w_router, topk, bias, renormalize)
        if return_logits:
            lg = x.float() @ w_router.float()
            return idx, w, (lg + bias.float() if bias is not None else lg)
        return idx, w
    x = contiguous_bf16(x, "x")
    w_router = contiguous_bf16(w_router, "w_router")
    fn = declare("b200_router_topk_simple",
                 [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p])
    idx = torch.empty((T, topk), dtype=torch.int32, device=x.device)
    w = torch.empty((T, topk), dtype=torch.float32, device=x.device)
    logits = torch.empty((T, E), dtype=torch.float32, device=x.device) if return_logits else None
    b = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
    rc = fn(ptr(x), ptr(w_router), ptr(b), T, D, E, topk, int(renormalize), ptr(idx), ptr(w),
            ptr(logits), stream_ptr(x))
    if rc != 0:
        raise RuntimeError(f"router_topk launch failed ({rc})")
    return (idx, w, logits) if return_logits else (idx, w)
