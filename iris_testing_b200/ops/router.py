"""Router: softmax over router logits, then top-k (indices and weights).

Reference: utils.py:201-202 computes ``softmax(tokens @ router)`` and keeps only
the top-k *indices*; this op also returns the top-k probabilities, which the
combine step needs.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import cpu_ref
from ._common import contiguous_bf16, declare, default_status, ptr, require, stream_ptr, use_native

MAX_TOPK = 8


def router_topk(x: torch.Tensor, w_router: torch.Tensor, topk: int,
                bias: Optional[torch.Tensor] = None, renormalize: bool = False,
                return_logits: bool = False, force_simple: bool = False,
                status: Optional[torch.Tensor] = None):
    """x [T, D], w_router [D, E] -> (idx int32 [T, k], weight fp32 [T, k][, logits fp32 [T, E]]).

    On CUDA the logits are computed on the tensor cores and softmax/top-k run in that
    kernel's epilogue (hidden_dim % 8 == 0 and E <= 256); other shapes, ``return_logits``
    and ``force_simple`` take a CUDA-core kernel."""
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
    idx = torch.empty((T, topk), dtype=torch.int32, device=x.device)
    w = torch.empty((T, topk), dtype=torch.float32, device=x.device)
    b = None if bias is None else bias.to(device=x.device, dtype=torch.float32).contiguous()
    if T == 0:
        return (idx, w, torch.empty((0, E), dtype=torch.float32, device=x.device)) if return_logits else (idx, w)
    if not return_logits and not force_simple and D % 8 == 0 and E <= 256:
        _router_tensor_core(x, router_kmajor(w_router), b, topk, renormalize, idx, w, status)
        return idx, w
    fn = declare("b200_router_topk_simple",
                 [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                  C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p])
    logits = torch.empty((T, E), dtype=torch.float32, device=x.device) if return_logits else None
    rc = fn(ptr(x), ptr(w_router), ptr(b), T, D, E, topk, int(renormalize), ptr(idx), ptr(w),
            ptr(logits), stream_ptr(x))
    if rc != 0:
        raise RuntimeError(f"router_topk launch failed ({rc})")
    return (idx, w, logits) if return_logits else (idx, w)


def router_kmajor(w_router: torch.Tensor) -> torch.Tensor:
    """[D, E] -> contiguous [E, D] (the layout the tensor-core router reads).

    The transposed copy is cached on the tensor object itself together with the tensor's
    version counter, so an unchanged parameter is transposed once, an in-place update
    refreshes it, and the cache cannot outlive the tensor (an address-keyed cache would hand
    a new tensor that reuses freed memory somebody else's transposed weights)."""
    ver = w_router._version
    hit = getattr(w_router, "_b200_kmajor", None)
    if hit is not None and hit[0] == ver and hit[1].device == w_router.device:
        return hit[1]
    t = w_router.detach().t().contiguous()
    try:
        w_router._b200_kmajor = (ver, t)
    except AttributeError:      # exotic tensor subclasses without a __dict__: just do not cache
        pass
    return t


def _router_tensor_core(x, wr_kmajor, bias, topk, renormalize, idx, w, status=None) -> None:
    """Logits on tcgen05 (the grouped GEMM with one group and a narrow MMA), softmax and
    top-k in the epilogue: each epilogue thread owns one token's accumulator row."""
    from .. import _native as nv
    from .expert import sm_count
    T, D = x.shape
    E = wr_kmajor.shape[0]
    if status is None:
        status = default_status(x.device)
    ga = nv.GemmArgs()
    ga.num_groups, ga.N, ga.K, ga.n_out, ga.group_m = 1, E, D, E, 16
    ga.group_rows = None
    ga.single_group_rows = T
    ga.mma_n = max(16, (E + 15) // 16 * 16)
    ga.a_base = x.data_ptr()           # lets the kernel prefetch whole token rows into L2
    ga.status = status.data_ptr()
    ga.wait_budget_ns = int(2e9)
    ra = nv.RouterArgs()
    ra.num_experts, ra.topk, ra.renorm = E, topk, int(renormalize)
    ra.bias = None if bias is None else bias.data_ptr()
    ra.topk_idx, ra.topk_w = idx.data_ptr(), w.data_ptr()
    rc = nv.lib().b200_grouped_gemm(ptr(x), T, ptr(wr_kmajor), nv.EPI_ROUTER, 0, C.byref(ga), None, None,
                                    C.byref(ra), sm_count(x.device), stream_ptr(x))
    nv.check(rc, "tensor-core router launch")
