"""Local expert layer: persistent grouped GEMM on tcgen05 tensor cores.

Reference: layers/expert.py:6-65 and the kernel text kernels.py:207-289 describe
a persistent grouped GEMM ``[m_e, H] x [H, F] -> [m_e, F]`` over the local
experts with ``m_e`` read from a device array (never wired up there).  Here it
is the tcgen05/TMEM kernel of csrc/grouped_gemm.cu, with an optional SiLU-gate
epilogue; ``expert`` keeps the reference's call shape.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _native as nv
from . import cpu_ref
from ._common import contiguous_bf16, default_status, ptr, require, stream_ptr, use_native

_SM_COUNT = {}


def sm_count(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def to_kmajor(weights: torch.Tensor) -> torch.Tensor:
    """[G, K, N] ("x @ W" layout, as the reference generates) -> [G, N, K] contiguous."""
    return weights.transpose(1, 2).contiguous()


def grouped_gemm(a: torch.Tensor, w_kmajor: torch.Tensor, group_rows: torch.Tensor, *,
                 epilogue: int = nv.EPI_STORE, out: Optional[torch.Tensor] = None,
                 status: Optional[torch.Tensor] = None, group_m: int = 0,
                 num_ctas: Optional[int] = None, wait_budget_ms: float = 2000.0,
                 cta_pair: Optional[bool] = None, l2_hints: int = 0, wide_tiles: int = 0,
                 epilogue_trace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[rows of group g] = a[rows of group g] @ w_kmajor[g].T   (bf16 in, fp32 accumulate).

    a          [M, K] bf16, groups packed back to back
    w_kmajor   [G, N, K] bf16
    group_rows int32 [G] on the device (rows per group; sum <= M)
    group_m    M-tiles per L2-blocking chunk; 0 picks about 48 MB of activations per chunk.
    cta_pair   True: two CTAs per MMA (tcgen05 cta_group::2, 256-row tiles); None picks it
               when the groups average at least 128 rows.
    wide_tiles CTA pairs only: 512-column tiles that use both TMEM accumulators at once (25 % fewer
               operand bytes per FLOP, but the epilogue is no longer hidden); 1 = on, 0 = off (default).
    epilogue   EPI_STORE -> out [M, N];  EPI_SILU_GATE -> out [M, N/2] where every
               256-row block of a group's weight holds 128 gate rows then 128 up rows.
    """
    require(a.dim() == 2 and w_kmajor.dim() == 3 and a.shape[1] == w_kmajor.shape[2],
            "grouped_gemm: a must be [M, K] and w_kmajor [G, N, K]")
    G, N, K = w_kmajor.shape
    gated = epilogue == nv.EPI_SILU_GATE
    n_out = N // 2 if gated else N
    if not use_native(a):
        ref = cpu_ref.grouped_linear_ref(a, w_kmajor.transpose(1, 2), group_rows.tolist())
        if gated:
            r = ref.view(a.shape[0], N // 256, 2, 128)
            ref = (torch.nn.functional.silu(r[:, :, 0]) * r[:, :, 1]).reshape(a.shape[0], n_out)
        res = ref.to(a.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res
    a = contiguous_bf16(a, "a")
    w_kmajor = contiguous_bf16(w_kmajor, "w_kmajor")
    require(group_rows.dtype == torch.int32 and group_rows.is_cuda and group_rows.numel() == G,
            "group_rows must be an int32 CUDA tensor with one entry per group")
    require(K % 8 == 0 and N % 8 == 0, "K and N must be multiples of 8")
    require(G <= nv.MAX_GROUPS, f"at most {nv.MAX_GROUPS} groups")
    if gated:
        require(N % 256 == 0, "the gated epilogue needs N (= 2 * ffn_dim) to be a multiple of 256")
    M = a.shape[0]
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=a.device)
    else:
        require(out.is_contiguous() and out.shape == (M, n_out) and out.dtype == torch.bfloat16,
                "out must be contiguous bf16 [M, n_out]")
    if M == 0:
        return out
    if status is None:
        status = default_status(a.device)
    ga = nv.GemmArgs()
    ga.num_groups, ga.N, ga.K, ga.n_out, ga.group_m = G, N, K, n_out, group_m
    ga.group_rows = group_rows.data_ptr()
    ga.out, ga.ldo = out.data_ptr(), n_out
    ga.status = status.data_ptr()
    ga.wait_budget_ns = int(wait_budget_ms * 1e6)
    if cta_pair is None:
        cta_pair = M >= 128 * G
    ga.cta_pair = int(bool(cta_pair))
    ga.l2_hints = int(l2_hints)
    ga.wide_tiles = int(wide_tiles)
    ga.dbg = None if epilogue_trace is None else epilogue_trace.data_ptr()   # int64 [8] profiling words
    ctas = num_ctas or sm_count(a.device)
    rc = nv.lib().b200_grouped_gemm(ptr(a), M, ptr(w_kmajor), epilogue, 0, C.byref(ga), None, None,
                                    None, ctas, stream_ptr(a))
    nv.check(rc, "grouped_gemm launch")
    return out


class Expert(torch.autograd.Function):
    """Per-device grouped Linear over the local experts (forward only, like the reference)."""

    @staticmethod
    def forward(ctx, tokens, weights, local_expert_cnt, aggregate_exp_cnt=None):
        # weights: [e_local, H, F] as produced by gen_local_weights (utils.py:248-261)
        if not tokens.is_cuda:
            return cpu_ref.grouped_linear_ref(tokens, weights, local_expert_cnt.tolist()).to(tokens.dtype)
        return grouped_gemm(tokens, to_kmajor(weights), local_expert_cnt.to(torch.int32))

    @staticmethod
    def backward(ctx, *grad_outputs):
        raise NotImplementedError("the expert layer is forward-only")


def expert(tokens: torch.Tensor, weights: torch.Tensor, local_expert_cnt: torch.Tensor,
           aggregate_exp_cnt: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``expert(tokens [S, H], weights [E, H, F], local_expert_cnt [E])`` -> [S, F].

    Same call shape as the reference's ``Expert.apply`` (layers/expert.py:6-15);
    ``aggregate_exp_cnt`` (the exclusive scan of the counts) is recomputed on the
    device and accepted only for signature compatibility.
    """
    return Expert.apply(tokens, weights, local_expert_cnt, aggregate_exp_cnt)
