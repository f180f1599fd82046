"""Routing + packing front-end with the reference's return contract.

``route_and_pack_padding_free`` returns ``(send_payload, send_counts, dst_offsets,
dst_sizes)`` exactly as utils.py:176-246 does -- payload rows ordered by destination
rank, then local expert, stable in (token, top-k slot); a token routed to k experts
appears k times -- but builds them with the router / plan / pack kernels (or their
PyTorch restatements on CPU) instead of a Python loop with one ``.item()`` per copy.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import cpu_ref
from ..ops.plan import Plan, make_plan, pack_rows
from ..ops.router import router_topk


def build_expert_offsets(send_counts: torch.Tensor) -> torch.Tensor:
    """expert_offs[dst, e] = first row of expert e inside dst's block (int32)."""
    if send_counts.dtype != torch.int32:
        raise ValueError("send_counts must be int32")
    return cpu_ref.expert_offsets_ref(send_counts).contiguous()


def build_dst_offsets(send_counts: torch.Tensor) -> torch.Tensor:
    """dst_offsets[dst] = first payload row of destination dst (int32)."""
    return cpu_ref.dst_offsets_ref(send_counts).contiguous()


def route_and_pack(tokens: torch.Tensor, router: torch.Tensor, topk: int, world_size: int,
                   num_experts_total: int, bias: Optional[torch.Tensor] = None,
                   renormalize: bool = False):
    """Like :func:`route_and_pack_padding_free` but also returns what a combine needs:
    ``(send_payload, send_counts, dst_offsets, dst_sizes, topk_idx, topk_weight, plan)``."""
    if num_experts_total % world_size != 0:
        raise ValueError("num_experts_total must be divisible by world_size")
    e_local = num_experts_total // world_size
    idx, wgt = router_topk(tokens, router, topk, bias, renormalize)
    plan: Plan = make_plan(idx, num_experts_total)
    payload = pack_rows(tokens.contiguous(), plan.send_order, topk)
    send_counts = plan.counts.view(world_size, e_local)
    dst_sizes = send_counts.sum(dim=1).to(torch.int32)
    dst_offsets = build_dst_offsets(send_counts)
    return payload, send_counts, dst_offsets, dst_sizes, idx, wgt, plan


def route_and_pack_padding_free(tokens: torch.Tensor, router: torch.Tensor, topk: int,
                                world_size: int, num_experts_total: int
                                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(send_payload [sum_send, H], send_counts int32 [world, e_local],
    dst_offsets int32 [world], dst_sizes int32 [world])."""
    out = route_and_pack(tokens, router, topk, world_size, num_experts_total)
    return out[0], out[1], out[2], out[3]


def compute_capacity_from_pca(pca: torch.Tensor, group=None) -> int:
    """CAP = max(1, max over all ranks of max(pca)) (utils.py:118-121)."""
    cap = pca.max().to(torch.int32).reshape(1)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=group)
    return max(int(cap.item()), 1)


def compute_capacity_device(probe, send_counts: torch.Tensor) -> torch.Tensor:
    """Device-side capacity rule: int32 ``[CAP, M, max rows received, rows received here]``.

    ``CAP`` is the rule above (largest cell over all ranks), ``M`` the README's message size
    (largest number of rows any rank sends to any one rank, README.md:5-7).  ``probe`` is a
    :class:`~iris_testing_b200.parallel.padded_a2a.CapacityProbe`; nothing is copied to the
    host, so the result can size later launches from a graph or be read once with ``.tolist()``."""
    return probe.measure(send_counts.contiguous())
