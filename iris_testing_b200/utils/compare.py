"""Comparison helpers for padded buffers and rank agreement (benchmark.py:31-35, 52-90)."""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def masked_stats(a: torch.Tensor, b: torch.Tensor, counts: torch.Tensor
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """max|a-b| and the two sums over the valid region only.

    a, b: [E, world, CAP, H]; counts: [E, world] valid rows per cell.
    Returns 0-dim fp32 tensors (max_diff, sum_a, sum_b)."""
    if a.shape != b.shape:
        raise ValueError("shape mismatch")
    cap = a.shape[2]
    m = torch.arange(cap, device=a.device).view(1, 1, cap)
    mask = (m < counts.to(a.device).unsqueeze(-1)).unsqueeze(-1)
    af, bf = a.float(), b.float()
    zero = torch.zeros((), device=a.device)
    diff = torch.where(mask, (af - bf).abs(), zero)
    return diff.max() if diff.numel() else zero, torch.where(mask, af, zero).sum(), torch.where(mask, bf, zero).sum()


def _reduce(x: torch.Tensor, op) -> torch.Tensor:
    y = x.clone()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(y, op=op)
    return y


def allreduce_max(x: torch.Tensor) -> torch.Tensor:
    return _reduce(x, dist.ReduceOp.MAX)


def allreduce_min(x: torch.Tensor) -> torch.Tensor:
    return _reduce(x, dist.ReduceOp.MIN)


def allreduce_sum(x: torch.Tensor) -> torch.Tensor:
    return _reduce(x, dist.ReduceOp.SUM)


def all_ranks_ok(ok: bool, device="cpu") -> bool:
    """True only if every rank passed ``ok=True``: lets all ranks leave a failed phase
    together instead of some of them blocking in the next collective."""
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    return bool(allreduce_min(flag).item() == 1)


def sync_and_check(ok: bool, device="cpu") -> bool:
    """Agreement, then a barrier only when everybody is healthy."""
    good = all_ranks_ok(ok, device)
    if good and dist.is_available() and dist.is_initialized():
        dist.barrier()
    return good
