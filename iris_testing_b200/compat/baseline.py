"""Names and call shapes of the reference's ``baseline.py`` (baseline.py:30-305)."""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..parallel.baseline_nccl import (ExchangeBuffers as BaselineBuffers, exchange_counts,  # noqa: F401
                                      exchange_payload, init_baseline_buffers,
                                      relayout_to_token_buf, run_baseline)


def exchange_counts_a2a(send_counts: torch.Tensor, buffers: BaselineBuffers, strict_capacity: bool,
                        capacity: int) -> torch.Tensor:
    """recv_counts[src, e] from send_counts[dst, e]; optionally fail when a cell exceeds ``capacity``."""
    recv = exchange_counts(send_counts)
    buffers.recv_counts = recv
    if strict_capacity and int(recv.max().item()) > capacity:
        raise ValueError(f"recv_counts max={int(recv.max().item())} exceeds capacity={capacity}")
    return recv


def exchange_payload_a2a(send_payload: torch.Tensor, send_counts: torch.Tensor,
                         recv_counts: torch.Tensor, buffers: BaselineBuffers):
    """Ragged payload all-to-all; returns (recv_payload_flat, in_splits, out_splits) as tensors."""
    out, ins, outs = exchange_payload(send_payload, send_counts, recv_counts, buffers)
    dev = send_payload.device
    return out, torch.tensor(ins, dtype=torch.int32, device=dev), torch.tensor(outs, dtype=torch.int32, device=dev)


def reorder_flat_to_token_buf(recv_payload_flat: torch.Tensor, recv_counts: torch.Tensor, capacity: int,
                              token_buf_out: torch.Tensor) -> torch.Tensor:
    return relayout_to_token_buf(recv_payload_flat, recv_counts, capacity, token_buf_out)


def run_baseline_ref(rank: int, world_size: int, e_local: int, capacity: int, hidden_dim: int,
                     send_payload: torch.Tensor, send_counts: torch.Tensor, buffers: BaselineBuffers,
                     do_reorder: bool = False, profile: bool = True, strict_capacity: bool = True,
                     barrier: bool = True
                     ) -> Tuple[Optional[torch.Tensor], Dict[str, float], Dict[str, object]]:
    """Same arguments and return triple as the reference's runner (baseline.py:227-305)."""
    import torch.distributed as dist
    if send_counts.shape != (world_size, e_local):
        raise ValueError(f"send_counts shape {tuple(send_counts.shape)} != ({world_size},{e_local})")
    if barrier and dist.is_initialized():
        dist.barrier()
    token_buf, timings, meta = run_baseline(send_payload, send_counts, capacity, buffers, do_reorder)
    if strict_capacity and int(meta["recv_counts"].max().item()) > capacity:
        raise ValueError("recv_counts exceeds capacity (strict_capacity=True)")
    meta["total_send"] = sum(meta["in_splits"])
    meta["total_recv"] = sum(meta["out_splits"])
    return token_buf, timings, meta
