"""CPU / gloo expert-parallel backend (plumbing oracle, no GPU needed).

Implements the reference's *stated* exchange scheme (README.md:5-7): count the
tokens routed between every rank pair, let M be the maximum over all pairs,
and send exactly M rows -- zero padded -- between each pair with a fixed-size
``all_to_all_single``; then run the local experts on the valid rows, return the
results with a second fixed-size all-to-all and combine them with the top-k
weights.  Works with any ``torch.distributed`` backend that has
``all_to_all_single`` (gloo on CPU); with no process group it degrades to a
single rank.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist

from ..ops import cpu_ref
from ..ops.plan import make_plan
from ..ops.router import router_topk


def _world_rank(group=None) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def pair_message_rows(send_counts: torch.Tensor, group=None) -> int:
    """M = max over all (src, dst) pairs of rows sent (README.md:5-7); at least 1."""
    m = send_counts.sum(dim=1).max().to(torch.int64).reshape(1)
    world, _ = _world_rank(group)
    if world > 1:
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=group)
    return max(int(m.item()), 1)


def padded_exchange(payload: torch.Tensor, send_counts: torch.Tensor, group=None
                    ) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Fixed-size padded all-to-all of a (dst, expert)-packed payload.

    Returns (recv [world(src), M, H], recv_counts [world(src), e_local], M): rows
    ``recv[src, :recv_counts[src].sum()]`` are src's rows for this rank, expert-major;
    the rest is zero padding.
    """
    world, rank = _world_rank(group)
    H = payload.shape[1]
    M = pair_message_rows(send_counts, group)
    send = payload.new_zeros(world, M, H)
    sizes = send_counts.sum(dim=1).tolist()
    off = 0
    for d in range(world):
        send[d, :sizes[d]] = payload[off:off + sizes[d]]
        off += sizes[d]
    recv = torch.empty_like(send)
    recv_counts = torch.empty_like(send_counts)
    if world > 1:
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=group)
        dist.all_to_all_single(recv, send, group=group)
    else:
        recv.copy_(send)
        recv_counts.copy_(send_counts)
    return recv, recv_counts, M


def padded_return_exchange(results: torch.Tensor, group=None) -> torch.Tensor:
    """Mirror of :func:`padded_exchange`: results [world(src), M, H] go back to their sources."""
    world, _ = _world_rank(group)
    back = torch.empty_like(results)
    if world > 1:
        dist.all_to_all_single(back, results.contiguous(), group=group)
    else:
        back.copy_(results)
    return back


def local_experts(layer, rows: torch.Tensor, e: int) -> torch.Tensor:
    """Apply local expert ``e`` of ``layer`` to ``rows`` (fp32 math, result in rows.dtype)."""
    if rows.shape[0] == 0:
        return rows.new_zeros(0, layer.cfg.out_dim)
    w1, w3, w2 = layer.reference_weights()
    if layer.cfg.gated:
        out = cpu_ref.gated_mlp_ref(rows, w1[e], w3[e], w2[e], round_hidden=rows.dtype)
    else:
        out = rows.float() @ w1[e].float()
    return out.to(rows.dtype)


def moe_forward_gloo(layer, x: torch.Tensor, group=None) -> torch.Tensor:
    """Full distributed forward of ``layer`` on CPU tensors."""
    cfg = layer.cfg
    world, rank = _world_rank(group)
    if world != cfg.world_size:
        raise ValueError(f"process group has {world} ranks but the config says {cfg.world_size}")
    EL, k = cfg.e_local, cfg.topk
    idx, wgt = router_topk(x, layer.router, k, layer.router_bias, cfg.renormalize)
    plan = make_plan(idx, cfg.num_experts)
    payload = cpu_ref.pack_ref(x, plan.send_order, k)
    send_counts = plan.counts.view(world, EL)
    recv, recv_counts, M = padded_exchange(payload, send_counts, group)
    # local experts on the valid rows of every source block
    results = recv.new_zeros(world, M, cfg.out_dim)
    rc = recv_counts.tolist()
    for s in range(world):
        off = 0
        for e in range(EL):
            n = rc[s][e]
            results[s, off:off + n] = local_experts(layer, recv[s, off:off + n], e)
            off += n
    back = padded_return_exchange(results, group)          # [world(dst), M, out]
    # row j of the payload came back as back[dst, j - dst_offset[dst]]
    dst_off = cpu_ref.dst_offsets_ref(send_counts).long()
    sizes = send_counts.sum(dim=1).long()
    dst_of_row = torch.repeat_interleave(torch.arange(world), sizes)
    pos = torch.arange(payload.shape[0]) - dst_off[dst_of_row]
    returned = back[dst_of_row, pos]                        # [T*k, out] in payload order
    per_slot = returned[plan.dst_slot.long()].float() * wgt.reshape(-1, 1)
    layer.last_routing = (idx, wgt)
    layer.last_message_rows = M
    return per_slot.view(x.shape[0], k, -1).sum(dim=1).to(x.dtype)
