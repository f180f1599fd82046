"""Plain-PyTorch restatements of every op (the oracles of the test-suite).

Each function states one kernel's semantics with ordinary tensor ops, in fp32
where arithmetic is involved.  They run on any device, never call the native
library, and are also what the CPU/gloo plumbing backend executes.
Reference semantics: router utils.py:201-202, expert->rank map and stable
(token, slot) order utils.py:210-219, layouts layers/all_to_all.py:19-45,
shuffle order layers/token_shuffle.py:31-56, expert oracle unit_tests.py:224-237.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


def router_topk_ref(x: torch.Tensor, w_router: torch.Tensor, topk: int,
                    bias: Optional[torch.Tensor] = None, renormalize: bool = False
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax(x @ w_router + bias) then top-k.  Returns (idx int32 [T,k], weight fp32 [T,k]).

    ``w_router`` is [hidden, experts].  Ties resolve to the lower expert index.
    """
    logits = x.float() @ w_router.float()
    if bias is not None:
        logits = logits + bias.float()
    probs = F.softmax(logits, dim=-1)
    # stable descending sort => lower index first on ties
    order = torch.sort(probs, dim=-1, descending=True, stable=True)
    idx = order.indices[:, :topk]
    w = order.values[:, :topk]
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return idx.to(torch.int32).contiguous(), w.contiguous()


@dataclass
class PlanRef:
    counts: torch.Tensor          # int32 [E]   rows routed to each (global) expert
    bucket_start: torch.Tensor    # int32 [E+1] exclusive scan of counts
    send_order: torch.Tensor      # int32 [T*k] flat (t*k+slot) sorted by (expert, t, slot)
    dst_slot: torch.Tensor        # int32 [T*k] inverse of send_order
    rank_in_bucket: torch.Tensor  # int32 [T*k]


def plan_ref(topk_idx: torch.Tensor, num_experts: int) -> PlanRef:
    """Bucket every routed copy by expert, keeping (token, slot) order inside a bucket."""
    flat = topk_idx.reshape(-1).to(torch.int64)
    n = flat.numel()
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    start = torch.zeros(num_experts + 1, dtype=torch.int64, device=flat.device)
    start[1:] = torch.cumsum(counts, 0)
    order = torch.sort(flat, stable=True).indices
    dst_slot = torch.empty(n, dtype=torch.int64, device=flat.device)
    dst_slot[order] = torch.arange(n, device=flat.device)
    rank = dst_slot - start[flat]
    i32 = torch.int32
    return PlanRef(counts.to(i32), start.to(i32), order.to(i32), dst_slot.to(i32), rank.to(i32))


def pack_ref(x: torch.Tensor, send_order: torch.Tensor, topk: int) -> torch.Tensor:
    """payload[j] = x[send_order[j] // topk] (a token routed to k experts appears k times)."""
    return x[(send_order.long() // topk)]


def expert_offsets_ref(send_counts: torch.Tensor) -> torch.Tensor:
    """expert_offs[dst, e]: first row of expert e inside the block sent to dst (utils.py:20-31)."""
    c = send_counts.to(torch.int64)
    return (torch.cumsum(c, dim=1) - c).to(torch.int32)


def dst_offsets_ref(send_counts: torch.Tensor) -> torch.Tensor:
    """dst_offsets[dst]: first payload row of destination dst (benchmark.py:44-49)."""
    s = send_counts.to(torch.int64).sum(dim=1)
    return (torch.cumsum(s, 0) - s).to(torch.int32)


def padded_dispatch_ref(payloads: Sequence[torch.Tensor], send_counts: Sequence[torch.Tensor],
                        cap: int) -> Tuple[List[torch.Tensor], List[torch.Tensor]]:
    """All ranks at once.  payloads[src] is [sum_send, H] packed by (dst, expert).

    Returns (token_bufs, pcas): token_bufs[dst][e, src, m, :] and pcas[dst][e, src]
    exactly as the padded dispatch kernel leaves them (padding rows are zero).
    """
    world = len(payloads)
    e_local = send_counts[0].shape[1]
    H = payloads[0].shape[1]
    bufs = [torch.zeros(e_local, world, cap, H, dtype=payloads[0].dtype, device=payloads[0].device)
            for _ in range(world)]
    pcas = [torch.zeros(e_local, world, dtype=torch.int32, device=payloads[0].device)
            for _ in range(world)]
    for src in range(world):
        off = 0
        sc = send_counts[src].tolist()
        for dst in range(world):
            for e in range(e_local):
                n = int(sc[dst][e])
                pcas[dst][e, src] = n
                m = min(n, cap)
                bufs[dst][e, src, :m] = payloads[src][off:off + m]
                off += n
    return bufs, pcas


def shuffle_ref(token_buf: torch.Tensor, pca: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Drop padding: rows ordered by (expert, src, arrival).  Returns (packed, rows per expert)."""
    e_local, world, cap, H = token_buf.shape
    parts = []
    for e in range(e_local):
        for s in range(world):
            parts.append(token_buf[e, s, :min(int(pca[e, s]), cap)])
    packed = torch.cat(parts, 0) if parts else token_buf.new_zeros(0, H)
    group_rows = pca.clamp(max=cap).sum(dim=1).to(torch.int32)
    return packed, group_rows


def unshuffle_ref(packed: torch.Tensor, pca: torch.Tensor, cap: int) -> torch.Tensor:
    """Inverse of :func:`shuffle_ref` (padding rows zero)."""
    e_local, world = pca.shape
    out = packed.new_zeros(e_local, world, cap, packed.shape[1])
    off = 0
    for e in range(e_local):
        for s in range(world):
            n = min(int(pca[e, s]), cap)
            out[e, s, :n] = packed[off:off + n]
            off += n
    return out


def silu_gate_ref(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (F.silu(gate.float()) * up.float())


def grouped_linear_ref(tokens: torch.Tensor, weights: torch.Tensor, group_rows) -> torch.Tensor:
    """Per-expert dense matmul over a packed buffer.  weights: [G, K, N] ("x @ W")."""
    out = torch.zeros(tokens.shape[0], weights.shape[2], dtype=torch.float32, device=tokens.device)
    off = 0
    for g, n in enumerate([int(v) for v in group_rows]):
        if n:
            out[off:off + n] = tokens[off:off + n].float() @ weights[g].float()
        off += n
    return out


def gated_mlp_ref(x: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor,
                  round_hidden: Optional[torch.dtype] = None) -> torch.Tensor:
    """(silu(x W1) * (x W3)) W2 in fp32; ``round_hidden`` rounds the hidden activation
    to that dtype first, as a kernel that stores it in bf16 does."""
    h = F.silu(x.float() @ w1.float()) * (x.float() @ w3.float())
    if round_hidden is not None:
        h = h.to(round_hidden).float()
    return h @ w2.float()


def dense_moe_ref(x: torch.Tensor, w_router: torch.Tensor, topk: int, *,
                  w1: Optional[torch.Tensor] = None, w3: Optional[torch.Tensor] = None,
                  w2: Optional[torch.Tensor] = None, w_single: Optional[torch.Tensor] = None,
                  bias: Optional[torch.Tensor] = None, renormalize: bool = False,
                  round_hidden: Optional[torch.dtype] = None,
                  routing: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> torch.Tensor:
    """Single-process dense MoE layer over ALL experts (fp32).

    Gated: w1, w3 [E, D, F], w2 [E, F, D].  Single Linear: w_single [E, D, N].
    y[t] = sum_slot weight[t, slot] * expert_{idx[t, slot]}(x[t]).
    ``routing`` = (idx [T, k], weight [T, k]) replaces the oracle's own router.
    """
    idx, wgt = routing if routing is not None else router_topk_ref(x, w_router, topk, bias, renormalize)
    E = (w1 if w1 is not None else w_single).shape[0]
    out_dim = w2.shape[2] if w2 is not None else w_single.shape[2]
    y = torch.zeros(x.shape[0], out_dim, dtype=torch.float32, device=x.device)
    for e in range(E):
        tok, slot = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        if w_single is not None:
            oe = xe.float() @ w_single[e].float()
        else:
            oe = gated_mlp_ref(xe, w1[e], w3[e], w2[e], round_hidden)
        y.index_add_(0, tok, oe * wgt[tok, slot].unsqueeze(1))
    return y


def interleave_gate_up(w1: torch.Tensor, w3: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[E, D, F] x2  ->  [E, 2F, D] "K-major" weight whose rows alternate
    ``block`` gate features (from W1) and ``block`` up features (from W3): the
    layout the SiLU-gated GEMM epilogue expects.  F must be a multiple of ``block``."""
    E, D, Fdim = w1.shape
    if Fdim % block != 0:
        raise ValueError(f"ffn_dim {Fdim} must be a multiple of {block}")
    g = w1.transpose(1, 2).reshape(E, Fdim // block, 1, block, D)
    u = w3.transpose(1, 2).reshape(E, Fdim // block, 1, block, D)
    return torch.cat([g, u], dim=2).reshape(E, 2 * Fdim, D).contiguous()


def clear_routing_mask(x: torch.Tensor, w_router: torch.Tensor, topk: int,
                       bias: Optional[torch.Tensor] = None, min_gap: float = 1e-6) -> torch.Tensor:
    """bool [T]: tokens whose top-k choice is unambiguous -- every gap between consecutive sorted
    probabilities down to the (k+1)-th exceeds ``min_gap``.  On the other tokens two correct
    routers may legitimately pick different experts (or order them differently)."""
    logits = x.float() @ w_router.float()
    if bias is not None:
        logits = logits + bias.float()
    srt = torch.sort(F.softmax(logits, dim=-1), dim=-1, descending=True).values
    if srt.shape[1] <= topk:
        return torch.ones(x.shape[0], dtype=torch.bool, device=x.device)
    return (srt[:, :topk] - srt[:, 1:topk + 1]).min(dim=1).values > min_gap


def compare_with_dense(y: torch.Tensor, x: torch.Tensor, w_router: torch.Tensor, topk: int, kernel_idx,
                       *, bias=None, renormalize: bool = False, tol: float = 1e-2, **weights) -> dict:
    """Compare a layer output with :func:`dense_moe_ref`, tokens with an ambiguous top-k set aside.

    Returns ``max_rel_err`` (largest |y - ref| over the clear tokens, relative to max |ref|),
    the same over all tokens, the number of ambiguous tokens, whether the kernel's expert sets
    equal the oracle's on every clear token, and ``ok``."""
    if x.shape[0] == 0:           # a rank without tokens: nothing to compare
        return dict(max_rel_err=0.0, max_rel_err_all_tokens=0.0, ambiguous_tokens=0, tokens=0, routing_ok=True,
                    tol=tol, ok=bool(y.shape[0] == 0))
    ref = dense_moe_ref(x, w_router, topk, bias=bias, renormalize=renormalize, **weights)
    clear = clear_routing_mask(x, w_router, topk, bias)
    ridx, _ = router_topk_ref(x, w_router, topk, bias, renormalize)
    same = (torch.sort(kernel_idx.long(), dim=1).values == torch.sort(ridx.long(), dim=1).values).all(dim=1)
    scale = float(ref.abs().max().clamp_min(1e-20))
    diff = (y.float() - ref).abs().max(dim=1).values if y.numel() else torch.zeros(0, device=y.device)
    err_clear = float(diff[clear].max()) / scale if bool(clear.any()) else 0.0
    err_all = float(diff.max()) / scale if diff.numel() else 0.0
    routing_ok = bool(same[clear].all()) if bool(clear.any()) else True
    return dict(max_rel_err=err_clear, max_rel_err_all_tokens=err_all, ambiguous_tokens=int((~clear).sum()),
                tokens=int(x.shape[0]), routing_ok=routing_ok, tol=tol,
                ok=bool(routing_ok and err_clear <= tol))
