"""Library all-to-all baseline (``torch.distributed.all_to_all_single``).

Two things live here:

* This package's own baseline path -- a functional equivalent of the reference's
  ``baseline.py`` (counts exchange baseline.py:79-117, ragged payload exchange
  baseline.py:121-173, re-layout baseline.py:178-222, timed runner
  baseline.py:227-305), written to work on NCCL *and* gloo so that it doubles as
  a CPU test oracle, and extended to a full layer (expert MLP, return
  all-to-all, weighted sum) in :class:`AllToAllMoEBaseline`.
* :class:`ReferenceLayerHarness`, which drives the *unmodified* reference modules
  (passed in by the caller) for the benchmark's reference arm.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ops import cpu_ref
from ..utils import gen


# --------------------------------------------------------------------------- own baseline
@dataclass
class ExchangeBuffers:
    recv_counts: torch.Tensor                       # int32 [world, e_local]
    recv_payload: Optional[torch.Tensor] = None     # [total_recv, H]
    token_buf: Optional[torch.Tensor] = None        # [e_local, world, CAP, H]
    in_splits: List[int] = field(default_factory=list)
    out_splits: List[int] = field(default_factory=list)


def init_baseline_buffers(world_size: int, e_local: int, capacity: int, hidden_dim: int,
                          token_dtype: torch.dtype, device, total_recv: int,
                          allocate_token_buf: bool = False) -> ExchangeBuffers:
    """Persistent buffers allocated once outside the timing loop (cf. baseline.py:44-74)."""
    return ExchangeBuffers(
        recv_counts=torch.empty((world_size, e_local), dtype=torch.int32, device=device),
        recv_payload=torch.empty((total_recv, hidden_dim), dtype=token_dtype, device=device),
        token_buf=(torch.empty((e_local, world_size, capacity, hidden_dim), dtype=token_dtype, device=device)
                   if allocate_token_buf else None))


def _world(group=None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def exchange_counts(send_counts: torch.Tensor, group=None) -> torch.Tensor:
    """send_counts [world(dst), e_local] -> recv_counts [world(src), e_local]."""
    if send_counts.dtype != torch.int32:
        raise ValueError("send_counts must be int32")
    recv = torch.empty_like(send_counts)
    if _world(group) > 1:
        dist.all_to_all_single(recv, send_counts.contiguous(), group=group)
    else:
        recv.copy_(send_counts)
    return recv


def exchange_payload(payload: torch.Tensor, send_counts: torch.Tensor, recv_counts: torch.Tensor,
                     buffers: Optional[ExchangeBuffers] = None, group=None
                     ) -> Tuple[torch.Tensor, List[int], List[int]]:
    """Ragged all-to-all of the packed payload.  Split sizes are read back to the host
    (one synchronisation), as any ``all_to_all_single`` with uneven splits requires."""
    splits = torch.stack([send_counts.sum(dim=1), recv_counts.sum(dim=1)]).to("cpu").tolist()
    in_splits, out_splits = [int(v) for v in splits[0]], [int(v) for v in splits[1]]
    total = sum(out_splits)
    out = None if buffers is None else buffers.recv_payload
    if out is None or out.shape[0] != total or out.shape[1] != payload.shape[1]:
        out = payload.new_empty((total, payload.shape[1]))
        if buffers is not None:
            buffers.recv_payload = out
    if _world(group) > 1:
        dist.all_to_all_single(out, payload, output_split_sizes=out_splits,
                               input_split_sizes=in_splits, group=group)
    else:
        out.copy_(payload)
    if buffers is not None:
        buffers.in_splits, buffers.out_splits = in_splits, out_splits
    return out, in_splits, out_splits


def relayout_to_token_buf(recv_payload: torch.Tensor, recv_counts: torch.Tensor, capacity: int,
                          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Flat (src, expert)-packed rows -> ``[e_local, world, CAP, H]`` with zero padding,
    vectorised (one scatter instead of a Python loop over cells)."""
    world, e_local = recv_counts.shape
    H = recv_payload.shape[1]
    if out is None:
        out = recv_payload.new_zeros(e_local, world, capacity, H)
    else:
        out.zero_()
    c = recv_counts.reshape(-1).long()                         # cell order: (src, e)
    if int(c.max().item()) > capacity:
        raise ValueError("a (src, expert) cell exceeds the capacity")
    cell = torch.repeat_interleave(torch.arange(c.numel(), device=c.device), c)
    start = torch.cumsum(c, 0) - c
    m = torch.arange(cell.numel(), device=c.device) - start[cell]
    src, e = cell // e_local, cell % e_local
    out.view(-1, H)[(e * world + src) * capacity + m] = recv_payload
    return out


def run_baseline(payload: torch.Tensor, send_counts: torch.Tensor, capacity: int,
                 buffers: Optional[ExchangeBuffers] = None, do_reorder: bool = False, group=None
                 ) -> Tuple[Optional[torch.Tensor], Dict[str, float], Dict[str, object]]:
    """Counts exchange then payload exchange, each timed (CUDA events on GPU, wall clock on CPU)."""
    timings: Dict[str, float] = {}

    def timed(name, fn):
        if payload.is_cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            r = fn()
            b.record()
            b.synchronize()
            timings[name] = a.elapsed_time(b)
        else:
            import time
            t = time.perf_counter()
            r = fn()
            timings[name] = (time.perf_counter() - t) * 1e3
        return r

    recv_counts = timed("step1_ms", lambda: exchange_counts(send_counts, group))
    if buffers is None:
        buffers = ExchangeBuffers(recv_counts)
    buffers.recv_counts = recv_counts
    recv, ins, outs = timed("step2_ms",
                            lambda: exchange_payload(payload, send_counts, recv_counts, buffers, group))
    token_buf = None
    timings["reorder_ms"] = 0.0
    if do_reorder:
        token_buf = timed("reorder_ms",
                          lambda: relayout_to_token_buf(recv, recv_counts, capacity, buffers.token_buf))
        buffers.token_buf = token_buf
    meta = dict(recv_counts=recv_counts, in_splits=ins, out_splits=outs, recv_payload=recv)
    return token_buf, timings, meta


class AllToAllMoEBaseline:
    """Full MoE layer on library collectives: route, pack, all-to-all, per-expert
    matmuls, return all-to-all, weighted sum.  Works with NCCL (GPU) and gloo (CPU)."""

    def __init__(self, layer, group=None) -> None:
        self.layer = layer
        self.group = group
        self._weights = None      # x @ W layouts, materialised once

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        layer, cfg = self.layer, self.layer.cfg
        world, k, EL = cfg.world_size, cfg.topk, cfg.e_local
        idx, wgt = cpu_ref.router_topk_ref(x, layer.router, k, layer.router_bias, cfg.renormalize)
        plan = cpu_ref.plan_ref(idx, cfg.num_experts)
        payload = cpu_ref.pack_ref(x, plan.send_order, k)
        send_counts = plan.counts.view(world, EL)
        recv_counts = exchange_counts(send_counts, self.group)
        recv, ins, outs = exchange_payload(payload, send_counts, recv_counts, None, self.group)
        if self._weights is None:
            self._weights = layer.reference_weights()
        w1, w3, w2 = self._weights
        out = recv.new_empty(recv.shape[0], cfg.out_dim)
        rc = recv_counts.tolist()
        off = 0
        for s in range(world):
            for e in range(EL):
                n = rc[s][e]
                rows = recv[off:off + n]
                if cfg.gated:
                    h = F.silu(rows @ w1[e]) * (rows @ w3[e])
                    out[off:off + n] = h @ w2[e]
                else:
                    out[off:off + n] = rows @ w1[e]
                off += n
        back = out.new_empty(payload.shape[0], cfg.out_dim)
        if world > 1:
            dist.all_to_all_single(back, out, output_split_sizes=ins, input_split_sizes=outs,
                                   group=self.group)
        else:
            back.copy_(out)
        per_slot = back[plan.dst_slot.long()].float() * wgt.reshape(-1, 1)
        return per_slot.view(x.shape[0], k, -1).sum(dim=1).to(x.dtype)


# --------------------------------------------------------------------------- reference arm
class ReferenceLayerHarness:
    """One MoE layer step built on the UNMODIFIED reference modules.

    ``ref_baseline`` / ``ref_utils`` are the reference's ``baseline.py`` and ``utils.py``
    imported from its installed copy.  Routing and packing use the reference's own
    ``route_and_pack_padding_free`` (a Python loop; run once per input before timing, as
    the reference's benchmark does); the timed step is the reference's
    ``run_baseline_ref`` (counts + payload ``all_to_all_single``), followed by what the
    reference lacks, written in plain PyTorch: the expert MLP (``torch.matmul``), the
    return ``all_to_all_single`` and the weighted ``index_add_``.  None of this package's
    kernels run here.
    """

    def __init__(self, ref_baseline, ref_utils, model: str, batch: int, seq: int, seed: int,
                 rank: int, world: int, dev: torch.device) -> None:
        from ..config import preset
        self.rb, self.ru = ref_baseline, ref_utils
        cfg = preset(model, world_size=world)
        self.cfg, self.rank, self.world, self.dev = cfg, rank, world, dev
        D, EL, k = cfg.hidden_dim, cfg.e_local, cfg.topk
        T = batch * seq
        self.T = T
        dt = torch.bfloat16
        self.router = gen.gen_router(D, cfg.num_experts, dt, dev, seed, std=None)
        self.w1, self.w3, self.w2 = gen.gen_gated_expert_weights(EL, D, cfg.ffn_dim, dt, dev, seed, rank)
        self.inputs = []
        for i in range(2):
            x = gen.gen_local_tokens(batch, seq, D, dt, dev, seed + 1000 * i, rank, "normal")
            payload, send_counts, _, _ = ref_utils.route_and_pack_padding_free(
                x, self.router, k, world, cfg.num_experts)
            send_counts = send_counts.to(torch.int32).contiguous()
            # the reference discards the routing weights; recompute them with its formula
            probs = F.softmax(torch.einsum("th,he->te", x, self.router), dim=-1)
            vals, idx = torch.topk(probs, k, dim=-1)
            order = torch.sort(idx.reshape(-1), stable=True).indices      # payload row -> flat slot
            gathered = [torch.zeros_like(send_counts) for _ in range(world)]
            dist.all_gather(gathered, send_counts)
            counts_all = torch.stack(gathered)                             # [src, dst, e]
            recv_counts = counts_all[:, rank, :].contiguous()              # [src, e]
            cap = max(int(counts_all.max().item()), 1)
            total_recv = int(recv_counts.sum().item())
            bufs = ref_baseline.init_baseline_buffers(world, EL, cap, D, dt, dev, total_recv,
                                                      allocate_token_buf=False)
            # rows arrive (src, expert)-major; experts want them expert-major
            cell_e = torch.arange(EL, device=dev).repeat(world)
            row_e = torch.repeat_interleave(cell_e, recv_counts.reshape(-1).long())
            perm = torch.sort(row_e, stable=True).indices
            self.inputs.append(dict(
                x=x, x_host=x.cpu().pin_memory(), payload=payload, send_counts=send_counts,
                token_of_row=(order // k), w_of_row=vals.reshape(-1)[order].to(dt).unsqueeze(1),
                cap=cap, bufs=bufs, perm=perm if EL > 1 else None,
                rows_per_expert=recv_counts.sum(dim=0).tolist(),
                in_splits=send_counts.sum(dim=1).tolist(), out_splits=recv_counts.sum(dim=1).tolist()))
        self.h2d_bytes = T * D * 2

    def load_from_host(self, i: int) -> None:
        """H2D of step i's tokens from pinned memory, then a vectorised on-device pack
        (kinder to the reference than its Python packer, which takes seconds)."""
        inp = self.inputs[i]
        inp["x"].copy_(inp["x_host"], non_blocking=True)
        inp["payload"] = inp["x"].index_select(0, inp["token_of_row"])

    @torch.no_grad()
    def step(self, i: int) -> torch.Tensor:
        inp, cfg = self.inputs[i], self.cfg
        _, _, meta = self.rb.run_baseline_ref(
            rank=self.rank, world_size=self.world, e_local=cfg.e_local, capacity=inp["cap"],
            hidden_dim=cfg.hidden_dim, send_payload=inp["payload"], send_counts=inp["send_counts"],
            buffers=inp["bufs"], do_reorder=False, profile=False, strict_capacity=False, barrier=False)
        recv = inp["bufs"].recv_payload_flat
        rows = recv if inp["perm"] is None else recv.index_select(0, inp["perm"])
        out_sorted = torch.empty_like(rows)
        off = 0
        for e, n in enumerate(inp["rows_per_expert"]):
            r = rows[off:off + n]
            h = F.silu(r @ self.w1[e]) * (r @ self.w3[e])
            torch.matmul(h, self.w2[e], out=out_sorted[off:off + n])
            off += n
        if inp["perm"] is None:
            out = out_sorted
        else:
            out = torch.empty_like(out_sorted)
            out.index_copy_(0, inp["perm"], out_sorted)
        back = torch.empty_like(inp["payload"])
        dist.all_to_all_single(back, out, output_split_sizes=inp["in_splits"],
                               input_split_sizes=inp["out_splits"])
        y = torch.zeros((self.T, cfg.hidden_dim), dtype=back.dtype, device=self.dev)
        y.index_add_(0, inp["token_of_row"], back * inp["w_of_row"])
        return y
