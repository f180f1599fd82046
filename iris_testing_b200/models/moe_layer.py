"""``MoELayer``: one expert-parallel Mixture-of-Experts block.

Forward pass on B200 (six launches, no host synchronisation):

1. router          softmax -> top-k (indices + weights)
2. plan            per-expert counts, stable bucket ranks, send order; pushes this
                   rank's counts to every peer
3. dispatch+GEMM1  ONE kernel: sender warps store routed token rows into the owning
                   rank's receive buffer over NVLink and signal per M-tile, while the
                   tcgen05 grouped GEMM of the same kernel consumes tiles as they land
                   (SiLU-gate epilogue -> hidden activation, local HBM)
4. GEMM2+combine   ONE kernel: second grouped GEMM whose epilogue scales each row by
                   its top-k weight and stores it straight into the source rank's return
                   buffer (at the row's send-order position), counting arrivals there
5. slot reduce     waits for the arrivals, gathers and sums the k results per token, retires the
                   iteration (re-arms counters, tells peers the parity slot is free)

The reference project wires none of this together (its intended forward pass is
reconstructed from layers/all_to_all.py, layers/token_shuffle.py, layers/expert.py);
router math follows utils.py:201-202 and the expert->rank map utils.py:216-218.

On CPU tensors the layer runs the same math through PyTorch (and gloo when a
process group is up), which is what the plumbing tests use.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import _native as nv
from ..config import MoEConfig
from ..ops import cpu_ref
from ..ops._common import declare, ptr, stream_ptr
from ..ops.expert import sm_count
from ..ops.plan import Plan, PlanPushArgs, make_plan
from ..ops.router import router_kmajor, router_topk
from ..utils import gen

_NVTX = os.getenv("B200MOE_NVTX", "0") == "1"   # NVTX range around every forward
_CANARY = 0x5A5A5A5A
BM = 128          # rows per GEMM tile
BN = 256          # weight rows per GEMM tile


class RetireArgs(C.Structure):
    _fields_ = [
        ("world", C.c_int), ("rank", C.c_int),
        ("iter_done_value", C.c_uint32),
        ("peer_iter_done", C.c_ulonglong * nv.MAX_WORLD),
        ("ready_counters", C.c_void_p),
        ("num_ready", C.c_int),
        ("ticket", C.c_void_p),
        ("iter_ptr", C.c_void_p),
        ("stride_ready", C.c_ulonglong),
    ]


def heap_bytes_needed(cfg: MoEConfig, max_tokens: int, cap_rows: Optional[int] = None) -> int:
    """Symmetric-heap bytes one ``MoELayer`` of this shape allocates (plus slack)."""
    W, k, D = cfg.world_size, cfg.topk, cfg.hidden_dim
    cap = cap_rows if cap_rows is not None else default_cap_rows(cfg, max_tokens)
    mt = cap // BM + cfg.e_local + 1
    total = 2 * cap * D * 2 + 2 * cap * 8 + 2 * mt * 4 + 2 * W * cfg.num_experts * 4
    total += max_tokens * k * cfg.out_dim * 2
    return total + (1 << 20)


def default_cap_rows(cfg: MoEConfig, max_tokens: int) -> int:
    """Receive capacity (rows) of every rank.

    Balanced routing gives a rank ``max_tokens * topk`` rows; ``capacity_factor`` (default
    1.25) scales that, plus one tile of slack per local expert.  ``capacity_factor=None``
    sizes for the worst case (every routed copy of every rank lands on one rank), which can
    never overflow but costs ``world_size`` times the memory.  A step that needs more rows
    than the capacity reports an overflow with the number needed;
    :meth:`MoELayer.forward_checked` grows the buffers and repeats the step."""
    worst = cfg.world_size * max_tokens * cfg.topk
    if cfg.capacity_factor is None:
        rows = worst
    else:
        rows = min(worst, int(cfg.capacity_factor * max_tokens * cfg.topk) + cfg.e_local * BM)
    return (max(rows, BM) + BM - 1) // BM * BM


class MoELayer(nn.Module):
    """Expert-parallel MoE block: ``y = sum_k w_k * expert_k(x)``.

    Parameters live in kernel-friendly ("K-major") layouts:

    * ``router``  [D, E]                      (reference layout, utils.py:156-173)
    * ``w13``     [e_local, 2F, D]  gated: blocks of 128 gate rows / 128 up rows
                  [e_local, N, D]   single Linear (``cfg.gated == False``)
    * ``w2``      [e_local, D, F]   gated only

    ``load_reference_weights`` / ``reference_weights`` convert from / to the
    ``x @ W`` layouts ([e, D, F], [e, D, F], [e, F, D]).
    """

    def __init__(self, cfg: MoEConfig, max_tokens: int, heap=None, device=None, seed: int = 0,
                 rank: Optional[int] = None, router_std: Optional[float] = None,
                 cap_rows: Optional[int] = None, num_ctas: Optional[int] = None,
                 debug_canaries: bool = False) -> None:
        super().__init__()
        self.cfg = cfg
        self.max_tokens = int(max_tokens)
        self.heap = heap
        if rank is None:
            rank = heap.rank if heap is not None else (
                dist.get_rank() if dist.is_available() and dist.is_initialized() else 0)
        self.rank = rank
        device = torch.device(device) if device is not None else (
            heap.device if heap is not None else torch.device("cpu"))
        D, F, EL = cfg.hidden_dim, cfg.ffn_dim, cfg.e_local
        self.router = nn.Parameter(gen.gen_router(D, cfg.num_experts, cfg.dtype, device, seed,
                                                  std=router_std), requires_grad=False)
        self.router_bias: Optional[torch.Tensor] = None
        if cfg.gated:
            if F % 128 != 0:
                raise ValueError("gated experts need ffn_dim to be a multiple of 128")
            w1, w3, w2 = gen.gen_gated_expert_weights(EL, D, F, cfg.dtype, device, seed, rank)
            self.w13 = nn.Parameter(cpu_ref.interleave_gate_up(w1, w3), requires_grad=False)
            self.w2 = nn.Parameter(w2.transpose(1, 2).contiguous(), requires_grad=False)
        else:
            w = gen.gen_local_weights(EL, D, cfg.out_dim, cfg.dtype, device, seed, rank)
            self.w13 = nn.Parameter(w.transpose(1, 2).contiguous(), requires_grad=False)
            self.w2 = None
        self._iteration = 0
        self._engine_ready = False
        self._cap_rows = cap_rows
        self._num_ctas = num_ctas       # persistent grid of the GEMM kernels (default: one CTA per SM)
        self._debug_canaries = bool(debug_canaries)
        self._canaries = []
        # L2 eviction-priority hints of the two GEMM kernels (bit 0: keep activations, bit 1: stream
        # weights, bit 2: stream the hidden output); B200MOE_L2_HINTS="h1,h2" overrides
        env = os.getenv("B200MOE_L2_HINTS")
        self.l2_hints = tuple(int(v) for v in env.split(",")) if env else (0, 0)
        self.group_m = (0, 0)           # M-tiles per L2 chunk of the two GEMM kernels (0: automatic)
        self.tma_store = os.getenv("B200MOE_TMA_STORE", "1") != "0"   # hidden output through bulk tensor stores
        # 512-column tiles (both TMEM accumulators per tile) in the first / second GEMM kernel:
        # 1 on, 0 off; B200MOE_WIDE_TILES="w1,w2" overrides
        env = os.getenv("B200MOE_WIDE_TILES")
        self.wide_tiles = tuple(int(v) for v in env.split(",")) if env else (0, 0)
        self.small_path = os.getenv("B200MOE_SMALL_PATH", "1") != "0"
        self.drop_signal = False        # fault-injection aid for the timeout test
        self.profile = False            # record CUDA events between the phases of forward()
        self.phase_events = []
        self.trace_arrivals = False     # record when each received M-tile became usable (fused kernel)
        self._trace = None
        if device.type == "cuda":
            if heap is None:
                raise ValueError("a SymmetricHeap is required on CUDA")
            self._build_engine()

    # ---------------------------------------------------------------- weights
    def load_reference_weights(self, w1: torch.Tensor, w3: Optional[torch.Tensor] = None,
                               w2: Optional[torch.Tensor] = None) -> None:
        with torch.no_grad():
            if self.cfg.gated:
                self.w13.copy_(cpu_ref.interleave_gate_up(w1.to(self.w13.device), w3.to(self.w13.device)))
                self.w2.copy_(w2.to(self.w2.device).transpose(1, 2))
            else:
                self.w13.copy_(w1.to(self.w13.device).transpose(1, 2))

    def reference_weights(self) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[torch.Tensor]]:
        """Weights in the ``x @ W`` layouts: (W1 [e,D,F], W3 [e,D,F], W2 [e,F,D]) or (W [e,D,N], None, None)."""
        if not self.cfg.gated:
            return self.w13.transpose(1, 2).contiguous(), None, None
        EL, F2, D = self.w13.shape
        blk = self.w13.view(EL, F2 // 256, 2, 128, D)
        w1 = blk[:, :, 0].reshape(EL, F2 // 2, D).transpose(1, 2).contiguous()
        w3 = blk[:, :, 1].reshape(EL, F2 // 2, D).transpose(1, 2).contiguous()
        return w1, w3, self.w2.transpose(1, 2).contiguous()

    # ----------------------------------------------------------------- engine
    def _build_engine(self) -> None:
        cfg, heap = self.cfg, self.heap
        W, EL, ET, k, D = cfg.world_size, cfg.e_local, cfg.num_experts, cfg.topk, cfg.hidden_dim
        if heap.world != W:
            raise ValueError(f"heap spans {heap.world} ranks but the config says {W}")
        if ET > nv.MAX_EXPERTS or EL > nv.MAX_GROUPS:
            raise ValueError(f"at most {nv.MAX_EXPERTS} experts are supported")
        if D % 8 or (cfg.gated and cfg.ffn_dim % 128):
            raise ValueError("hidden_dim must be a multiple of 8 and ffn_dim of 128")
        T = self.max_tokens
        if T * k >= (1 << 24):
            raise ValueError("max_tokens * topk must stay below 2^24")
        dev = heap.device
        cap = self._cap_rows if self._cap_rows is not None else default_cap_rows(cfg, T)
        u32 = torch.int32
        # symmetric state (identical offsets on every rank).  Fixed-size part first, so that the
        # capacity-dependent buffers sit at the end of the heap and can be re-made larger.
        self._guard()
        self.counts_all = heap.zeros((2, W, ET), u32)
        self.counts_flag = heap.zeros((2, W), u32)
        self.iter_done = heap.zeros((W,), u32)
        self.arrived = heap.zeros((1,), u32)
        self._guard()
        self.out_slots = heap.empty((T * k, cfg.out_dim), cfg.dtype)
        self._guard()
        # local state
        i32 = dict(dtype=torch.int32, device=dev)
        self.group_rows = torch.zeros(EL, **i32)
        self.ticket = torch.zeros(1, **i32)
        # iteration number, kept on the device: kernels read it and the last kernel of a forward
        # pass increments it, so launch arguments never change (CUDA-graph replay works)
        self.iter_dev = torch.zeros(1, **i32)
        n = T * k
        self._plan = Plan(torch.empty(ET, **i32), torch.empty(ET + 1, **i32), torch.empty(n, **i32),
                          torch.empty(n, **i32), torch.empty(n, **i32))
        self._slot_reduce = declare(
            "b200_slot_reduce",
            [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint, C.c_int, C.c_int, C.c_int, C.c_void_p,
             C.POINTER(RetireArgs), C.c_void_p, C.c_ulonglong, C.c_void_p])
        self._route_plan_small = declare(
            "b200_route_plan_small",
            [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
             C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(PlanPushArgs), C.c_void_p,
             C.c_void_p])
        self._small_ticket = torch.zeros(1, dtype=torch.int32, device=dev)   # "last CTA plans" hand-over word
        self._ctas = int(self._num_ctas) if self._num_ctas else sm_count(dev)
        pair = cfg.cta_pair
        if os.getenv("B200MOE_CTA_PAIR", "") in ("0", "1"):       # override for tile-shape experiments
            pair = os.environ["B200MOE_CTA_PAIR"] == "1"
        if pair is None:
            # 256-row tiles pay off once experts average 128 rows: from there on many experts hold more than
            # one 128-row tile, and a second tile streams the expert's weights again (Mixtral shape, one GPU:
            # 700 -> 666 us at 128 rows per expert, 773 -> 670 us at 192; 555 -> 643 us at 64)
            pair = (T * k * W) // max(ET, 1) >= 128
        self._cta_pair = int(bool(pair))
        self._budget_ns = int(cfg.wait_budget_ms * 1e6)
        self.recv = self.meta = self.ready = self.hidden = None
        self._alloc_capacity(cap)
        # every rank's buffers exist and are zeroed before anyone dispatches
        torch.cuda.synchronize(dev)
        if W > 1:
            dist.barrier(group=heap.group)
        self._engine_ready = True

    def _guard(self) -> None:
        """Debug aid: a guard block of known words between two symmetric buffers."""
        if self._debug_canaries:
            g = self.heap.empty((256,), torch.int32)
            g.fill_(_CANARY)
            self._canaries.append(g)

    def check_canaries(self) -> None:
        """Raise if any guard block around the symmetric buffers was written to (needs
        ``debug_canaries=True``).  Synchronises."""
        for i, g in enumerate(self._canaries):
            bad = int((g != _CANARY).sum().item())
            if bad:
                raise nv.NativeError(f"rank {self.rank}: guard block {i} of the symmetric buffers was "
                                     f"overwritten ({bad} of {g.numel()} words)")

    def _alloc_capacity(self, cap: int) -> None:
        """(Re)make the buffers whose size follows the receive capacity."""
        cfg, heap = self.cfg, self.heap
        D, EL = cfg.hidden_dim, cfg.e_local
        guards = self._canaries[self._fixed_guards:] if self.recv is not None else []
        for t in [*reversed(guards), self.ready, self.meta, self.recv]:   # reverse order: the heap's tail shrinks
            if t is not None:
                heap.free(t)
        if self.recv is not None:
            del self._canaries[self._fixed_guards:]
        else:
            self._fixed_guards = len(self._canaries)
        self.cap_rows = int(cap)
        self.cap_mtiles = self.cap_rows // BM + EL + 1
        self.recv = heap.empty((2, self.cap_rows, D), cfg.dtype)
        self._guard()
        self.meta = heap.zeros((2, self.cap_rows, 2), torch.int32)
        self._guard()
        self.ready = heap.zeros((2, self.cap_mtiles), torch.int32)
        self._guard()
        self.hidden = (torch.empty((self.cap_rows, cfg.ffn_dim), dtype=cfg.dtype, device=heap.device)
                       if cfg.gated else None)
        self._trace = None
        self._graph = None

    def memory_bytes(self) -> dict:
        """Bytes this layer holds per rank: symmetric (peer-visible) and local buffers, weights apart."""
        sym = sum(t.numel() * t.element_size() for t in
                  (self.recv, self.meta, self.ready, self.counts_all, self.counts_flag, self.iter_done,
                   self.out_slots, self.arrived))
        local = (self.hidden.numel() * 2 if self.hidden is not None else 0)
        local += sum(t.numel() * 4 for t in (self._plan.send_order, self._plan.dst_slot, self._plan.rank_in_bucket))
        return dict(symmetric=int(sym), local=int(local), capacity_rows=self.cap_rows,
                    balanced_rows=self.max_tokens * self.cfg.topk)

    # ------------------------------------------------------------ capacity
    def reset_state(self) -> None:
        """Collective: bring the cross-rank counters back to their between-steps state after a
        step that failed on some rank (overflow, timeout).  Synchronises every rank."""
        W = self.cfg.world_size
        torch.cuda.synchronize(self.heap.device)
        if W > 1:
            dist.barrier(group=self.heap.group)          # nobody is still writing into a peer
        self.arrived.zero_()
        self.ready.zero_()
        self.ticket.zero_()
        self._small_ticket.zero_()
        self.heap.status.zero_()
        torch.cuda.synchronize(self.heap.device)
        if W > 1:
            dist.barrier(group=self.heap.group)

    def close(self) -> None:
        """Collective: give this layer's symmetric buffers back to the heap (every rank, between
        steps, in the same order for layers that share a heap).  The layer cannot run afterwards."""
        if getattr(self, "_closed", False) or self.heap is None or not getattr(self, "_engine_ready", False):
            return
        W = self.cfg.world_size
        torch.cuda.synchronize(self.heap.device)
        if W > 1:
            dist.barrier(group=self.heap.group)          # nobody is still writing into a peer
        if not self.heap.closed:
            for t in [*reversed(self._canaries), self.ready, self.meta, self.recv, self.out_slots,
                      self.arrived, self.iter_done, self.counts_flag, self.counts_all]:
                if t is not None:
                    self.heap.free(t)
        self._canaries = []
        self.recv = self.meta = self.ready = self.out_slots = self.hidden = None
        self.arrived = self.iter_done = self.counts_flag = self.counts_all = None
        self._graph = None
        self._closed = True

    def resize(self, cap_rows: int) -> None:
        """Collective: re-make the receive buffers for ``cap_rows`` rows per rank (rounded up to
        a tile).  Every rank must call it with the same value, between steps."""
        cap = (int(cap_rows) + BM - 1) // BM * BM
        self.reset_state()
        self._alloc_capacity(cap)
        torch.cuda.synchronize(self.heap.device)
        if self.cfg.world_size > 1:
            dist.barrier(group=self.heap.group)

    def forward_checked(self, x: torch.Tensor, max_retries: int = 3, growth: float = 1.1) -> torch.Tensor:
        """``forward`` followed by a status check on every rank (a host synchronisation).

        When some rank's routed rows exceeded the receive capacity, every rank re-makes its
        buffers for the largest number of rows any rank needed (times ``growth``) and the step
        is repeated -- what the reference's benchmark can only skip (benchmark.py:133-142).
        Other failures raise on every rank.  Use it for the first steps of a run (to settle
        the capacity) or throughout where a host synchronisation per step is acceptable."""
        W = self.cfg.world_size
        for attempt in range(max_retries + 1):
            y = self.forward(x)
            torch.cuda.synchronize(self.heap.device)
            st = self.heap.status[:2].clone()
            code, needed = int(st[0].item()), int(st[1].item())
            info = torch.tensor([1 if code == nv.ST_OVERFLOW else 0, needed,
                                 1 if code not in (0, nv.ST_OVERFLOW) else 0, code],
                                dtype=torch.int64, device=self.heap.device)
            if W > 1:
                dist.all_reduce(info, op=dist.ReduceOp.MAX, group=self.heap.group)
            overflow, needed_max, other, worst = (int(v) for v in info.tolist())
            if not overflow and not other:
                return y
            if not overflow or attempt == max_retries:
                self.reset_state()
                raise nv.NativeError(f"rank {self.rank}: step failed with device status {worst}: "
                                     f"{nv.status_message(worst)} (this rank: {code})")
            self.resize(max(int(needed_max * growth), self.cap_rows + BM))
        raise AssertionError("unreachable")

    SMALL_MAX_FLAT = 4096          # routed copies the single-launch route+plan kernel takes
    SMALL_MAX_TRIPS = 16           # dependent load round trips per warp up to which its CUDA-core router wins

    def uses_small_path(self, T: int) -> bool:
        """True when a forward of ``T`` tokens takes the small-token path: router and plan in ONE
        launch instead of three.  The kernel gives every token a warp (eight per CTA, at most 148
        CTAs) that walks the token's row once per group of eight experts, two 16-byte pieces per
        lane and trip; the Mixtral shape at 2048 tokens (16 trips) is where it stops being faster
        than the tensor-core router plus the two plan kernels."""
        cfg = self.cfg
        if not self.small_path or T * cfg.topk > self.SMALL_MAX_FLAT:
            return False
        trips = (-(-T // (148 * 8))) * (-(-cfg.num_experts // 8)) * (-(-cfg.hidden_dim // (8 * 64)))
        return trips <= self.SMALL_MAX_TRIPS

    def launches_for(self, T: int) -> int:
        """Kernel launches of one fused forward of ``T`` tokens: router + plan (3 launches, or 1 on
        the small-token path), fused GEMM kernel(s), slot reduce."""
        return (1 if self.uses_small_path(T) else 3) + (2 if self.cfg.gated else 1) + 1

    @property
    def launches_per_forward(self) -> int:
        return self.launches_for(self.max_tokens)

    @property
    def status(self) -> torch.Tensor:
        return self.heap.status

    def check_status(self) -> None:
        """Host-side check of the device status word (synchronises)."""
        self.heap.check_status()

    # ---------------------------------------------------------------- forward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            return self._forward_cpu(x)
        if _NVTX:
            torch.cuda.nvtx.range_push("MoELayer.forward")
            try:
                return self._forward_fused(x)
            finally:
                torch.cuda.nvtx.range_pop()
        return self._forward_fused(x)

    def route(self, x: torch.Tensor):
        return router_topk(x, self.router, self.cfg.topk, self.router_bias, self.cfg.renormalize,
                           status=self.heap.status if (x.is_cuda and self.heap is not None) else None)

    def _forward_fused(self, x: torch.Tensor) -> torch.Tensor:
        cfg, heap = self.cfg, self.heap
        W, EL, ET, k, D = cfg.world_size, cfg.e_local, cfg.num_experts, cfg.topk, cfg.hidden_dim
        T = x.shape[0]
        if getattr(self, "_closed", False):
            raise RuntimeError("this MoELayer was closed: its symmetric buffers went back to the heap")
        if T > self.max_tokens or x.shape[1] != D:
            raise ValueError(f"x must be [T <= {self.max_tokens}, {D}]")
        if x.dtype != cfg.dtype or not x.is_contiguous():
            x = x.to(cfg.dtype).contiguous()
        lib = nv.lib()
        iter_p = self.iter_dev.data_ptr()
        esz = 2   # bytes per bf16
        st = stream_ptr(x)
        status_p = heap.status.data_ptr()

        ev = self._mark if self.profile else (lambda name: None)
        if self.profile:
            self.phase_events = []
        ev("start")
        push = PlanPushArgs()
        push.world, push.rank = W, heap.rank
        push.iter_done = self.iter_done.data_ptr()
        push.peer_counts = heap.peer_ptrs(self.counts_all[0])
        push.peer_flags = heap.peer_ptrs(self.counts_flag[0])
        push.iter_ptr = iter_p
        push.stride_counts = W * ET * 4
        push.stride_flags = W * 4
        push.status = status_p
        push.wait_budget_ns = self._budget_ns
        plan = self._plan
        n = T * k
        view = Plan(plan.counts, plan.bucket_start, plan.send_order[:n], plan.dst_slot[:n],
                    plan.rank_in_bucket[:n])
        if self.uses_small_path(T):
            # 1+2. small batch: router and plan in one launch
            idx = torch.empty((T, k), dtype=torch.int32, device=x.device)
            wgt = torch.empty((T, k), dtype=torch.float32, device=x.device)
            bias = None if self.router_bias is None else self.router_bias.to(
                device=x.device, dtype=torch.float32).contiguous()
            nv.check(self._route_plan_small(ptr(x), ptr(router_kmajor(self.router)), ptr(bias), T, D, ET, k,
                                            int(cfg.renormalize), ptr(idx), ptr(wgt), ptr(view.counts),
                                            ptr(view.bucket_start), ptr(view.send_order), ptr(view.dst_slot),
                                            C.byref(push), ptr(self._small_ticket), st), "route+plan launch")
            ev("router")
            ev("plan")
        else:
            # 1. router
            idx, wgt = self.route(x)
            ev("router")
            # 2. plan (+ counts push)
            make_plan(idx, ET, out=view, push=push)
            ev("plan")

        # 3. dispatch + GEMM1 (one kernel)
        da = nv.DispatchArgs()
        da.world, da.rank, da.e_local, da.topk, da.num_tokens = W, heap.rank, EL, k, T
        da.x = x.data_ptr()
        da.send_order = plan.send_order.data_ptr()
        da.topk_weight = wgt.data_ptr()
        da.counts_all = self.counts_all[0].data_ptr()
        da.counts_flag = self.counts_flag[0].data_ptr()
        da.cap_rows = self.cap_rows
        da.cap_mtiles = self.cap_mtiles
        da.drop_signal = int(self.drop_signal)
        da.peer_recv = heap.peer_ptrs(self.recv[0])
        da.peer_meta = heap.peer_ptrs(self.meta[0])
        da.peer_ready = heap.peer_ptrs(self.ready[0])
        da.iter_ptr = iter_p
        da.stride_counts = W * ET * 4
        da.stride_flag = W * 4
        da.stride_recv = self.cap_rows * D * esz
        da.stride_meta = self.cap_rows * 8
        da.stride_ready = self.cap_mtiles * 4
        da.group_rows_out = self.group_rows.data_ptr()
        if self.trace_arrivals:
            if self._trace is None:
                self._trace = torch.zeros(2 + 2 * self.cap_mtiles, dtype=torch.int64, device=x.device)
            self._trace.zero_()
            da.trace = self._trace.data_ptr()
            da.trace_tiles = self.cap_mtiles

        ca = nv.CombineArgs()
        ca.world = W
        ca.row_meta = self.meta[0].data_ptr()
        ca.iter_ptr = iter_p
        ca.stride_meta = self.cap_rows * 8
        ca.out_row_stride = cfg.out_dim
        ca.max_slots = self.max_tokens * k
        ca.peer_out = heap.peer_ptrs(self.out_slots)
        ca.peer_arrived = heap.peer_ptrs(self.arrived)

        ga = nv.GemmArgs()
        ga.num_groups, ga.K, ga.group_m = EL, D, self.group_m[0]
        ga.status, ga.wait_budget_ns = status_p, self._budget_ns
        ga.cta_pair = self._cta_pair
        ga.l2_hints = self.l2_hints[0]
        ga.tma_store = 0 if self.tma_store else -1
        ga.wide_tiles = self.wide_tiles[0]
        recv = self.recv[0]
        if cfg.gated:
            F = cfg.ffn_dim
            ga.N, ga.n_out = 2 * F, F
            ga.out, ga.ldo = self.hidden.data_ptr(), F
            nv.check(lib.b200_grouped_gemm(ptr(recv), self.cap_rows, ptr(self.w13), nv.EPI_SILU_GATE, 1,
                                           C.byref(ga), C.byref(da), None, None, self._ctas, st),
                     "dispatch+GEMM1 launch")
            ev("dispatch+gemm1")
            # 4. GEMM2 + combine (one kernel)
            gb = nv.GemmArgs()
            gb.num_groups, gb.N, gb.K, gb.n_out, gb.group_m = EL, D, F, D, self.group_m[1]
            gb.group_rows = self.group_rows.data_ptr()
            gb.status, gb.wait_budget_ns = status_p, self._budget_ns
            gb.cta_pair = self._cta_pair
            gb.l2_hints = self.l2_hints[1]
            gb.wide_tiles = self.wide_tiles[1]
            nv.check(lib.b200_grouped_gemm(ptr(self.hidden), self.cap_rows, ptr(self.w2), nv.EPI_COMBINE,
                                           0, C.byref(gb), None, C.byref(ca), None, self._ctas, st),
                     "GEMM2+combine launch")
            ev("gemm2+combine")
        else:
            # single Linear: dispatch, GEMM and combine are ONE kernel
            ga.N = ga.n_out = cfg.out_dim
            nv.check(lib.b200_grouped_gemm(ptr(recv), self.cap_rows, ptr(self.w13), nv.EPI_COMBINE, 1,
                                           C.byref(ga), C.byref(da), C.byref(ca), None, self._ctas, st),
                     "dispatch+GEMM+combine launch")
            ev("dispatch+gemm+combine")

        # 5. slot reduce + retire
        y = torch.empty((T, cfg.out_dim), dtype=cfg.dtype, device=x.device)
        ra = RetireArgs()
        ra.world, ra.rank = W, heap.rank
        ra.peer_iter_done = heap.peer_ptrs(self.iter_done)
        ra.ready_counters = self.ready[0].data_ptr()
        ra.iter_ptr = iter_p
        ra.stride_ready = self.cap_mtiles * 4
        ra.num_ready = self.cap_mtiles
        ra.ticket = self.ticket.data_ptr()
        n_tiles = (cfg.out_dim + BN - 1) // BN
        nv.check(self._slot_reduce(ptr(self.out_slots), ptr(plan.dst_slot), ptr(self.arrived),
                                   T * k * n_tiles, T, k,
                                   cfg.out_dim, ptr(y), C.byref(ra), C.c_void_p(status_p),
                                   self._budget_ns, st), "slot reduce launch")
        ev("slot_reduce")
        self._iteration += 1
        self.last_routing = (idx, wgt)
        return y

    # ------------------------------------------------------------ CUDA graphs
    def capture(self, num_tokens: Optional[int] = None) -> None:
        """Capture one forward pass for ``num_tokens`` tokens into a CUDA graph.

        Every launch argument is fixed (the iteration number and the parity of the
        double-buffered peer state live in device memory), so the graph can be replayed for
        every later step with :meth:`replay`.  In a multi-rank job all ranks must capture and
        replay in step.  The layer is warmed up first: kernel attributes and driver entry
        points are resolved outside the capture."""
        T = self.max_tokens if num_tokens is None else int(num_tokens)
        dev = self.heap.device
        # the warm-up input is random, not zero: equal logits would send every token of every rank
        # to the first experts and overflow a capacity sized for balanced routing
        self._graph_x = torch.randn((T, self.cfg.hidden_dim), device=dev).to(self.cfg.dtype)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            self._forward_fused(self._graph_x)          # warm-up outside the capture
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.check_status()
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._graph_y = self._forward_fused(self._graph_x)

    def replay(self, x: torch.Tensor) -> torch.Tensor:
        """Run the captured forward pass on ``x`` (copied into the graph's static input);
        returns the graph's static output tensor, valid until the next replay."""
        if getattr(self, "_graph", None) is None:
            raise RuntimeError("call capture() first")
        if x.shape != self._graph_x.shape:
            raise ValueError(f"the graph was captured for input shape {tuple(self._graph_x.shape)}")
        self._graph_x.copy_(x, non_blocking=True)
        self._graph.replay()
        self._iteration += 1
        return self._graph_y

    def arrival_report(self) -> dict:
        """Overlap evidence from the last forward run with ``trace_arrivals = True``: when (relative
        to the fused kernel's start) the received M-tiles became usable, and how long the TMA
        producers stalled waiting for rows (summed over CTAs).  Synchronises."""
        if self._trace is None:
            raise RuntimeError("set layer.trace_arrivals = True before the forward pass")
        torch.cuda.synchronize()
        t = self._trace.cpu()
        start = int(t[0])
        seen_all = t[2:2 + self.cap_mtiles]
        seen = seen_all[seen_all > 0] - start
        if seen.numel() == 0:
            return dict(tiles=0)
        s = torch.sort(seen.double()).values / 1e3
        pick = lambda q: float(s[min(int(q * (s.numel() - 1)), s.numel() - 1)])
        sent_all = t[2 + self.cap_mtiles:]
        sent = torch.sort((sent_all[sent_all > 0] - start).double()).values / 1e3
        extra = {}
        if sent.numel():
            extra = dict(own_first_published_us=float(sent[0]), own_last_published_us=float(sent[-1]))
        return dict(tiles=int(s.numel()), **extra, first_us=float(s[0]), p50_us=pick(0.5), p90_us=pick(0.9),
                    last_us=float(s[-1]), producer_stall_us_sum=float(t[1]) / 1e3,
                    producer_stall_us_per_cta=float(t[1]) / 1e3 / max(self._ctas, 1))

    def _mark(self, name: str) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.phase_events.append((name, e))

    def phase_times_us(self) -> dict:
        """Device time of each phase of the last profiled forward (synchronises)."""
        torch.cuda.synchronize()
        out = {}
        for (_, a), (name, b) in zip(self.phase_events[:-1], self.phase_events[1:]):
            out[name] = a.elapsed_time(b) * 1000.0
        return out

    # -------------------------------------------------------------- CPU path
    def _forward_cpu(self, x: torch.Tensor) -> torch.Tensor:
        from ..parallel.gloo_moe import moe_forward_gloo
        return moe_forward_gloo(self, x)
