"""Building blocks of the two-arm benchmark (``bench.py``).

Both arms -- this library and the unmodified reference -- are driven by the SAME loops:

* :func:`device_timed` times K forward steps with CUDA events on the launching stream;
* :func:`e2e_loop` times the same step end to end: every step's tokens are copied from pinned
  host memory on a copy stream (the copy of step i+1 overlaps the compute of step i) and
  the step's result scalar is read back on the host one step late, so the GPU never idles
  waiting for the host.

An *arm* is an object with ``hosts`` (two pinned token buffers), ``inputs`` (their device
copies), ``run(x_dev, i)`` (one step on device tokens ``x_dev``; ``i & 1`` says which of the two
inputs it is) and ``result(out)`` (a one-element fp32 tensor that depends on the step's output).
Arms of this library: :class:`LayerArm` (``MoELayer.forward``) and :class:`A2AArm`
(``PaddedAllToAll``).  Arms of the reference: :class:`RefLayerArm` and :class:`RefA2AArm`, whose
timed communication is the reference's own ``run_baseline_ref`` (baseline.py:227-305), imported
from its installed copy; none of this library's kernels run in them.
"""
from __future__ import annotations

import datetime
import os
import statistics
import subprocess
import tempfile
import time
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .config import MoEConfig, preset
from .utils import gen

# Shapes of the benchmark configurations (tokens per rank = batch * seq).
MODEL_DEFAULTS = {
    "mixtral-8x7b": dict(batch=4, seq=4096),
    "fine-grained": dict(batch=8, seq=2048),
    "large": dict(batch=8, seq=4096),
    "mixtral-2e": dict(batch=1, seq=4096),
    "tiny": dict(batch=1, seq=64),
    "a2a": dict(batch=4, seq=1024),
}


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs (read-only)."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def mark_begin(self) -> None:
        self.t_begin = time.time()

    def mark_end(self) -> None:
        self.t_end = time.time()

    def start(self) -> None:
        self.t_begin, self.t_end = 0.0, float("inf")
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
            return
        # nvidia-smi needs a moment to enumerate the GPUs: wait for its first sample
        t0 = time.time()
        while time.time() - t0 < 10.0:
            try:
                if os.path.getsize(self.path) > 0:
                    break
            except OSError:
                pass
            time.sleep(0.05)

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power = [], [], []
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:   # keep only samples taken inside the timed region
                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    if ts < self.t_begin - 0.05 or ts > self.t_end + 0.05:
                        continue
                except ValueError:
                    pass
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2])); power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons),
                       samples=len(sm), power_w_max=max(power))
        return out


# --------------------------------------------------------------------------- NVLink counters
class NvlinkCounters:
    """Reads the GPU's NVLink data-byte counters through NVML (queries only, nothing is set or
    reset).  ``read()`` returns (tx_bytes, rx_bytes) summed over all links, or None where the
    driver does not expose the counters."""

    def __init__(self, gpu_index: int) -> None:
        self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            # NVML enumerates physical GPUs; honour CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if vis:
                ids = [v.strip() for v in vis.split(",") if v.strip()]
                if gpu_index < len(ids) and ids[gpu_index].isdigit():
                    phys = int(ids[gpu_index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
        except Exception:
            self.handle = None

    def read(self):
        if self.handle is None:
            return None
        nv = self.nv
        try:
            all_links = 0xFFFFFFFF
            vals = nv.nvmlDeviceGetFieldValues(self.handle, [
                (nv.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX, all_links),
                (nv.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX, all_links)])
            out = []
            for v in vals:
                if v.nvmlReturn != 0:
                    return None
                out.append(int(v.value.ullVal) * 1024)      # the counters are in KiB
            return tuple(out)
        except Exception:
            return None


# --------------------------------------------------------------------------- loops
def fence(world: int) -> None:
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, dev, world: int) -> float:
    if world == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def device_timed(arm, steps: int, world: int, sampler: Optional[ClockSampler] = None) -> float:
    """Microseconds per step of ``arm.run`` on its device-resident inputs (CUDA events on the
    launching stream, barrier + synchronize on both sides); this rank's value."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence(world)
    if sampler is not None:
        sampler.mark_begin()
    e0.record()
    for i in range(steps):
        arm.run(arm.inputs[i & 1], i)
    e1.record()
    fence(world)
    if sampler is not None:
        sampler.mark_end()
    return e0.elapsed_time(e1) * 1000.0 / steps


def e2e_loop(arm, steps: int, world: int, dev) -> float:
    """Microseconds per step, end to end: H2D of every step's tokens from pinned memory (on a
    copy stream, one step ahead), the step, and a D2H read of its result scalar (one step late)."""
    main = torch.cuda.current_stream(dev)
    copy_stream = torch.cuda.Stream(dev)
    bufs = [torch.empty_like(arm.inputs[0]) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    freed = [torch.cuda.Event() for _ in range(2)]
    result_host = torch.zeros(2, dtype=torch.float32).pin_memory()
    result_ready = [torch.cuda.Event() for _ in range(2)]

    def stage(i: int) -> None:
        b = i & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(freed[b])
            bufs[b].copy_(arm.hosts[b], non_blocking=True)
            ready[b].record(copy_stream)

    for b in range(2):
        freed[b].record(main)
    fence(world)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    stage(0)
    acc = 0.0
    for i in range(steps):
        b = i & 1
        if i + 1 < steps:
            stage(i + 1)                      # prefetch overlaps this step's compute
        main.wait_event(ready[b])
        out = arm.run(bufs[b], i)
        freed[b].record(main)
        result_host[b:b + 1].copy_(arm.result(out), non_blocking=True)
        result_ready[b].record(main)
        if i > 0:                             # D2H read of the previous step's result
            result_ready[1 - b].synchronize()
            acc += float(result_host[1 - b])
    result_ready[(steps - 1) & 1].synchronize()
    acc += float(result_host[(steps - 1) & 1])
    t1.record()
    fence(world)
    return t0.elapsed_time(t1) * 1000.0 / steps


# --------------------------------------------------------------------------- configuration
def make_config(args, world: int) -> MoEConfig:
    """The layer configuration an invocation names (``--model`` preset plus overrides)."""
    over = {}
    if args.experts:
        over["num_experts"] = args.experts
    if args.topk:
        over["topk"] = args.topk
    name = args.model if args.mode == "layer" else "mixtral-8x7b"
    cfg = preset(name, world_size=world, **over)
    return cfg


def describe_config(args, cfg: MoEConfig, world: int) -> dict:
    """The ``config`` entry of the JSON line: identical for both arms of one invocation."""
    T = args.batch * args.seq
    if args.mode == "a2a":
        e_local = (args.experts or 8 * world) // world
        return dict(model=f"padded all-to-all {'dispatch+combine' if args.combine else 'dispatch'} "
                          f"(D={args.hidden}, E={e_local * world}, top-{args.topk or 2})",
                    mode="a2a", combine=bool(args.combine), hidden=args.hidden, experts=e_local * world,
                    topk=args.topk or 2, global_batch=args.batch * world, seq_len=args.seq,
                    tokens_per_rank=T, parallelism=f"ep{world}",
                    l2="every exchange moves its own payload between GPUs; two alternating inputs")
    return dict(model=f"{args.model} MoE layer (D={cfg.hidden_dim}, F={cfg.ffn_dim}, E={cfg.num_experts}, "
                      f"top-{cfg.topk}, SiLU-gated)",
                mode="layer", hidden=cfg.hidden_dim, ffn=cfg.ffn_dim, experts=cfg.num_experts, topk=cfg.topk,
                zipf_s=args.zipf, global_batch=args.batch * world, seq_len=args.seq, tokens_per_rank=T,
                parallelism=f"ep{world}",
                l2="inputs alternate between two token buffers and the expert weights are streamed "
                   "every step: the working set exceeds the 126 MB L2")


def router_bias_for(args, cfg: MoEConfig, dev):
    if not args.zipf or args.zipf <= 0:
        return None
    return gen.zipf_expert_bias(cfg.num_experts, args.zipf, scale=args.zipf_scale, seed=args.seed, device=dev)


def layer_tokens(args, cfg: MoEConfig, rank: int, dev):
    return [gen.gen_local_tokens(args.batch, args.seq, cfg.hidden_dim, torch.bfloat16, dev,
                                 args.seed + 1000 * i, rank, "normal") for i in range(2)]


# --------------------------------------------------------------------------- this library's arms
class LayerArm:
    """``MoELayer.forward``: router + plan + fused dispatch/GEMM1 + fused GEMM2/combine + slot reduce."""

    api = "iris_testing_b200.models.MoELayer.forward"
    timed = "router + plan + dispatch + expert MLP + combine (MoELayer.forward)"

    def __init__(self, args, rank: int, world: int, dev) -> None:
        from .models.moe_layer import MoELayer, heap_bytes_needed
        from .parallel.symm import SymmetricHeap
        self.args, self.rank, self.world, self.dev = args, rank, world, dev
        cfg = make_config(args, world)
        self.cfg = cfg
        T = args.batch * args.seq
        self.T = T
        need = heap_bytes_needed(cfg, T) + (64 << 20)
        worst = heap_bytes_needed(cfg, T, cap_rows=world * T * cfg.topk) + (64 << 20)
        self.heap = SymmetricHeap(need, max_bytes=max(worst, need))     # room to grow after an overflow
        self.layer = MoELayer(cfg, max_tokens=T, heap=self.heap, seed=args.seed, router_std=None)
        self.layer.router_bias = router_bias_for(args, cfg, dev)
        self.inputs = layer_tokens(args, cfg, rank, dev)
        self.hosts = [x.cpu().pin_memory() for x in self.inputs]
        self.h2d_bytes = T * cfg.hidden_dim * 2

    def settle(self) -> None:
        """First steps with a status check on every rank: grows the receive buffers if the
        routing of these inputs needs more than the default capacity."""
        for x in self.inputs:
            self.layer.forward_checked(x)

    def run(self, x: torch.Tensor, i: int) -> torch.Tensor:
        return self.layer(x)

    def result(self, out: torch.Tensor) -> torch.Tensor:
        return torch.linalg.vector_norm(out).reshape(1)

    def check_status(self) -> None:
        self.layer.check_status()

    def memory(self) -> dict:
        return self.layer.memory_bytes()

    def launches_expected(self, steps: int) -> int:
        return self.layer.launches_per_forward * steps

    def remote_bytes(self) -> Optional[dict]:
        """Algorithmic bytes per step that must cross NVLink on this rank: rows routed to other
        ranks (dispatch, out) and, for the combine, their results coming back (in)."""
        cfg = self.cfg
        idx, _ = self.layer.last_routing
        dst = (idx.reshape(-1) // cfg.e_local)
        remote_rows = int((dst != self.rank).sum().item())
        return dict(dispatch_tx=remote_rows * cfg.hidden_dim * 2, combine_rx=remote_rows * cfg.out_dim * 2)

    def close(self) -> None:
        self.layer = None
        self.heap.close()

    def check(self, tokens: int = 2048) -> dict:
        """One step of at most ``tokens`` tokens per rank against the dense single-process oracle
        over the all-gathered expert weights (the correctness report of the reference's
        benchmark, benchmark.py:354-440, for the whole layer)."""
        from .ops import cpu_ref
        cfg, layer = self.cfg, self.layer
        n = min(tokens, self.T)
        x = self.inputs[0][:n].contiguous()
        y = layer(x)
        torch.cuda.synchronize()
        layer.check_status()
        idx, _ = layer.last_routing
        ws = []
        for w in layer.reference_weights():
            if self.world > 1:
                parts = [torch.empty_like(w) for _ in range(self.world)]
                dist.all_gather(parts, w.contiguous())
                w = torch.cat(parts)
            ws.append(w)
        rep = cpu_ref.compare_with_dense(y, x, layer.router, cfg.topk, idx, bias=layer.router_bias,
                                         renormalize=cfg.renormalize, w1=ws[0], w3=ws[1], w2=ws[2],
                                         round_hidden=torch.bfloat16)
        flags = torch.tensor([0 if rep["ok"] else 1, rep["ambiguous_tokens"]], dtype=torch.float64, device=self.dev)
        errs = torch.tensor([rep["max_rel_err"], rep["max_rel_err_all_tokens"]], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            dist.all_reduce(flags, op=dist.ReduceOp.SUM)
            dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        return dict(max_rel_err=round(float(errs[0]), 6), max_rel_err_all_tokens=round(float(errs[1]), 6),
                    ambiguous_tokens=int(flags[1]), tokens_per_rank=n, tol=rep["tol"], ok=bool(flags[0] == 0),
                    oracle="dense fp32 MoE over all-gathered weights, tokens with a top-k gap below 1e-6 set aside")


class A2AArm:
    """Padded dispatch (+ return and weighted sum) through ``PaddedAllToAll``; routing is precomputed
    per input, as in the reference's benchmark (benchmark.py:119-123)."""

    api = "iris_testing_b200.parallel.PaddedAllToAll (dispatch, wait[, send_back, reduce])"

    def __init__(self, args, rank: int, world: int, dev) -> None:
        from .ops.plan import pack_rows
        from .parallel.padded_a2a import CapacityProbe, PaddedAllToAll
        from .parallel.symm import SymmetricHeap
        from .utils.pack import route_and_pack
        self.args, self.rank, self.world, self.dev = args, rank, world, dev
        self.pack_rows = pack_rows
        H, k = args.hidden, args.topk or 2
        self.e_local = (args.experts or 8 * world) // world
        E = self.e_local * world
        self.k, self.H = k, H
        dt = torch.bfloat16
        router = gen.gen_router(H, E, dt, dev, args.seed, std=None)
        self.inputs = [gen.gen_local_tokens(args.batch, args.seq, H, dt, dev, args.seed + 1000 * i, rank, "normal")
                       for i in range(2)]
        self.hosts = [x.cpu().pin_memory() for x in self.inputs]
        self.h2d_bytes = args.batch * args.seq * H * 2
        self.routed = []
        small = SymmetricHeap(8 << 20)
        probe = CapacityProbe(small, self.e_local)
        caps = []
        for x in self.inputs:
            payload, counts, dst_off, _, idx, wgt, plan = route_and_pack(x, router, k, world, E)
            self.routed.append(dict(payload=payload, counts=counts.contiguous(), dst_off=dst_off, idx=idx,
                                    wgt=wgt, plan=plan))
            caps.append(probe.measure(counts.contiguous()))
        caps = torch.stack(caps).max(dim=0).values.tolist()       # one read: CAP, M, rows received
        self.cap, self.pair_rows = max(int(caps[0]), 1), int(caps[1])
        small.close()
        cells = self.e_local * world * self.cap * H * 2
        self.heap = SymmetricHeap(cells * (2 if args.combine else 1) + (64 << 20))
        self.a2a = PaddedAllToAll(self.heap, self.e_local, self.cap, H, dt, with_return=bool(args.combine))
        self.timed = ("padded dispatch kernel + device-side arrival wait"
                      + (" + padded return + weighted sum" if args.combine else ""))

    def settle(self) -> None:
        pass

    def run(self, x: torch.Tensor, i: int) -> torch.Tensor:
        r = self.routed[i & 1]
        payload = r["payload"] if x is self.inputs[i & 1] else self.pack_rows(x, r["plan"].send_order, self.k)
        self.a2a.dispatch(payload, r["counts"], r["dst_off"])
        self.a2a.wait()
        if self.args.combine:
            self.a2a.send_back()
            return self.a2a.reduce(r["plan"], r["idx"], r["wgt"])
        return self.a2a.token_sync

    def result(self, out: torch.Tensor) -> torch.Tensor:
        if self.args.combine:
            return torch.linalg.vector_norm(out).reshape(1)
        return out.sum().float().reshape(1)

    def check_status(self) -> None:
        self.heap.check_status()

    def memory(self) -> dict:
        return dict(symmetric=self.heap.bytes_in_use, capacity_rows_per_cell=self.cap,
                    pair_rows_max_M=self.pair_rows)

    def launches_expected(self, steps: int) -> int:
        return (4 if self.args.combine else 2) * steps

    def remote_bytes(self) -> Optional[dict]:
        c = self.routed[0]["counts"]
        remote_rows = int(c.sum().item()) - int(c[self.rank].sum().item())
        out = dict(dispatch_tx=remote_rows * self.H * 2)
        if self.args.combine:
            out["combine_rx"] = remote_rows * self.H * 2
        return out

    def close(self) -> None:
        self.a2a = None
        self.heap.close()

    def check(self, tokens: int = 0) -> dict:
        """The reference's correctness report (benchmark.py:354-440): pca exact, valid region of
        token_buf bit-equal to the library all-to-all re-laid out, and with ``--combine`` the
        weighted sum against a plain-PyTorch evaluation."""
        from .parallel.baseline_nccl import ExchangeBuffers, relayout_to_token_buf, run_baseline
        from .utils.compare import masked_stats
        r = self.routed[0]
        self.a2a.dispatch(r["payload"], r["counts"], r["dst_off"])
        self.a2a.wait()
        torch.cuda.synchronize()
        _, _, meta = run_baseline(r["payload"], r["counts"], self.cap, ExchangeBuffers(torch.empty_like(r["counts"])))
        expected_pca = meta["recv_counts"].t().contiguous()
        tb = relayout_to_token_buf(meta["recv_payload"], meta["recv_counts"], self.cap)
        pca_diff = float((self.a2a.pca - expected_pca).abs().max())
        mx, s1, s2 = masked_stats(self.a2a.token_buf, tb, expected_pca)
        bad = [pca_diff, float(mx)]
        if self.args.combine:
            self.a2a.send_back()
            y = self.a2a.reduce(r["plan"], r["idx"], r["wgt"])
            x = self.inputs[0]
            ref = x.float() * r["wgt"].sum(dim=1, keepdim=True)      # every copy comes home unchanged
            bad.append(float((y.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-20)))
        torch.cuda.synchronize()
        self.heap.check_status()
        t = torch.tensor(bad, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        vals = t.tolist()
        ok = vals[0] == 0 and vals[1] == 0 and (len(vals) < 3 or vals[2] <= 1e-2)
        return dict(pca_max_diff=vals[0], token_buf_max_diff_valid=vals[1],
                    max_rel_err=(round(vals[2], 6) if len(vals) > 2 else 0.0), ok=bool(ok),
                    oracle="library all_to_all_single re-laid out to [e, src, m, :] (exact)")


# --------------------------------------------------------------------------- the reference's arms
def reference_pack(ref_utils, x, router, k, world, E, bias, how: str):
    """(payload, send_counts int32 [world, e_local], flat order, top-k values, top-k idx).

    ``how="reference"`` calls the reference's own ``route_and_pack_padding_free`` (a Python loop
    with one device read per routed copy: seconds for large inputs; it cannot take a router
    bias); ``how="vectorized"`` builds the same payload with tensor ops."""
    logits = torch.einsum("th,he->te", x, router)          # the reference's own expression (utils.py:201)
    if bias is not None:
        logits = logits.float() + bias.float()
    probs = F.softmax(logits, dim=-1)
    vals, idx = torch.topk(probs, k, dim=-1)
    order = torch.sort(idx.reshape(-1), stable=True).indices              # payload row -> flat (token, slot)
    if how == "reference" and bias is None:
        payload, send_counts, _, _ = ref_utils.route_and_pack_padding_free(x, router, k, world, E)
    else:
        payload = x.index_select(0, order // k)
        send_counts = torch.bincount(idx.reshape(-1), minlength=E)[:E].view(world, E // world)
    return payload, send_counts.to(torch.int32).contiguous(), order, vals, idx


class _RefBase:
    def __init__(self, ref_baseline, ref_utils, args, rank, world, dev):
        self.rb, self.ru = ref_baseline, ref_utils
        self.args, self.rank, self.world, self.dev = args, rank, world, dev

    def settle(self) -> None:
        pass

    def check_status(self) -> None:
        pass

    def check(self, tokens: int = 0):
        return None

    def launches_expected(self, steps: int) -> int:
        return 0

    def remote_bytes(self):
        return None

    def close(self) -> None:
        self.prepared = None

    def _prepare(self, x, router, k, E, bias, H):
        """Routing, packing and receive-side bookkeeping of one input (untimed, as in the
        reference's benchmark.py:119-161)."""
        world, rank, dev = self.world, self.rank, self.dev
        EL = E // world
        how = self.packer
        payload, send_counts, order, vals, _ = reference_pack(self.ru, x, router, k, world, E, bias, how)
        gathered = [torch.zeros_like(send_counts) for _ in range(world)]
        dist.all_gather(gathered, send_counts)
        counts_all = torch.stack(gathered)                             # [src, dst, e]
        recv_counts = counts_all[:, rank, :].contiguous()              # [src, e]
        cap = max(int(counts_all.max().item()), 1)
        total_recv = int(recv_counts.sum().item())
        bufs = self.rb.init_baseline_buffers(world, EL, cap, H, x.dtype, dev, total_recv,
                                             allocate_token_buf=False)
        return dict(x=x, payload=payload, send_counts=send_counts, token_of_row=(order // k),
                    w_of_row=vals.reshape(-1)[order].to(x.dtype).unsqueeze(1), cap=cap, bufs=bufs,
                    recv_counts=recv_counts, in_splits=send_counts.sum(dim=1).tolist(),
                    out_splits=recv_counts.sum(dim=1).tolist())

    def _exchange(self, inp, payload, e_local, H):
        self.rb.run_baseline_ref(rank=self.rank, world_size=self.world, e_local=e_local, capacity=inp["cap"],
                                 hidden_dim=H, send_payload=payload, send_counts=inp["send_counts"],
                                 buffers=inp["bufs"], do_reorder=False, profile=False, strict_capacity=False,
                                 barrier=False)
        return inp["bufs"].recv_payload_flat


class RefLayerArm(_RefBase):
    """One MoE layer step on the UNMODIFIED reference modules: the reference's
    ``run_baseline_ref`` (counts + payload ``all_to_all_single``), then what the reference lacks in
    plain PyTorch: expert MLP (``torch.matmul``), return ``all_to_all_single``, weighted
    ``index_add_``.  Routing/packing runs once per input before timing, as in its benchmark."""

    api = "reference baseline.run_baseline_ref + torch expert MLP + all_to_all_single return"
    timed = ("reference run_baseline_ref (counts + payload all_to_all_single) + torch expert MLP + NCCL "
             "return all-to-all + weighted index_add; the reference's router/packer runs before the "
             "timed region, as in its benchmark.py")

    def __init__(self, ref_baseline, ref_utils, args, rank, world, dev) -> None:
        super().__init__(ref_baseline, ref_utils, args, rank, world, dev)
        cfg = make_config(args, world)
        self.cfg = cfg
        D, EL, k = cfg.hidden_dim, cfg.e_local, cfg.topk
        self.T = args.batch * args.seq
        dt = torch.bfloat16
        self.packer = args.ref_packer if args.ref_packer != "auto" else (
            "reference" if (self.T * k <= 65536 and not args.zipf) else "vectorized")
        self.router = gen.gen_router(D, cfg.num_experts, dt, dev, args.seed, std=None)
        self.w1, self.w3, self.w2 = gen.gen_gated_expert_weights(EL, D, cfg.ffn_dim, dt, dev, args.seed, rank)
        bias = router_bias_for(args, cfg, dev)
        self.inputs = layer_tokens(args, cfg, rank, dev)
        self.hosts = [x.cpu().pin_memory() for x in self.inputs]
        self.h2d_bytes = self.T * D * 2
        self.prepared = []
        for x in self.inputs:
            inp = self._prepare(x, self.router, k, cfg.num_experts, bias, D)
            # rows arrive (src, expert)-major; the experts want them expert-major
            cell_e = torch.arange(EL, device=dev).repeat(world)
            row_e = torch.repeat_interleave(cell_e, inp["recv_counts"].reshape(-1).long())
            inp["perm"] = torch.sort(row_e, stable=True).indices if EL > 1 else None
            inp["rows_per_expert"] = inp["recv_counts"].sum(dim=0).tolist()
            self.prepared.append(inp)

    def memory(self) -> dict:
        return dict(recv_rows=[int(sum(p["rows_per_expert"])) for p in self.prepared])

    @torch.no_grad()
    def run(self, x: torch.Tensor, i: int) -> torch.Tensor:
        inp, cfg = self.prepared[i & 1], self.cfg
        # device-resident input: the payload packed before timing; staged input: pack it now
        payload = inp["payload"] if x is self.inputs[i & 1] else x.index_select(0, inp["token_of_row"])
        recv = self._exchange(inp, payload, cfg.e_local, cfg.hidden_dim)
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
        back = torch.empty_like(payload)
        dist.all_to_all_single(back, out, output_split_sizes=inp["in_splits"],
                               input_split_sizes=inp["out_splits"])
        y = torch.zeros((self.T, cfg.hidden_dim), dtype=back.dtype, device=self.dev)
        y.index_add_(0, inp["token_of_row"], back * inp["w_of_row"])
        return y

    def result(self, out: torch.Tensor) -> torch.Tensor:
        return torch.linalg.vector_norm(out).reshape(1)


class RefA2AArm(_RefBase):
    """The reference's library path for the exchange alone: ``run_baseline_ref`` (counts + ragged
    payload ``all_to_all_single``); with ``--combine`` the return ``all_to_all_single`` and the
    weighted ``index_add_`` in plain PyTorch."""

    api = "reference baseline.run_baseline_ref (+ all_to_all_single return + weighted index_add)"

    def __init__(self, ref_baseline, ref_utils, args, rank, world, dev) -> None:
        super().__init__(ref_baseline, ref_utils, args, rank, world, dev)
        H, k = args.hidden, args.topk or 2
        self.H, self.k = H, k
        self.e_local = (args.experts or 8 * world) // world
        E = self.e_local * world
        dt = torch.bfloat16
        self.T = args.batch * args.seq
        self.packer = args.ref_packer if args.ref_packer != "auto" else (
            "reference" if self.T * k <= 65536 else "vectorized")
        router = gen.gen_router(H, E, dt, dev, args.seed, std=None)
        self.inputs = [gen.gen_local_tokens(args.batch, args.seq, H, dt, dev, args.seed + 1000 * i, rank, "normal")
                       for i in range(2)]
        self.hosts = [x.cpu().pin_memory() for x in self.inputs]
        self.h2d_bytes = self.T * H * 2
        self.prepared = [self._prepare(x, router, k, E, None, H) for x in self.inputs]
        self.timed = ("reference run_baseline_ref (counts + payload all_to_all_single)"
                      + (" + NCCL return all-to-all + weighted index_add" if args.combine else ""))

    def memory(self) -> dict:
        return dict(capacity_rows_per_cell=max(p["cap"] for p in self.prepared))

    @torch.no_grad()
    def run(self, x: torch.Tensor, i: int) -> torch.Tensor:
        inp = self.prepared[i & 1]
        payload = inp["payload"] if x is self.inputs[i & 1] else x.index_select(0, inp["token_of_row"])
        recv = self._exchange(inp, payload, self.e_local, self.H)
        if not self.args.combine:
            return inp["bufs"].recv_counts
        back = torch.empty_like(payload)
        dist.all_to_all_single(back, recv, output_split_sizes=inp["in_splits"],
                               input_split_sizes=inp["out_splits"])
        y = torch.zeros((self.T, self.H), dtype=back.dtype, device=self.dev)
        y.index_add_(0, inp["token_of_row"], back * inp["w_of_row"])
        return y

    def result(self, out: torch.Tensor) -> torch.Tensor:
        if self.args.combine:
            return torch.linalg.vector_norm(out).reshape(1)
        return out.sum().float().reshape(1)
