#!/usr/bin/env python
"""Benchmark + correctness driver, configured by environment variables.

Counterpart of the reference's ``benchmark.py`` (benchmark.py:96-463): the same
variables (``WORLD_SIZE BATCH SEQ HIDDEN TOPK E_LOCAL CAPACITY SEED WARMUP ITERS CHECK
CLEAR_TOKEN_BUF SKIP_ON_OVERFLOW``; ``SYMM_HEAP_GIB`` with ``IRIS_HEAP_GIB`` accepted),
the same phases (route+pack, overflow check, warm-up, timed custom path, timed library
baseline, max-over-ranks report, correctness report), but timed with CUDA events on
the device instead of a host clock around prints and a host barrier.

``MODE`` selects what is measured:

* ``a2a``   (default) padded dispatch (``PaddedAllToAll``: the ``custom_a2a`` buffer contract
            driven by epochs, so no memset or barrier sits between calls) + device-side
            arrival wait  vs the ``all_to_all_single`` baseline; with ``COMBINE=1`` the padded
            return and the weighted sum are included on both sides.  ``CAPACITY=0`` sizes the
            cells from the device-side capacity rule.
* ``layer`` the fused MoE layer (router + dispatch + experts + combine) vs the same layer
            on library collectives (``AllToAllMoEBaseline``); needs ``FFN`` (0 = single Linear).
            ``TRACE=1`` adds one JSON line per rank: device time of each phase and when
            (relative to the fused kernel's start) the received tiles became usable.

Launch: ``python benchmark.py`` spawns ``WORLD_SIZE`` processes (one per GPU); under
``torch.distributed.run`` it uses the ranks it is given.  One JSON line per run is printed
by rank 0 and appended to ``$BENCH_OUT`` when set.
"""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent))

from iris_testing_b200.utils import (allreduce_max, allreduce_sum, gen_local_tokens, gen_router,  # noqa: E402
                                     mark, masked_stats, route_and_pack, sync_and_check, zipf_expert_bias)


def env_int(name: str, default: int) -> int:
    return int(os.getenv(name, str(default)))


def event_timer():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def max_rank_mean(times_ms, dev) -> float:
    t = torch.tensor([sum(times_ms) / max(len(times_ms), 1)], device=dev, dtype=torch.float32)
    return float(allreduce_max(t).item())


def report(rank: int, payload: dict) -> None:
    if rank != 0:
        return
    line = json.dumps(payload)
    print(line, flush=True)
    out = os.getenv("BENCH_OUT")
    if out:
        with open(out, "a") as f:
            f.write(line + "\n")


# --------------------------------------------------------------------------- a2a mode
def run_a2a(rank: int, world: int, dev: torch.device) -> None:
    from iris_testing_b200.parallel import run_baseline
    from iris_testing_b200.parallel.baseline_nccl import ExchangeBuffers
    from iris_testing_b200.parallel.padded_a2a import CapacityProbe, PaddedAllToAll
    from iris_testing_b200.parallel.symm import SymmetricHeap

    batch, seq, H = env_int("BATCH", 4), env_int("SEQ", 2048), env_int("HIDDEN", 4096)
    topk, e_local, cap = env_int("TOPK", 2), env_int("E_LOCAL", 4), env_int("CAPACITY", 1024)
    seed, warmup, iters = env_int("SEED", 42), env_int("WARMUP", 5), env_int("ITERS", 20)
    check, clear = env_int("CHECK", 1), env_int("CLEAR_TOKEN_BUF", 0)
    combine = env_int("COMBINE", 0)
    auto_cap = cap <= 0
    E = world * e_local
    dt = torch.bfloat16
    dist_name = os.getenv("TOKEN_DIST", "uniform")
    x = gen_local_tokens(batch, seq, H, dt, dev, seed, rank, dist_name)
    router = gen_router(H, E, dt, dev, seed, std=None if os.getenv("ROUTER_STD", "") == "" else float(os.environ["ROUTER_STD"]))
    payload, counts, dst_off, _, idx, wgt, plan = route_and_pack(x, router, topk, world, E)
    # CAP (largest cell over all ranks) and M (largest per-pair message) on the device, one read
    ctl = SymmetricHeap(8 << 20)
    cap_cell, pair_max, recv_max, _ = CapacityProbe(ctl, e_local).measure(counts.contiguous()).tolist()
    ctl.close()
    global_max = int(cap_cell)
    if auto_cap:
        cap = max(global_max, 1)
    if global_max > cap and env_int("SKIP_ON_OVERFLOW", 1):
        if rank == 0:
            print(f"[SKIP] max_recv_count={global_max} > CAPACITY={cap}. Increase CAPACITY or reduce "
                  f"(BATCH, SEQ, TOPK), or set SKIP_ON_OVERFLOW=0.", flush=True)
        return
    need = e_local * world * cap * H * 2 * (2 if combine else 1) + (256 << 20)
    heap_gib = env_int("SYMM_HEAP_GIB", env_int("IRIS_HEAP_GIB", 0))
    heap = SymmetricHeap(max(need, heap_gib << 30))
    a2a = PaddedAllToAll(heap, e_local, cap, H, dt, with_return=bool(combine))
    base = ExchangeBuffers(recv_counts=torch.empty_like(counts))

    def custom_once():
        if clear:
            a2a.token_buf.zero_()                      # debug aid of the reference (CLEAR_TOKEN_BUF)
        a2a.dispatch(payload, counts, dst_off)         # flags are re-armed inside the kernel
        a2a.wait()                                     # device-side: everything for this rank has landed
        if combine:
            a2a.send_back()
            return a2a.reduce(plan, idx, wgt)
        return a2a.token_buf

    def baseline_once():
        _, _, meta = run_baseline(payload, counts, cap, base, do_reorder=False)
        if combine:
            back = torch.empty_like(payload)
            if world > 1:
                dist.all_to_all_single(back, meta["recv_payload"], output_split_sizes=meta["in_splits"],
                                       input_split_sizes=meta["out_splits"])
            else:
                back.copy_(meta["recv_payload"])
            per = back[plan.dst_slot.long()].float() * wgt.reshape(-1, 1)
            return per.view(x.shape[0], topk, -1).sum(1).to(dt)
        return meta["recv_payload"]

    trace = env_int("TRACE", 0)
    ok = True
    err = None
    try:
        if trace:
            mark("warm-up: custom path")
        for _ in range(warmup):
            custom_once()
        torch.cuda.synchronize()
        heap.check_status()
        for _ in range(warmup):
            baseline_once()
        torch.cuda.synchronize()
    except Exception as exc:      # every rank must learn of a failure before the next collective
        ok, err = False, repr(exc)
    if not sync_and_check(ok, dev):
        if rank == 0 or err:
            print(f"[warm-up failed] rank{rank}: {err}", flush=True)
        return

    custom_ms, base_ms = [], []
    for _ in range(iters):
        torch.cuda.synchronize()
        s, e = event_timer()
        s.record()
        custom_once()
        e.record()
        torch.cuda.synchronize()
        custom_ms.append(s.elapsed_time(e))
    dist.barrier() if world > 1 else None
    for _ in range(iters):
        torch.cuda.synchronize()
        s, e = event_timer()
        s.record()
        baseline_once()
        e.record()
        torch.cuda.synchronize()
        base_ms.append(s.elapsed_time(e))
    heap.check_status()
    c_ms, b_ms = max_rank_mean(custom_ms, dev), max_rank_mean(base_ms, dev)
    rows_out = int(counts.sum().item())
    remote = rows_out * H * 2 * (world - 1) / max(world, 1) * (2 if combine else 1)
    report(rank, dict(mode="a2a+combine" if combine else "a2a", world=world, e_local=e_local, cap=cap,
                      hidden=H, batch=batch, seq=seq, topk=topk, pair_rows_max_M=int(pair_max),
                      cell_rows_max=global_max, recv_rows_max=int(recv_max), custom_us=round(c_ms * 1e3, 1),
                      baseline_us=round(b_ms * 1e3, 1), speedup=round(b_ms / c_ms, 3),
                      payload_mb=round(rows_out * H * 2 / 1e6, 2),
                      nvlink_floor_us=round(remote / 770e9 * 1e6 / (2 if combine else 1), 1),
                      timing="CUDA events, mean over iters, max over ranks"))
    if rank == 0:
        print("=== COMM-only perf (device-timed, max over ranks) ===")
        print(f"world={world} E_local={e_local} CAP={cap} H={H} batch={batch} seq={seq} topk={topk}")
        print(f"custom_ms:   {c_ms:.3f}\nbaseline_ms: {b_ms:.3f}\nspeedup:     {b_ms / c_ms:.3f}x", flush=True)

    if check:
        a2a.token_buf.zero_()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a2a.dispatch(payload, counts, dst_off)
        a2a.wait()
        torch.cuda.synchronize()
        tb, _, meta = run_baseline(payload, counts, cap, ExchangeBuffers(torch.empty_like(counts)),
                                   do_reorder=True)
        expected_pca = meta["recv_counts"].t().contiguous()
        pca_diff = (a2a.pca - expected_pca).abs().max().float().reshape(1)
        mx, s1, s2 = masked_stats(a2a.token_buf, tb, expected_pca)
        pca_g, mx_g = allreduce_max(pca_diff), allreduce_max(mx.reshape(1))
        s1_g, s2_g = allreduce_sum(s1.reshape(1)), allreduce_sum(s2.reshape(1))
        if rank == 0:
            passed = pca_g.item() == 0 and mx_g.item() == 0 and abs(s1_g.item() - s2_g.item()) < 1e-3 * max(1.0, abs(s2_g.item()))
            print("=== Correctness report ===")
            print(f"PCA max|diff| (global): {pca_g.item():.6g}")
            print(f"TOKEN_BUF max|diff| valid (global): {mx_g.item():.6g}")
            print(f"TOKEN_BUF sum(valid) custom / baseline: {s1_g.item():.6g} / {s2_g.item():.6g}")
            print("PASS" if passed else "FAIL", flush=True)


# --------------------------------------------------------------------------- layer mode
def run_layer(rank: int, world: int, dev: torch.device) -> None:
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer, heap_bytes_needed
    from iris_testing_b200.parallel import AllToAllMoEBaseline
    from iris_testing_b200.parallel.symm import SymmetricHeap

    batch, seq, D, F = env_int("BATCH", 4), env_int("SEQ", 4096), env_int("HIDDEN", 4096), env_int("FFN", 14336)
    topk, e_local = env_int("TOPK", 2), env_int("E_LOCAL", 1)
    if os.getenv("EXPERTS"):
        e_local = env_int("EXPERTS", 8) // world
    seed, warmup, iters = env_int("SEED", 0), env_int("WARMUP", 3), env_int("ITERS", 10)
    cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=e_local * world, topk=topk, world_size=world,
                    gated=F > 0)
    T = batch * seq
    need = heap_bytes_needed(cfg, T) + (64 << 20)
    worst = heap_bytes_needed(cfg, T, cap_rows=world * T * topk) + (64 << 20)
    heap = SymmetricHeap(need, max_bytes=max(need, worst))          # room to grow after an overflow
    layer = MoELayer(cfg, max_tokens=T, heap=heap, seed=seed, router_std=None)
    zipf = float(os.getenv("ZIPF_S", "0"))
    if zipf > 0:
        layer.router_bias = zipf_expert_bias(cfg.num_experts, zipf, scale=float(os.getenv("ZIPF_SCALE", "1")),
                                             seed=seed, device=dev)
    x = gen_local_tokens(batch, seq, D, torch.bfloat16, dev, seed, rank, "normal")
    base = AllToAllMoEBaseline(layer)
    ok, err = True, None
    try:
        y = layer.forward_checked(x)          # grows the receive buffers if this routing needs it
        for _ in range(warmup):
            y = layer(x)
        torch.cuda.synchronize()
        layer.check_status()
        for _ in range(min(warmup, 2)):
            yb = base.forward(x)
        torch.cuda.synchronize()
    except Exception as exc:
        ok, err = False, repr(exc)
    if not sync_and_check(ok, dev):
        print(f"[warm-up failed] rank{rank}: {err}", flush=True)
        return

    def timed(fn):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s, e = event_timer()
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) / iters]

    ours = max_rank_mean(timed(lambda: layer(x)), dev)
    lib = max_rank_mean(timed(lambda: base.forward(x)), dev)
    layer.check_status()
    if env_int("TRACE", 0):
        # per-rank overlap evidence: phase times and when received tiles became usable
        layer.profile = True
        layer.trace_arrivals = True
        if world > 1:
            dist.barrier()
        layer(x)
        phases = {k: round(v) for k, v in layer.phase_times_us().items()}
        arrivals = {k: (round(v, 1) if isinstance(v, float) else v) for k, v in layer.arrival_report().items()}
        layer.profile = layer.trace_arrivals = False
        print(json.dumps(dict(rank=rank, rows=int(layer.group_rows.sum().item()), phases_us=phases,
                              arrivals=arrivals)), flush=True)
    rows = int(layer.group_rows.sum().item())
    rows_max = int(allreduce_max(torch.tensor([rows], device=dev)).item())
    flops = 2.0 * rows_max * D * (3 * F if F > 0 else cfg.out_dim)
    scale = yb.float().abs().max().clamp_min(1e-6)
    row_err = (y.float() - yb.float()).abs().max(dim=1).values / scale
    err_rel = float(row_err.max().item())
    # tokens whose top-k choice is a near tie may be routed differently by two correct routers:
    # report the difference with and without them
    from iris_testing_b200.ops import cpu_ref
    clear = cpu_ref.clear_routing_mask(x, layer.router, topk, layer.router_bias)
    err_clear = float(row_err[clear].max().item()) if bool(clear.any()) else 0.0
    report(rank, dict(mode="layer", world=world, hidden=D, ffn=F, experts=cfg.num_experts, e_local=e_local,
                      topk=topk, batch=batch, seq=seq, zipf_s=zipf, recv_rows_max=rows_max,
                      fused_us=round(ours * 1e3, 1), library_us=round(lib * 1e3, 1),
                      speedup=round(lib / ours, 3), gemm_tflops_at_fused=round(flops / ours / 1e9, 1),
                      rel_diff_vs_library=round(err_rel, 5), rel_diff_clear_tokens=round(err_clear, 5),
                      ambiguous_tokens=int((~clear).sum().item()), capacity_rows=layer.cap_rows,
                      symmetric_mb=round(layer.memory_bytes()["symmetric"] / 1e6, 1),
                      local_mb=round(layer.memory_bytes()["local"] / 1e6, 1),
                      timing="CUDA events, mean over iters, max over ranks"))


def worker(rank: int, world: int, spawned: bool) -> None:
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 or not spawned:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        mode = os.getenv("MODE", "a2a")
        (run_layer if mode == "layer" else run_a2a)(rank, world, dev)
    finally:
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if "RANK" in os.environ:                          # launched by torch.distributed.run
        worker(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), spawned=False)
    else:
        world = env_int("WORLD_SIZE", torch.cuda.device_count() or 1)
        if world == 1:
            worker(0, 1, spawned=True)
        else:
            import torch.multiprocessing as mp
            mp.spawn(worker, args=(world, True), nprocs=world, join=True)
