"""Per-kernel micro-benchmarks with roofline fractions.

    python -m iris_testing_b200.bench_kernels gemm   [--groups 4 --rows 4096 --n 2048 --k 4096 --gated 0]
    python -m iris_testing_b200.bench_kernels router [--tokens 16384 --hidden 4096 --experts 8 --topk 2]
    python -m iris_testing_b200.bench_kernels plan   [--tokens 16384 --experts 8 --topk 2]
    python -m iris_testing_b200.bench_kernels layer  [--model mixtral-8x7b --tokens 16384 --graph 0]
    python -m iris_testing_b200.bench_kernels pipeline [--tokens 8192 --hidden 2048 --experts 8 --topk 2]

Each sub-command warms up, times ``--iters`` launches with CUDA events and prints one JSON
line: achieved TFLOP/s or GB/s and the fraction of the measured peaks (``MEASURED_PEAKS.json``
at the repository root when present: a plain device copy and a cuBLAS bf16 GEMM; otherwise
6.65 TB/s and 1.59 PFLOP/s, marked "of fallback").  Small default sizes keep a profiler
capture of one launch short while still exceeding the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch


def peaks():
    p = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d["bf16_tflops"], tflops_sustained=d.get("bf16_tflops_sustained"),
                    kind="of measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, kind="of fallback")


def time_launches(fn, iters: int, warmup: int = 3) -> float:
    """Mean milliseconds per call; an L2-sized buffer is rewritten between timed calls."""
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters


def cmd_gemm(a) -> dict:
    from . import _native as nv
    from .ops import grouped_gemm
    dev = torch.device("cuda")
    G, M, N, K = a.groups, a.rows, a.n, a.k
    x = torch.randn(G * M, K, device=dev).to(torch.bfloat16)
    w = (torch.randn(G, N, K, device=dev) * 0.02).to(torch.bfloat16)
    rows = torch.full((G,), M, dtype=torch.int32, device=dev)
    epi = nv.EPI_SILU_GATE if a.gated else nv.EPI_STORE
    out = torch.empty(G * M, N // 2 if a.gated else N, dtype=torch.bfloat16, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    ms = time_launches(lambda: grouped_gemm(x, w, rows, epilogue=epi, out=out, status=status,
                                            group_m=a.group_m), a.iters)
    flops = 2.0 * G * M * N * K
    pk = peaks()
    tf = flops / ms / 1e9
    byts = (x.numel() + w.numel() + out.numel()) * 2
    return dict(kernel="grouped_gemm", groups=G, rows=M, N=N, K=K, gated=bool(a.gated), ms=round(ms, 4),
                tflops=round(tf, 1), frac_of_peak=round(tf / pk["tflops"], 3), peak=pk["kind"],
                algorithmic_mb=round(byts / 1e6, 1), status=int(status[0].item()))


def cmd_router(a) -> dict:
    from .ops import router_topk
    from .utils import gen_local_tokens, gen_router
    dev = torch.device("cuda")
    x = gen_local_tokens(1, a.tokens, a.hidden, torch.bfloat16, dev, 0, 0, "normal")
    wr = gen_router(a.hidden, a.experts, torch.bfloat16, dev, 0, std=None)
    ms = time_launches(lambda: router_topk(x, wr, a.topk), a.iters)
    byts = x.numel() * 2 + wr.numel() * 2 + a.tokens * a.topk * 8
    pk = peaks()
    gbs = byts / ms / 1e6
    return dict(kernel="router_topk", tokens=a.tokens, hidden=a.hidden, experts=a.experts, topk=a.topk,
                ms=round(ms, 4), gbs=round(gbs, 1), frac_of_hbm=round(gbs / pk["hbm_gbs"], 3), peak=pk["kind"])


def cmd_plan(a) -> dict:
    from .ops import make_plan
    dev = torch.device("cuda")
    idx = torch.randint(0, a.experts, (a.tokens, a.topk), dtype=torch.int32, device=dev)
    ms = time_launches(lambda: make_plan(idx, a.experts), a.iters)
    return dict(kernel="plan (2 launches)", tokens=a.tokens, experts=a.experts, topk=a.topk, ms=round(ms, 4))


def cmd_layer(a) -> dict:
    from .config import preset
    from .models import MoELayer, heap_bytes_needed
    from .parallel.symm import SymmetricHeap
    from .utils import gen_local_tokens
    cfg = preset(a.model)
    heap = SymmetricHeap(heap_bytes_needed(cfg, a.tokens) + (64 << 20))
    layer = MoELayer(cfg, max_tokens=a.tokens, heap=heap, router_std=None)
    x = gen_local_tokens(1, a.tokens, cfg.hidden_dim, torch.bfloat16, heap.device, 0, 0, "normal")
    if a.graph:                                   # replay a captured CUDA graph instead of 6 launches
        layer.capture(a.tokens)
        ms = time_launches(lambda: layer.replay(x), a.iters)
    else:
        ms = time_launches(lambda: layer(x), a.iters)
    layer.check_status()
    flops = 2.0 * a.tokens * cfg.topk * cfg.hidden_dim * 3 * cfg.ffn_dim
    pk = peaks()
    tf = flops / ms / 1e9
    return dict(kernel="MoELayer.forward (1 GPU)" + (", CUDA graph replay" if a.graph else ""),
                model=a.model, tokens=a.tokens, ms=round(ms, 4),
                tflops=round(tf, 1), frac_of_peak=round(tf / pk["tflops"], 3),
                frac_of_sustained=round(tf / pk["tflops_sustained"], 3) if pk["tflops_sustained"] else None,
                peak=pk["kind"])


def cmd_pipeline(a) -> dict:
    """The unfused, reference-shaped pipeline on one GPU, one launch of every stand-alone kernel:
    router (CUDA-core variant) -> plan -> pack -> padded dispatch -> shuffle -> expert GEMM ->
    SiLU gate -> unshuffle -> padded return -> weighted gather, plus the barrier."""
    from .ops import custom_a2a, expert, router_topk, shuffle, silu_gate, unshuffle
    from .ops.combine import padded_return, weighted_gather
    from .parallel.symm import SymmetricHeap
    from .utils import (alloc_return_buffers, alloc_shmem_buffers, gen_local_tokens, gen_local_weights,
                        gen_router, reset_dispatch_flags, route_and_pack)
    dev = torch.device("cuda")
    T, D, E, k = a.tokens, a.hidden, a.experts, a.topk
    x = gen_local_tokens(1, T, D, torch.bfloat16, dev, 0, 0, "normal")
    router = gen_router(D, E, torch.bfloat16, dev, 0, std=None)
    w = gen_local_weights(E, D, D, torch.bfloat16, dev, 0, 0)
    cap = 2 * T * k // E
    heap = SymmetricHeap(2 * E * cap * D * 2 + (256 << 20))
    b = alloc_shmem_buffers(heap, 1, E, cap, D, torch.bfloat16)
    r = alloc_return_buffers(heap, 1, E, cap, D, torch.bfloat16)

    def once():
        router_topk(x, router, k, force_simple=True)
        payload, counts, dst_off, _, idx, wgt, plan = route_and_pack(x, router, k, 1, E)
        reset_dispatch_flags(b)
        r.ret_sync.zero_()
        heap.barrier(host_sync=False)
        custom_a2a(payload, counts, dst_off, b.pca, b.token_buf, b.counts_ready, b.token_sync,
                   b.heap_bases, E, cap)
        packed, rows = shuffle(b.token_buf, b.pca, b.token_sync, b.counts_ready, max_rows=T * k,
                               status=heap.status)
        out = expert(packed, w, rows)
        out = silu_gate(out, out)
        out_buf = unshuffle(out, b.pca, cap)
        padded_return(out_buf, b.pca, r.ret_buf, r.ret_sync, b.heap_bases)
        return weighted_gather(r.ret_buf, plan, idx, wgt, r.ret_sync, 1, cap, status=heap.status)

    ms = time_launches(once, a.iters, warmup=2)
    heap.check_status()
    return dict(kernel="unfused pipeline (1 GPU)", tokens=T, hidden=D, experts=E, topk=k, cap=cap,
                ms=round(ms, 4), payload_mb=round(T * k * D * 2 / 1e6, 1))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--groups", type=int, default=4); g.add_argument("--rows", type=int, default=4096)
    g.add_argument("--n", type=int, default=2048); g.add_argument("--k", type=int, default=4096)
    g.add_argument("--gated", type=int, default=0); g.add_argument("--group-m", dest="group_m", type=int, default=0)
    r = sub.add_parser("router")
    r.add_argument("--tokens", type=int, default=16384); r.add_argument("--hidden", type=int, default=4096)
    r.add_argument("--experts", type=int, default=8); r.add_argument("--topk", type=int, default=2)
    p = sub.add_parser("plan")
    p.add_argument("--tokens", type=int, default=16384); p.add_argument("--experts", type=int, default=8)
    p.add_argument("--topk", type=int, default=2)
    l = sub.add_parser("layer")
    l.add_argument("--model", default="mixtral-8x7b"); l.add_argument("--tokens", type=int, default=16384)
    l.add_argument("--graph", type=int, default=0)
    q = sub.add_parser("pipeline")
    q.add_argument("--tokens", type=int, default=8192); q.add_argument("--hidden", type=int, default=2048)
    q.add_argument("--experts", type=int, default=8); q.add_argument("--topk", type=int, default=2)
    for s in (g, r, p, l, q):
        s.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    out = dict(gemm=cmd_gemm, router=cmd_router, plan=cmd_plan, layer=cmd_layer, pipeline=cmd_pipeline)[a.cmd](a)
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
