#!/usr/bin/env python
"""Two-arm benchmark: this library against the unmodified reference, same loops, same config.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the reference's NCCL path (baseline/_ref)

Default (the headline): latency of one expert-parallel MoE layer -- dispatch all-to-all, expert
GEMMs, combine -- Mixtral-8x7B shape (D=4096, F=14336, E=8, top-2, SiLU-gated), B=4, S=4096
tokens per rank (weak scaling), bf16, x ~ N(0,1), router ~ N(0, 1/D), expert weights ~
N(0, 0.02); seeded synthetic data, random-init weights.  Other configurations:

    --model fine-grained [--experts E --topk k]     D=2048, F=1408, B=8, S=2048
    --model large --zipf 1.2                        D=6144, F=16384, B=8, S=4096, skewed routing
    --mode a2a [--combine] [--batch B --seq S]      padded all-to-all alone, D=4096, 8 experts/GPU

Rank 0 prints ONE JSON line.  ``value`` is microseconds per step (device-timed with CUDA events,
max over ranks; lower is better); ``e2e`` is the same step through the public API including,
every step, the host->device copy of that step's tokens from pinned memory and a device->host
read of the step's result.  Both arms run the same timing and staging loops
(``iris_testing_b200/bench_harness.py``) and print the same ``config``.  After the timed regions
the library arm checks one step against an oracle (``check``) and exits non-zero if it fails.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from iris_testing_b200.bench_harness import (MODEL_DEFAULTS, ClockSampler, NvlinkCounters,  # noqa: E402
                                             describe_config, device_timed, e2e_loop, fence, make_config,
                                             max_over_ranks)

METRIC = "moe_a2a_gemm_layer_us_max_over_ranks"
METRIC_A2A = "padded_a2a_us_max_over_ranks"


def init_dist(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus and not (n_gpus == 1 and world == 1):
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    return rank, world, local, torch.device("cuda", local)


def emit(args, cfg, rank, world, us, e2e, launches, clocks, impl, timed, memory, check, extra=None):
    if rank != 0:
        return
    tokens_total = args.batch * args.seq * world
    line = {
        "metric": METRIC if args.mode == "layer" else METRIC_A2A, "value": round(us, 2), "unit": "us",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(us / 1000.0, 5),
        "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded N(0,1) tokens, random-init weights)", "impl": impl,
        "tokens_per_s": round(tokens_total / (us * 1e-6), 1),
        "config": describe_config(args, cfg, world),
        "clocks": clocks, "gpu_launches": launches, "e2e": e2e,
        "time_x_sm_mhz": (round(us * clocks["sm_mhz"], 0) if clocks.get("sm_mhz") else None),
        "timed": timed, "memory": memory, "check": check,
    }
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def run_arm(args, arm, cfg, rank, world, local, dev, impl, count_fn=None) -> int:
    sampler = ClockSampler(local)
    sampler.start()
    arm.settle()
    for i in range(args.warmup):
        arm.run(arm.inputs[i & 1], i)
    fence(world)
    arm.check_status()
    links = NvlinkCounters(local)
    before = count_fn() if count_fn else 0
    nv0 = links.read()
    us = device_timed(arm, args.steps, world, sampler)
    nv1 = links.read()
    algo = arm.remote_bytes()          # from the routing of the last timed step
    launches = int(count_fn() - before) if count_fn else 0
    clocks = sampler.stop()
    arm.check_status()
    us = max_over_ranks(us, dev, world)
    e2e_loop(arm, max(2, min(args.warmup, 3)), world, dev)
    e2e_us = max_over_ranks(e2e_loop(arm, args.steps, world, dev), dev, world)
    arm.check_status()
    e2e = {"value": round(e2e_us, 2), "unit": "us", "h2d_bytes_per_step": arm.h2d_bytes,
           "d2h_bytes_per_step": 4, "api": arm.api,
           "loop": "pinned H2D on a copy stream one step ahead, result scalar read one step late (both arms)"}
    check = arm.check(args.check_tokens) if not args.no_check else None
    if count_fn and launches != arm.launches_expected(args.steps):      # counted vs expected: report only
        print(f"note: {launches} launches counted, {arm.launches_expected(args.steps)} expected",
              file=sys.stderr, flush=True)
    extra = dict(getattr(arm, "extra", None) or {})
    # NVLink bytes of rank 0's GPU during the device-timed region (NVML counters, read only) next
    # to the bytes the routing says must cross the links
    if nv0 is not None and nv1 is not None:
        extra["nvlink"] = dict(tx_bytes_per_step=round((nv1[0] - nv0[0]) / args.steps),
                               rx_bytes_per_step=round((nv1[1] - nv0[1]) / args.steps),
                               algorithmic_bytes_per_step=algo, source="NVML NVLINK_THROUGHPUT_DATA_TX/RX, rank 0")
    elif algo is not None:
        extra["nvlink"] = dict(counters="not readable on this box", algorithmic_bytes_per_step=algo)
    emit(args, cfg, rank, world, us, e2e, launches, clocks, impl, arm.timed, arm.memory(), check, extra=extra)
    return 0 if (check is None or check.get("ok", True)) else 3


SWEEPS = {
    # padded all-to-all alone, dispatch and dispatch+combine: batch sweep at S=1024, sequence sweep at B=4
    "config2": [dict(mode="a2a", batch=b, seq=1024, combine=c) for c in (False, True) for b in (1, 2, 4, 8, 16)]
               + [dict(mode="a2a", batch=4, seq=q, combine=c) for c in (False, True)
                  for q in (128, 256, 512, 2048, 4096)],
    # fine-grained experts: experts over the whole group x top-k
    "config4": [dict(mode="layer", model="fine-grained", experts=e, topk=k, batch=8, seq=2048)
                for e in (8, 32, 128) for k in (1, 2, 8)]
               + [dict(mode="layer", model="fine-grained", experts=e, topk=k, batch=8, seq=2048)
                  for e, k in ((16, 2), (64, 2), (64, 4), (64, 8))],
    # large experts, skewed and balanced routing
    "config5": [dict(mode="layer", model="large", zipf=z, batch=8, seq=4096, experts=0, topk=0) for z in (1.2, 0.0)],
    # the headline layer at small batches (the regime where the expert weights are streamed once per step)
    "small": [dict(mode="layer", model="mixtral-8x7b", batch=1, seq=q, experts=0, topk=0)
              for q in (64, 256, 512, 1024, 2048)],
}


def run_points(args, make_arm, rank, world, local, dev, impl, count_fn=None) -> int:
    """One JSON line per point of ``--sweep`` (or the single configuration), in one process."""
    import copy
    import gc
    points = SWEEPS[args.sweep] if args.sweep else [dict()]
    rc = 0
    for pt in points:
        a = copy.copy(args)
        for k, v in pt.items():
            setattr(a, k, v)
        if a.mode == "layer" and a.experts and a.experts % world:
            continue                                    # this expert count cannot be split over the ranks
        if a.mode == "layer" and a.experts and a.topk > a.experts:
            continue
        cfg = make_config(a, world)
        arm = make_arm(a)
        rc = max(rc, run_arm(a, arm, cfg, rank, world, local, dev, impl, count_fn))
        arm.close()
        del arm
        gc.collect()
        torch.cuda.empty_cache()
        fence(world)
    return rc


def run_ours(args) -> int:
    from iris_testing_b200 import _native
    from iris_testing_b200.bench_harness import A2AArm, LayerArm
    rank, world, local, dev = init_dist(args.gpus)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    count_fn = _native.lib().b200_launch_count      # incremented by every native launcher
    count_fn.restype = ctypes.c_longlong
    rc = run_points(args, lambda a: (LayerArm if a.mode == "layer" else A2AArm)(a, rank, world, dev),
                    rank, world, local, dev, "ours", count_fn)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return rc


# --------------------------------------------------------------------------- reference arm
def ensure_reference() -> str | None:
    """Returns an error string, or None once ``baseline/_ref`` holds the reference modules."""
    ref = ROOT / "baseline" / "_ref"
    if (ref / "baseline.py").exists() and (ref / "utils.py").exists():
        return None
    # not shipped with this checkout: install it now if the reference tree is mounted
    # REFERENCE_DIR, or a "reference" directory next to this repository
    src = Path(os.environ.get("REFERENCE_DIR", str(ROOT.parent / "reference")))
    if int(os.environ.get("RANK", "0")) == 0 and src.exists():
        sys.path.insert(0, str(ROOT / "baseline"))
        try:
            from install_reference import install
            err = install(src)
        except Exception as exc:
            err = repr(exc)[:200]
        if err is not None:
            return f"reference install failed: {err}"
    elif src.exists():                      # other ranks wait for rank 0's install
        t0 = time.time()
        while time.time() - t0 < 180 and not (ref / "unit_tests.py").exists():
            time.sleep(0.5)
        time.sleep(1.0)
    if (ref / "baseline.py").exists() and (ref / "utils.py").exists():
        return None
    return "baseline/_ref is missing and no reference tree is mounted to install it from"


def run_reference(args) -> int:
    err = ensure_reference()
    if err is not None:
        print(json.dumps({"impl": "reference", "unavailable": err}), flush=True)
        return 0
    sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    import importlib
    ref_baseline = importlib.import_module("baseline")     # the reference's baseline.py, unmodified
    ref_utils = importlib.import_module("utils")           # the reference's utils.py, unmodified
    from iris_testing_b200.bench_harness import RefA2AArm, RefLayerArm

    rank, world, local, dev = init_dist(args.gpus)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    def make(a):
        arm = (RefLayerArm if a.mode == "layer" else RefA2AArm)(ref_baseline, ref_utils, a, rank, world, dev)
        arm.extra = {"ref_packer": arm.packer}
        return arm

    rc = run_points(args, make, rank, world, local, dev, "reference")
    dist.barrier()
    dist.destroy_process_group()
    return rc


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--mode", choices=["layer", "a2a"], default="layer")
    ap.add_argument("--model", default="mixtral-8x7b", choices=sorted(set(MODEL_DEFAULTS) - {"a2a"}))
    ap.add_argument("--experts", type=int, default=0, help="experts over the whole EP group (0: the model's)")
    ap.add_argument("--topk", type=int, default=0, help="0: the model's")
    ap.add_argument("--batch", type=int, default=0, help="0: the configuration's default")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--hidden", type=int, default=4096, help="a2a mode: token width")
    ap.add_argument("--combine", action="store_true", help="a2a mode: include the return and the weighted sum")
    ap.add_argument("--zipf", type=float, default=0.0, help="Zipf exponent of a per-expert router bias (0: none)")
    ap.add_argument("--zipf-scale", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--check-tokens", type=int, default=2048)
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--sweep", choices=sorted(SWEEPS), default=None,
                    help="run every point of a published sweep in this one process, one JSON line each")
    ap.add_argument("--ref-packer", choices=["auto", "reference", "vectorized"], default="auto",
                    help="reference arm: its own Python packer, or the same payload built with tensor ops "
                         "(auto: its own packer up to 65536 routed copies)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    d = MODEL_DEFAULTS["a2a" if args.mode == "a2a" else args.model]
    args.batch = args.batch or d["batch"]
    args.seq = args.seq or d["seq"]
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    sys.exit(run_reference(args) if args.impl == "reference" else run_ours(args))


if __name__ == "__main__":
    main()
