import os
import socket
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_entry(rank, world, port, fn, args, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def run_gloo(fn, world: int = 2, args=()):
    """Run ``fn(rank, world, *args)`` on ``world`` CPU processes over gloo; return the results."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = free_port()
        procs = [ctx.Process(target=_gloo_entry, args=(r, world, port, fn, args, ret))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        for p in procs:
            if p.is_alive():
                p.terminate()
                raise RuntimeError("gloo worker timed out")
            if p.exitcode != 0:
                raise RuntimeError(f"gloo worker exited with code {p.exitcode}")
        return [ret[r] for r in range(world)]
