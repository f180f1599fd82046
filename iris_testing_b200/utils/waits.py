"""Host-side bounded waits on device flags, and a timestamped trace marker
(unit_tests.py:17-43, benchmark.py:24-28)."""
from __future__ import annotations

import time
from typing import Sequence

import torch
import torch.distributed as dist


class WaitTimeout(RuntimeError):
    pass


def spin_wait_counts_ready(counts_ready: torch.Tensor, world_size: int, timeout_s: float = 10.0,
                           poll_s: float = 1e-3) -> None:
    """Poll ``counts_ready[0] >= world_size`` from the host; raise with a state dump on timeout."""
    t0 = time.time()
    while True:
        v = int(counts_ready.reshape(-1)[0].item())
        if v >= world_size:
            return
        if time.time() - t0 > timeout_s:
            raise WaitTimeout(f"counts_ready={v}, expected >= {world_size} after {timeout_s}s")
        time.sleep(poll_s)


def expected_tiles(pca: torch.Tensor, block_m: int, capacity: int | None = None) -> torch.Tensor:
    """Per local expert: sum over sources of ceil(pca[e, src] / block_m)."""
    p = pca.to(torch.int64)
    if capacity is not None:
        p = p.clamp(max=capacity)
    return ((p + block_m - 1) // block_m).sum(dim=1)


def spin_wait_token_sync(token_sync: torch.Tensor, expected: torch.Tensor | Sequence[int],
                         timeout_s: float = 10.0, poll_s: float = 1e-3) -> None:
    """Poll ``token_sync[e] >= expected[e]`` for every local expert."""
    exp = torch.as_tensor(expected).to("cpu", torch.int64)
    t0 = time.time()
    while True:
        cur = token_sync.to("cpu", torch.int64)
        if bool((cur >= exp).all()):
            return
        if time.time() - t0 > timeout_s:
            raise WaitTimeout(f"token_sync={cur.tolist()}, expected >= {exp.tolist()} after {timeout_s}s")
        time.sleep(poll_s)


def mark(msg: str) -> None:
    """``[unix_ts] rankN: msg`` on stdout, flushed."""
    r = dist.get_rank() if dist.is_available() and dist.is_initialized() else -1
    print(f"[{time.time():.3f}] rank{r}: {msg}", flush=True)
