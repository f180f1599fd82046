"""Host-side liveness check between steps.

A rank may only leave a job between steps, with none of its kernels or collectives in
flight.  The others must learn of it on the host *before* their next launch: a fused step
whose peer is gone would only end when its bounded device waits run out.  ``HealthMonitor``
keeps a small gloo group with a short timeout next to the data-plane process group; one
tiny all-reduce per check either returns every rank's vote or raises within the timeout.

Counterpart of the reference's rank-agreement idiom (benchmark.py:31-35, 203-236): all ranks
agree on "healthy" before the next collective, so nobody is left waiting alone.
"""
from __future__ import annotations

import datetime
from typing import Optional

import torch
import torch.distributed as dist


class HealthMonitor:
    def __init__(self, timeout_s: float = 5.0, ranks: Optional[list] = None) -> None:
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("HealthMonitor needs an initialised process group")
        self.timeout_s = float(timeout_s)
        self.group = dist.new_group(ranks=ranks, backend="gloo",
                                    timeout=datetime.timedelta(seconds=self.timeout_s))
        self.last_error: Optional[str] = None

    def all_alive(self, healthy: bool = True) -> bool:
        """True only if every rank answered within the timeout and voted ``healthy``."""
        vote = torch.tensor([1 if healthy else 0], dtype=torch.int32)
        try:
            dist.all_reduce(vote, op=dist.ReduceOp.MIN, group=self.group)
        except Exception as exc:          # a peer is gone or did not answer in time
            self.last_error = f"{type(exc).__name__}: {exc}"[:300]
            return False
        return bool(vote.item() == 1)

    def step_done(self) -> bool:
        """Call after the step's ``torch.cuda.synchronize()``: a host-side handshake meaning "this
        step is finished on every rank's device".  Once it returns True no rank has a store into
        a peer's memory outstanding (the last kernel of a fused step publishes its retire stamp
        into the peers' heaps), so a rank may leave now.  False when a peer did not answer."""
        return self.all_alive(True)
