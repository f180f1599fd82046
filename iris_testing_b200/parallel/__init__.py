"""Process-level plumbing: symmetric heap over NVLink peer memory, the CPU/gloo
backend, and the library all-to-all baseline."""
from .baseline_nccl import (AllToAllMoEBaseline, ExchangeBuffers, exchange_counts,
                            exchange_payload, init_baseline_buffers, relayout_to_token_buf,
                            run_baseline)
from .gloo_moe import moe_forward_gloo, padded_exchange, pair_message_rows
from .health import HealthMonitor


def SymmetricHeap(*args, **kwargs):
    """Lazy constructor: the native library is only touched when a heap is made."""
    from .symm import SymmetricHeap as _H
    return _H(*args, **kwargs)


def PaddedAllToAll(*args, **kwargs):
    """Lazy constructor of :class:`iris_testing_b200.parallel.padded_a2a.PaddedAllToAll`."""
    from .padded_a2a import PaddedAllToAll as _P
    return _P(*args, **kwargs)


def CapacityProbe(*args, **kwargs):
    """Lazy constructor of :class:`iris_testing_b200.parallel.padded_a2a.CapacityProbe`."""
    from .padded_a2a import CapacityProbe as _C
    return _C(*args, **kwargs)
