"""Symmetric buffer sets with the reference's field names (utils.py:34-116).

``shmem`` is a :class:`~iris_testing_b200.parallel.symm.SymmetricHeap` on GPU, or
any object with ``zeros(shape, dtype)`` and ``get_heap_bases()`` (the CPU tests use
:class:`LocalHeap`).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


class LocalHeap:
    """Single-process stand-in for the symmetric heap (CPU tests, no peers)."""

    def __init__(self, device="cpu") -> None:
        self.device = torch.device(device)
        self.rank, self.world = 0, 1

    def zeros(self, shape, dtype, device=None) -> torch.Tensor:
        return torch.zeros(tuple(shape), dtype=dtype, device=self.device)

    def get_heap_bases(self) -> torch.Tensor:
        return torch.zeros(1, dtype=torch.int64, device=self.device)

    def barrier(self, *a, **k) -> None:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.barrier()


@dataclass
class CountsBuffers:
    pca: torch.Tensor            # int32 [e_local, world]
    counts_ready: torch.Tensor   # int32 [1]
    heap_bases: torch.Tensor


@dataclass
class TokenBuffers:
    token_buf: torch.Tensor      # [e_local, world, CAP, H]
    token_sync: torch.Tensor     # int32 [e_local]


@dataclass
class ShmemBuffers:
    pca: torch.Tensor
    counts_ready: torch.Tensor
    token_buf: torch.Tensor
    token_sync: torch.Tensor
    heap_bases: torch.Tensor


@dataclass
class ReturnBuffers:
    ret_buf: torch.Tensor        # [world(expert rank), e_local, CAP, H]
    ret_sync: torch.Tensor       # int32 [world]


def _register(shmem) -> torch.Tensor:
    bases = shmem.get_heap_bases()
    if hasattr(shmem, "peer_ptrs"):
        from ..ops.dispatch import register_heap
        register_heap(shmem)
    return bases


def alloc_counts_buffers(shmem, world_size: int, e_local: int) -> CountsBuffers:
    return CountsBuffers(pca=shmem.zeros((e_local, world_size), torch.int32),
                         counts_ready=shmem.zeros((1,), torch.int32), heap_bases=_register(shmem))


def alloc_token_buffers(shmem, world_size: int, e_local: int, capacity: int, hidden_dim: int,
                        token_dtype: torch.dtype) -> TokenBuffers:
    return TokenBuffers(token_buf=shmem.zeros((e_local, world_size, capacity, hidden_dim), token_dtype),
                        token_sync=shmem.zeros((e_local,), torch.int32))


def alloc_shmem_buffers(shmem, world_size: int, e_local: int, capacity: int, hidden_dim: int,
                        token_dtype: torch.dtype) -> ShmemBuffers:
    """All four dispatch buffers, zero-initialised, at identical offsets on every rank."""
    c = alloc_counts_buffers(shmem, world_size, e_local)
    t = alloc_token_buffers(shmem, world_size, e_local, capacity, hidden_dim, token_dtype)
    return ShmemBuffers(pca=c.pca, counts_ready=c.counts_ready, token_buf=t.token_buf,
                        token_sync=t.token_sync, heap_bases=c.heap_bases)


def alloc_return_buffers(shmem, world_size: int, e_local: int, capacity: int, out_dim: int,
                         dtype: torch.dtype) -> ReturnBuffers:
    return ReturnBuffers(ret_buf=shmem.zeros((world_size, e_local, capacity, out_dim), dtype),
                         ret_sync=shmem.zeros((world_size,), torch.int32))


def reset_counts_sync(cb) -> None:
    cb.counts_ready.zero_()


def reset_token_sync(tb) -> None:
    tb.token_sync.zero_()


def reset_token_buf_debug(tb) -> None:
    tb.token_buf.zero_()


def reset_dispatch_flags(b: ShmemBuffers, clear_tokens: bool = False) -> None:
    """What the reference does before every call (benchmark.py:176-180)."""
    b.pca.zero_()
    b.counts_ready.zero_()
    b.token_sync.zero_()
    if clear_tokens:
        b.token_buf.zero_()
