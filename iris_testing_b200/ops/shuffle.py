"""Token shuffle (drop the padding) and its inverse.

Reference design: layers/token_shuffle.py:7-61 / kernels.py:150-205 -- wait for
the dispatch flags, then copy the valid rows ``token_buf[e, src, m < pca[e, src]]``
to a packed ``[S_total, H]`` buffer ordered by (expert, src, arrival), which is
the order the grouped GEMM consumes.  The reference's device-side wait is
unbounded; this one gives up after a time budget and reports a status.
``unshuffle`` (not in the reference) scatters packed rows back to the padded layout.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from .. import _native as nv
from . import cpu_ref
from ._common import declare, default_status, ptr, require, stream_ptr
from .dispatch import tile_rows


def _fn():
    return declare("b200_shuffle", [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_void_p, C.c_int, C.c_void_p, C.c_ulonglong, C.c_void_p])


def shuffle(dispatched_tokens: torch.Tensor, pca: torch.Tensor, token_sync: Optional[torch.Tensor] = None,
            counts_ready: Optional[torch.Tensor] = None, *, max_rows: Optional[int] = None,
            status: Optional[torch.Tensor] = None, wait_budget_ms: float = 2000.0
            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """token_buf [e_local, world, CAP, H], pca [e_local, world] -> (packed, rows per expert).

    When ``token_sync`` and ``counts_ready`` are given the kernel first waits (bounded) for
    the dispatch to land.  On CUDA ``packed`` has ``max_rows`` rows (default: every cell
    full) so that no host synchronisation is needed; only the first ``sum(rows)`` are valid.
    More valid rows than ``max_rows`` are not copied: the kernel records an overflow (with the
    number of rows needed) in ``status`` -- the device's default status word when none is given,
    see :func:`iris_testing_b200.ops.check_default_status`.
    """
    e_local, world, cap, H = dispatched_tokens.shape
    if not dispatched_tokens.is_cuda:
        return cpu_ref.shuffle_ref(dispatched_tokens, pca)
    require(dispatched_tokens.is_contiguous() and H % 8 == 0 and dispatched_tokens.element_size() == 2,
            "token_buf must be contiguous 16-bit with hidden_dim % 8 == 0")
    rows = max_rows if max_rows is not None else e_local * world * cap
    packed = torch.empty((rows, H), dtype=dispatched_tokens.dtype, device=dispatched_tokens.device)
    group_rows = torch.empty((e_local,), dtype=torch.int32, device=pca.device)
    wait = int(token_sync is not None and counts_ready is not None)
    if status is None:
        status = default_status(pca.device)
    rc = _fn()(ptr(dispatched_tokens), ptr(packed), ptr(pca), ptr(counts_ready), ptr(token_sync),
               world, e_local, cap, H, tile_rows(), wait, 0, ptr(group_rows), rows, ptr(status),
               int(wait_budget_ms * 1e6), stream_ptr(pca))
    nv.check(rc, "shuffle launch")
    return packed, group_rows


def unshuffle(packed: torch.Tensor, pca: torch.Tensor, capacity: int,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inverse of :func:`shuffle`: packed rows back into ``[e_local, world, CAP, H]``.

    Padding rows of a freshly allocated ``out`` are zero; a caller-provided ``out``
    keeps whatever its padding rows held.
    """
    e_local, world = pca.shape
    H = packed.shape[1]
    if not packed.is_cuda:
        return cpu_ref.unshuffle_ref(packed, pca, capacity)
    if out is None:
        out = torch.zeros((e_local, world, capacity, H), dtype=packed.dtype, device=packed.device)
    rc = _fn()(ptr(out), ptr(packed), ptr(pca), None, None, world, e_local, capacity, H, tile_rows(),
               0, 1, None, packed.shape[0], ptr(default_status(pca.device)), 0, stream_ptr(pca))
    nv.check(rc, "unshuffle launch")
    return out


class TokenShuffle(torch.autograd.Function):
    """``shuffle = TokenShuffle.apply(dispatched_tokens, pca, token_sync)`` (layers/token_shuffle.py:61)."""

    @staticmethod
    def forward(ctx, dispatched_tokens, pca, token_sync=None, counts_ready=None):
        packed, _ = shuffle(dispatched_tokens, pca, token_sync, counts_ready)
        return packed

    @staticmethod
    def backward(ctx, *grad_outputs):
        raise NotImplementedError("the shuffle op is forward-only")
