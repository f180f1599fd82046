"""Padded all-to-all dispatch with the reference's buffer contract.

``custom_a2a(tokens, dest_counts, dst_offsets, local_pca, token_buf,
counts_ready, token_sync, heap_bases, experts, capacity)`` keeps the ten
positional arguments of the reference op (layers/all_to_all.py:13-46) and
returns ``token_buf`` without waiting for remote arrival (layers/all_to_all.py:119);
consumers wait on ``counts_ready`` / ``token_sync`` (the shuffle op does).

CUDA tensors: one kernel pushes counts and token rows straight into the peers'
symmetric buffers and signals per tile (csrc/exchange.cu).  CPU tensors: the same
contract over a gloo ``all_to_all_single`` (used by the plumbing tests).
"""
from __future__ import annotations

import ctypes as C
import os

import torch
import torch.distributed as dist

from .. import _native as nv
from ._common import declare, ptr, require, stream_ptr

def register_heap(heap) -> None:
    """Kept for callers of earlier versions: the heap-bases table now carries a weak reference
    to its heap, so nothing needs registering and nothing outlives the heap."""
    heap.get_heap_bases()


def _heap_of(heap_bases):
    if hasattr(heap_bases, "peer_ptrs"):
        return heap_bases
    ref = getattr(heap_bases, "_b200_heap", None)
    h = ref() if ref is not None else None
    if h is None or h.closed:
        raise ValueError("heap_bases must be the tensor returned by SymmetricHeap.get_heap_bases() "
                         "of a live heap (or the SymmetricHeap itself)")
    return h


def tile_rows() -> int:
    """Rows per dispatch tile / completion signal (reference: BLOCK_M=32, env TOK_BLOCK_M)."""
    return int(os.getenv("TOK_BLOCK_M", "32"))


def _cpu_dispatch(tokens, dest_counts, dst_offsets, local_pca, token_buf, counts_ready, token_sync,
                  experts, capacity):
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    e_local = experts // world
    H = tokens.shape[-1]
    bm = tile_rows()
    # fixed-size padded message per (dst, expert) cell
    send = tokens.new_zeros(world, e_local, capacity, H)
    sc = dest_counts.tolist()
    off = 0
    for d in range(world):
        for e in range(e_local):
            n = sc[d][e]
            send[d, e, :min(n, capacity)] = tokens[off:off + min(n, capacity)]
            off += n
    recv = torch.empty_like(send)
    recv_counts = torch.empty_like(dest_counts)
    if world > 1:
        dist.all_to_all_single(recv_counts, dest_counts.contiguous())
        dist.all_to_all_single(recv, send)
    else:
        recv_counts.copy_(dest_counts)
        recv.copy_(send)
    local_pca.copy_(recv_counts.t())
    token_buf.copy_(recv.permute(1, 0, 2, 3))
    counts_ready.fill_(world)
    tiles = (local_pca.clamp(max=capacity) + bm - 1) // bm
    token_sync.copy_(tiles.sum(dim=1).to(token_sync.dtype))
    return token_buf


class AllToAllOp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, dest_counts, dst_offsets, local_pca, token_buf, counts_ready,
                token_sync, heap_bases, experts, capacity):
        require(dest_counts.dtype == torch.int32 and dst_offsets.dtype == torch.int32,
                "dest_counts and dst_offsets must be int32")
        require(capacity == token_buf.shape[2], "capacity must equal token_buf.shape[2]")
        if not tokens.is_cuda:
            return _cpu_dispatch(tokens, dest_counts, dst_offsets, local_pca, token_buf,
                                 counts_ready, token_sync, experts, capacity)
        heap = _heap_of(heap_bases)
        world, rank = heap.world, heap.rank
        require(experts % world == 0, "experts must be divisible by the EP group size")
        e_local = experts // world
        H = tokens.shape[-1]
        require(tokens.is_contiguous() and tokens.element_size() == 2 and H % 8 == 0,
                "tokens must be contiguous 16-bit with hidden_dim % 8 == 0")
        fn = declare("b200_padded_dispatch",
                     [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_ulonglong),
                      C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong),
                      C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p])
        rc = fn(ptr(tokens), ptr(dest_counts), ptr(dst_offsets), heap.peer_ptrs(local_pca),
                heap.peer_ptrs(token_buf), heap.peer_ptrs(counts_ready), heap.peer_ptrs(token_sync),
                rank, world, e_local, capacity, H, tile_rows(), ptr(heap.status), stream_ptr(tokens))
        nv.check(rc, "padded dispatch launch")
        return token_buf

    @staticmethod
    def backward(ctx, *grad_outputs):
        raise NotImplementedError("the dispatch op is forward-only")


custom_a2a = AllToAllOp.apply


def zero_padding(token_buf: torch.Tensor, pca: torch.Tensor) -> torch.Tensor:
    """Zero every padding row ``token_buf[e, src, m >= pca[e, src]]`` in place.

    The dispatch transfers valid rows only (as the reference does, kernels.py:104), so a
    reused buffer keeps stale rows from an earlier, larger message in its padding.  Call this
    after the dispatch has landed when the consumer reads the padded layout directly; the
    shuffle and the grouped GEMM never look at padding rows.  Plain tensor ops, any device."""
    cap = token_buf.shape[2]
    m = torch.arange(cap, device=token_buf.device).view(1, 1, cap)
    pad = m >= pca.to(token_buf.device).unsqueeze(-1)
    token_buf.masked_fill_(pad.unsqueeze(-1), 0)
    return token_buf

