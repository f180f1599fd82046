#!/usr/bin/env python
"""Multi-process GPU unit tests (one process per GPU), runnable without pytest.

Counterpart of the reference's ``unit_tests.py`` (unit_tests.py:126-243): the dispatch
op is driven with deterministic *full* routing (every (dst, expert) cell gets exactly
``cap`` rows) and a payload whose values encode their coordinates, then every
(src, expert) block of ``token_buf`` is compared for exact equality with what the
source sent, after bounded host-side waits on ``counts_ready`` / ``token_sync``.
Added here: the return path (combine) on the same data and the fused MoE layer
against the dense reference.  ``WORLD_SIZE`` defaults to the number of visible GPUs.

    python unit_tests.py                         # spawns WORLD_SIZE processes
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 unit_tests.py
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent))


def _gather(t):
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def test_custom_a2a(heap, e_local: int, hidden_dim: int, cap: int) -> None:
    from iris_testing_b200.ops import custom_a2a, shuffle
    from iris_testing_b200.ops.combine import padded_return
    from iris_testing_b200.utils import (alloc_return_buffers, alloc_shmem_buffers, build_dst_offsets,
                                         expected_tiles, reset_dispatch_flags, spin_wait_counts_ready,
                                         spin_wait_token_sync)
    rank, world, dev = heap.rank, heap.world, heap.device
    counts = torch.full((world, e_local), cap, dtype=torch.int32, device=dev)
    d = torch.arange(world, device=dev).view(world, 1, 1)
    e = torch.arange(e_local, device=dev).view(1, e_local, 1)
    t = torch.arange(cap, device=dev).view(1, 1, cap)
    # small integers are exact in bf16, so distinct coordinates never collide
    val = (rank * 61 + d * 17 + e * 5 + t) % 251
    payload = val.reshape(-1, 1).expand(-1, hidden_dim).to(torch.bfloat16).contiguous()
    b = alloc_shmem_buffers(heap, world, e_local, cap, hidden_dim, torch.bfloat16)
    r = alloc_return_buffers(heap, world, e_local, cap, hidden_dim, torch.bfloat16)
    heap.barrier()
    for _ in range(2):
        reset_dispatch_flags(b)
        r.ret_sync.zero_()
        heap.barrier()
        custom_a2a(payload, counts, build_dst_offsets(counts), b.pca, b.token_buf, b.counts_ready,
                   b.token_sync, b.heap_bases, e_local * world, cap)
        spin_wait_counts_ready(b.counts_ready, world, timeout_s=10)
        spin_wait_token_sync(b.token_sync, expected_tiles(b.pca, int(os.getenv("TOK_BLOCK_M", "32"))),
                             timeout_s=10)
        everyone = torch.stack(_gather(payload)).view(world, world, e_local, cap, hidden_dim)
        for src in range(world):
            for el in range(e_local):
                assert torch.equal(b.token_buf[el, src], everyone[src, rank, el]), (rank, src, el)
        assert torch.equal(b.pca, torch.full((e_local, world), cap, dtype=torch.int32, device=dev))
        # return path: every row must come home to the cell it was sent from
        padded_return(b.token_buf, b.pca, r.ret_buf, r.ret_sync, b.heap_bases)
        spin_wait_token_sync(r.ret_sync, [e_local * ((cap + 31) // 32)] * world, timeout_s=10)
        assert torch.equal(r.ret_buf.view(-1, hidden_dim), payload), rank
        heap.barrier()
    packed, rows = shuffle(b.token_buf, b.pca, b.token_sync, b.counts_ready)
    assert rows.tolist() == [cap * world] * e_local
    heap.check_status()


def test_fused_layer(heap, D: int, F: int, e_local: int, topk: int, T: int) -> None:
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer
    from iris_testing_b200.ops import cpu_ref
    from iris_testing_b200.utils import gen_local_tokens
    world, rank, dev = heap.world, heap.rank, heap.device
    cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=e_local * world, topk=topk, world_size=world,
                    gated=F > 0)
    layer = MoELayer(cfg, max_tokens=T, heap=heap, router_std=None)
    w1, w3, w2 = layer.reference_weights()
    for i in range(3):
        x = gen_local_tokens(1, T, D, torch.bfloat16, dev, i, rank, "normal")
        y = layer(x)
        if F > 0:
            ref = cpu_ref.dense_moe_ref(x, layer.router, topk, w1=torch.cat(_gather(w1)),
                                        w3=torch.cat(_gather(w3)), w2=torch.cat(_gather(w2)),
                                        round_hidden=torch.bfloat16)
        else:
            ref = cpu_ref.dense_moe_ref(x, layer.router, topk, w_single=torch.cat(_gather(w1)))
        err, scale = float((y.float() - ref).abs().max()), float(ref.abs().max())
        assert err <= 3e-2 * scale, (rank, i, err, scale)
    # the same step replayed from a CUDA graph captured once (all ranks capture and replay in step)
    layer.capture(T)
    for _ in range(3):
        y = layer.replay(x)
        err = float((y.float() - ref).abs().max())
        assert err <= 3e-2 * scale, (rank, "graph", err, scale)
    layer.check_status()


def _worker(rank: int, world: int) -> None:
    from iris_testing_b200.parallel.symm import SymmetricHeap
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    heap = SymmetricHeap(int(os.getenv("SYMM_HEAP_SIZE", os.getenv("IRIS_HEAP_SIZE", str(1 << 30)))))
    say = (lambda *a: print(*a, flush=True)) if rank == 0 else (lambda *a: None)
    test_custom_a2a(heap, e_local=2, hidden_dim=128, cap=32)
    say("test_custom_a2a(e_local=2, H=128, cap=32) PASSED")
    test_custom_a2a(heap, e_local=4, hidden_dim=256, cap=16)
    say("test_custom_a2a(e_local=4, H=256, cap=16) PASSED")
    test_fused_layer(heap, D=256, F=512, e_local=2, topk=2, T=300)
    say("test_fused_layer(gated) PASSED")
    test_fused_layer(heap, D=256, F=0, e_local=4, topk=1, T=77)
    say("test_fused_layer(single Linear, one kernel) PASSED")
    test_fused_layer(heap, D=1024, F=768, e_local=8, topk=4, T=1500)
    say("test_fused_layer(many experts) PASSED")
    dist.barrier()
    dist.destroy_process_group()
    say("ALL PASSED")


if __name__ == "__main__":
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29501")
    if "RANK" in os.environ:
        _worker(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]))
    else:
        import torch.multiprocessing as mp
        world = int(os.getenv("WORLD_SIZE", str(torch.cuda.device_count() or 1)))
        mp.spawn(_worker, args=(world,), nprocs=world, join=True)
