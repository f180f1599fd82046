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
        clear = cpu_ref.clear_routing_mask(x, layer.router, topk)
        err, scale = float((y.float() - ref)[clear].abs().max()), float(ref.abs().max())
        assert err <= 1e-2 * scale and float(clear.float().mean()) > 0.95, (rank, i, err, scale)
    # the same step replayed from a CUDA graph captured once (all ranks capture and replay in step)
    layer.capture(T)
    for _ in range(3):
        y = layer.replay(x)
        err = float((y.float() - ref)[clear].abs().max())
        assert err <= 1e-2 * scale, (rank, "graph", err, scale)
    layer.check_status()


def test_heap_backends(world: int, rank: int, dev) -> None:
    """Every rank writes a pattern into every peer's copy of a symmetric tensor and every rank
    reads back what the others wrote, on both heap back-ends; closing the heaps gives the
    memory back."""
    from iris_testing_b200.parallel.symm import SymmetricHeap
    # the first use of the communicator and of peer access allocates driver / NCCL memory of its own:
    # warm both back-ends up before the reference reading
    dist.all_reduce(torch.zeros(1, device=dev))
    for backend in ("vmm", "ipc"):
        SymmetricHeap(8 << 20, backend=backend).close()
        dist.barrier()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for backend in ("vmm", "ipc"):
        heap = SymmetricHeap(32 << 20, backend=backend, max_bytes=128 << 20)
        assert heap.backend == backend, (heap.backend, heap.capabilities)
        t = heap.zeros((world, 1024), torch.int32)
        heap.barrier()
        for peer in range(world):
            src = torch.full((1024,), 1000 * rank + peer, dtype=torch.int32, device=dev)
            heap.copy_to_peer(t[rank], peer, src)             # row [rank] of the peer's copy
        torch.cuda.synchronize()
        heap.barrier()
        for src in range(world):
            assert int(t[src, 0]) == 1000 * src + rank and int(t[src, -1]) == 1000 * src + rank, (backend, src)
        for peer in range(world):                             # and read the peers' copies directly
            theirs = heap.copy_from_peer(t, peer)
            assert theirs[:, 7].tolist() == [1000 * s + peer for s in range(world)], (backend, peer)
        if backend == "vmm":                                  # growth is collective and moves nothing
            addr = t.data_ptr()
            big = heap.zeros((16 << 20,), torch.int32)        # 64 MiB > the 32 MiB mapped so far
            big.fill_(rank)
            heap.barrier()
            nxt = (rank + 1) % world
            assert int(heap.copy_from_peer(big[:8], nxt)[3]) == nxt and t.data_ptr() == addr
            del big
        heap.barrier()
        del t
        heap.close()
        dist.barrier()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert abs(free1 - free0) <= (16 << 20), (free0, free1)


def test_padded_engine(heap, e_local: int, H: int, T: int, topk: int, copy_mode: str) -> None:
    """The epoch-driven padded exchange with router-driven ragged counts, several exchanges in a
    row with changing routing: device-side capacity rule against host reductions, pca and
    the valid rows of token_buf bit-equal to the library all-to-all re-laid out, and the rows
    that come home summed with their weights."""
    from iris_testing_b200.parallel.baseline_nccl import ExchangeBuffers, relayout_to_token_buf, run_baseline
    from iris_testing_b200.parallel.padded_a2a import CapacityProbe, PaddedAllToAll
    from iris_testing_b200.utils import gen_local_tokens, gen_router, masked_stats, route_and_pack
    rank, world, dev = heap.rank, heap.world, heap.device
    E = e_local * world
    router = gen_router(H, E, torch.bfloat16, dev, 11, std=None)
    xs = [gen_local_tokens(1, T if (s + rank) % 3 else T // 2, H, torch.bfloat16, dev, 20 + s, rank, "normal")
          for s in range(3)]
    routed = [route_and_pack(x, router, topk, world, E) for x in xs]
    probe = CapacityProbe(heap, e_local)
    caps = torch.stack([probe.measure(r[1].contiguous()) for r in routed]).tolist()
    for c, r in zip(caps, routed):
        allc = torch.stack(_gather(r[1].contiguous()))                  # [src, dst, e]
        want = [int(allc.max()), int(allc.sum(dim=2).max()), int(allc.sum(dim=(0, 2)).max()),
                int(allc[:, rank].sum())]
        assert c == want, (rank, c, want)
    cap = max(c[0] for c in caps)
    a2a = PaddedAllToAll(heap, e_local, cap, H, torch.bfloat16, with_return=True, copy_mode=copy_mode)
    for x, (payload, counts, dst_off, _, idx, wgt, plan) in zip(xs, routed):
        a2a.dispatch(payload, counts, dst_off)
        a2a.wait()
        _, _, meta = run_baseline(payload, counts, cap, ExchangeBuffers(torch.empty_like(counts)))
        expected_pca = meta["recv_counts"].t().contiguous()
        assert torch.equal(a2a.pca, expected_pca), rank
        tb = relayout_to_token_buf(meta["recv_payload"], meta["recv_counts"], cap)
        mx, s1, s2 = masked_stats(a2a.token_buf, tb, expected_pca)
        assert float(mx) == 0.0, (rank, float(mx))
        a2a.send_back()
        y = a2a.reduce(plan, idx, wgt)
        ref = x.float() * wgt.sum(dim=1, keepdim=True)
        assert y.shape == ref.shape, (rank, y.shape, ref.shape)
        if ref.numel():                                   # a rank may hold no token in some exchange
            assert torch.allclose(y.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2), rank
    heap.check_status()


def test_skewed_layers(heap, D: int, F: int, e_local: int, topk: int, T: int) -> None:
    """Cross-rank corner cases of the fused layer: every token of every rank routed to rank 0's
    experts (all-to-one), a rank that holds no tokens at all, and a receive capacity that is
    too small at first (grown by ``forward_checked`` on every rank together)."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer
    from iris_testing_b200.ops import cpu_ref
    from iris_testing_b200.utils import gen_local_tokens
    world, rank, dev = heap.world, heap.rank, heap.device
    E = e_local * world
    cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=E, topk=topk, world_size=world,
                    capacity_factor=None, wait_budget_ms=heap.wait_budget_ns / 1e6)
    layer = MoELayer(cfg, max_tokens=T, heap=heap, router_std=None, debug_canaries=True)
    ws = [torch.cat(_gather(w)) for w in layer.reference_weights()]

    def check(x, tag):
        y = layer(x)
        torch.cuda.synchronize()
        layer.check_status()
        rep = cpu_ref.compare_with_dense(y, x, layer.router, topk, layer.last_routing[0], bias=layer.router_bias,
                                         w1=ws[0], w3=ws[1], w2=ws[2], round_hidden=torch.bfloat16)
        assert rep["ok"], (rank, tag, rep)

    x = gen_local_tokens(1, T, D, torch.bfloat16, dev, 5, rank, "normal")
    bias = torch.zeros(E, device=dev)
    bias[:e_local] = 30.0                                   # all-to-one: only rank 0's experts are ever chosen
    layer.router_bias = bias
    check(x, "all-to-one")
    rows = torch.stack(_gather(layer.group_rows.sum().reshape(1))).reshape(-1).tolist()
    assert rows[0] == world * T * topk and sum(rows[1:]) == 0, rows
    layer.router_bias = None
    check(x if rank != world - 1 else x[:0], "a rank without tokens")
    check(x, "all ranks again")
    layer.check_canaries()
    # a capacity that is too small on every rank: the checked forward grows it collectively
    tight = MoELayer(MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=E, topk=topk, world_size=world,
                               wait_budget_ms=200.0),
                     max_tokens=T, heap=heap, router_std=None, cap_rows=128)
    y = tight.forward_checked(x)
    assert tight.cap_rows > 128
    ws2 = [torch.cat(_gather(w)) for w in tight.reference_weights()]
    rep = cpu_ref.compare_with_dense(y, x, tight.router, topk, tight.last_routing[0], w1=ws2[0], w3=ws2[1],
                                     w2=ws2[2], round_hidden=torch.bfloat16)
    assert rep["ok"], (rank, "after growth", rep)
    tight.check_status()


def test_random_layers(heap, cases: int, seed: int) -> None:
    """Seeded sweep of layer shapes across the ranks (every rank draws the same shapes; token counts
    differ per rank, some ranks get none): ``forward_checked`` against the dense oracle over the
    gathered weights, then the layer's buffers go back to the shared heap."""
    import random
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer
    from iris_testing_b200.ops import cpu_ref
    from iris_testing_b200.utils import gen_local_tokens, zipf_expert_bias
    world, rank, dev = heap.world, heap.rank, heap.device
    rng = random.Random(seed)
    used0 = heap.bytes_in_use
    for case in range(cases):
        gated = rng.random() < 0.6
        D = rng.choice([8, 72, 128, 256, 520, 1024])
        F = rng.choice([128, 256, 384, 1408]) if gated else rng.choice([0, 8, 200, 256])
        e_local = rng.choice([1, 2, 3, 8, 16])
        E = e_local * world
        k = rng.randint(1, min(E, 8))
        T = rng.choice([1, 17, 64, 128, 129, 257, 1000])
        t_rank = [rng.choice([T, T, T // 2, 0]) for _ in range(world)]
        cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=E, topk=k, world_size=world, gated=gated,
                        cta_pair=rng.choice([None, True, False]), capacity_factor=rng.choice([None, 1.25]))
        layer = MoELayer(cfg, max_tokens=T, heap=heap, router_std=None, debug_canaries=True)
        layer.small_path = rng.random() < 0.7
        if rng.random() < 0.3:
            layer.router_bias = zipf_expert_bias(E, 1.2, scale=3.0, device=dev)
        w1, w3, w2 = layer.reference_weights()
        if gated:
            ws = dict(w1=torch.cat(_gather(w1)), w3=torch.cat(_gather(w3)), w2=torch.cat(_gather(w2)),
                      round_hidden=torch.bfloat16)
        else:
            ws = dict(w_single=torch.cat(_gather(w1)))
        for i in range(2):
            x = gen_local_tokens(1, T, D, torch.bfloat16, dev, i, rank, "normal")[: t_rank[rank]]
            y = layer.forward_checked(x)
            if x.shape[0]:
                ref = cpu_ref.dense_moe_ref(x, layer.router, k, bias=layer.router_bias, **ws)
                clear = cpu_ref.clear_routing_mask(x, layer.router, k, layer.router_bias)
                scale = float(ref.abs().max()) or 1.0
                err = float((y.float() - ref)[clear].abs().max()) if bool(clear.any()) else 0.0
                assert err <= 1e-2 * scale, (rank, case, (D, F, E, k, T, t_rank, gated), err, scale)
        layer.check_status()
        layer.check_canaries()
        layer.close()
        assert heap.bytes_in_use == used0, (rank, case)


def _worker(rank: int, world: int) -> None:
    from iris_testing_b200.parallel.symm import SymmetricHeap
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    say = (lambda *a: print(*a, flush=True)) if rank == 0 else (lambda *a: None)
    test_heap_backends(world, rank, dev)
    say("test_heap_backends(vmm, ipc) PASSED")
    size = int(os.getenv("SYMM_HEAP_SIZE", os.getenv("IRIS_HEAP_SIZE", str(1 << 30))))
    heap = SymmetricHeap(size, max_bytes=4 * size)
    say(f"heap back-end: {heap.backend}; capabilities: {heap.capabilities}")
    test_custom_a2a(heap, e_local=2, hidden_dim=128, cap=32)
    say("test_custom_a2a(e_local=2, H=128, cap=32) PASSED")
    test_custom_a2a(heap, e_local=4, hidden_dim=256, cap=16)
    say("test_custom_a2a(e_local=4, H=256, cap=16) PASSED")
    for mode in ("stores", "bulk"):
        test_padded_engine(heap, e_local=4, H=512, T=600, topk=2, copy_mode=mode)
        say(f"test_padded_engine({mode}) PASSED")
    for e_local, H, T, topk, mode in ((1, 8, 1, 1, "stores"), (3, 72, 33, 2, "bulk"), (5, 520, 257, 3, "stores"),
                                      (8, 1024, 2000, 4, "bulk"), (2, 4096, 64, 2, "stores")):
        test_padded_engine(heap, e_local=e_local, H=H, T=T, topk=topk, copy_mode=mode)
    say("test_padded_engine(odd shapes: one token, 16-byte rows, five experts per rank, empty ranks) PASSED")
    test_fused_layer(heap, D=256, F=512, e_local=2, topk=2, T=300)
    say("test_fused_layer(gated) PASSED")
    test_fused_layer(heap, D=256, F=0, e_local=4, topk=1, T=77)
    say("test_fused_layer(single Linear, one kernel) PASSED")
    test_fused_layer(heap, D=1024, F=768, e_local=8, topk=4, T=1500)
    say("test_fused_layer(many experts) PASSED")
    test_skewed_layers(heap, D=256, F=256, e_local=2, topk=2, T=256)
    say("test_skewed_layers(all-to-one, empty rank, capacity growth) PASSED")
    cases = int(os.getenv("RANDOM_LAYER_CASES", "24"))
    test_random_layers(heap, cases=cases, seed=int(os.getenv("RANDOM_LAYER_SEED", "7")))
    say(f"test_random_layers({cases} shapes, uneven token counts) PASSED")
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
