"""Multi-process CPU tests over gloo (world_size 2 and 4): the padded fixed-M exchange,
the dispatch/combine contract, the library baseline and host-side failure handling."""
import time

import pytest
import torch

from conftest import run_gloo


def _all_gather(t):
    import torch.distributed as dist
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def _plumbing_worker(rank, world, gated):
    """fp32 tokens [B=2, S=64, D=128], router N(0,1/D) [128, 8], E=8, top-2, seed 0."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer
    from iris_testing_b200.ops import cpu_ref
    from iris_testing_b200.parallel import AllToAllMoEBaseline
    from iris_testing_b200.utils import gen_local_tokens
    D = 128
    cfg = MoEConfig(hidden_dim=D, ffn_dim=256 if gated else 0, num_experts=8, topk=2,
                    world_size=world, gated=gated, dtype=torch.float32)
    layer = MoELayer(cfg, max_tokens=128, seed=0, router_std=None)
    x = gen_local_tokens(2, 64, D, torch.float32, "cpu", 0, rank, "normal")
    y = layer(x)
    w1, w3, w2 = layer.reference_weights()
    if gated:
        W1, W3, W2 = (torch.cat(_all_gather(w)) for w in (w1, w3, w2))
        ref = cpu_ref.dense_moe_ref(x, layer.router, 2, w1=W1, w3=W3, w2=W2)
    else:
        ref = cpu_ref.dense_moe_ref(x, layer.router, 2, w_single=torch.cat(_all_gather(w1)))
    base = AllToAllMoEBaseline(layer).forward(x)
    # M rule: every pair exchanges exactly M rows, M = max over pairs
    idx, _ = layer.last_routing
    plan = cpu_ref.plan_ref(idx, 8)
    pair_rows = torch.stack(_all_gather(plan.counts.view(world, -1).sum(1)))
    return dict(err=float((y - ref).abs().max()), base_err=float((base - ref).abs().max()),
                M=layer.last_message_rows, M_expected=int(pair_rows.max()))


@pytest.mark.parametrize("world,gated", [(2, False), (2, True), (4, False)])
def test_gloo_moe_matches_dense_reference(world, gated):
    for r in run_gloo(_plumbing_worker, world, (gated,)):
        assert r["err"] < 1e-4 and r["base_err"] < 1e-4
        assert r["M"] == r["M_expected"] >= 1


def _dispatch_worker(rank, world):
    """custom_a2a over gloo against the all-ranks restatement, plus the library baseline
    re-laid out into the same [e, src, m, :] buffer (benchmark.py:354-440)."""
    import torch.distributed as dist
    from iris_testing_b200.ops import cpu_ref, custom_a2a, shuffle, unshuffle
    from iris_testing_b200.ops.combine import padded_return, weighted_gather
    from iris_testing_b200.parallel import run_baseline
    from iris_testing_b200.utils import (LocalHeap, alloc_return_buffers, alloc_shmem_buffers,
                                         compute_capacity_from_pca, gen_local_tokens, gen_router,
                                         masked_stats, route_and_pack)
    D, E, k = 64, 4 * world, 2
    e_local = E // world
    x = gen_local_tokens(2, 32, D, torch.float32, "cpu", 42, rank)
    router = gen_router(D, E, torch.float32, "cpu", 42, std=None)
    payload, counts, dst_off, _, idx, wgt, plan = route_and_pack(x, router, k, world, E)
    all_counts = torch.stack(_all_gather(counts))            # [src, dst, e]
    expected_pca = all_counts[:, rank, :].t().contiguous()
    cap = compute_capacity_from_pca(expected_pca)
    heap = LocalHeap()
    b = alloc_shmem_buffers(heap, world, e_local, cap, D, torch.float32)
    custom_a2a(payload, counts, dst_off, b.pca, b.token_buf, b.counts_ready, b.token_sync,
               b.heap_bases, E, cap)
    tb, _, meta = run_baseline(payload, counts, cap, do_reorder=True)
    mx, s1, s2 = masked_stats(b.token_buf, tb, expected_pca)
    # identity experts: the combine must give back sum_k w_k * x
    r = alloc_return_buffers(heap, world, e_local, cap, D, torch.float32)
    padded_return(b.token_buf, b.pca, r.ret_buf, r.ret_sync, b.heap_bases)
    y = weighted_gather(r.ret_buf, plan, idx, wgt, None, world, cap)
    ident = x * wgt.sum(dim=1, keepdim=True)
    packed, rows = shuffle(b.token_buf, b.pca)
    return dict(pca_ok=torch.equal(b.pca, expected_pca), max_diff=float(mx),
                sum_diff=abs(float(s1) - float(s2)), ident_err=float((y - ident).abs().max()),
                round_trip=torch.equal(unshuffle(packed, b.pca, cap), b.token_buf),
                rows_ok=rows.tolist() == expected_pca.sum(1).tolist(),
                padding_zero=float(b.token_buf.abs().sum()) == pytest.approx(float(s1), rel=1e-5))


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_dispatch_contract_and_baseline_agreement(world):
    for r in run_gloo(_dispatch_worker, world):
        assert r["pca_ok"] and r["max_diff"] == 0.0 and r["sum_diff"] < 1e-3
        assert r["ident_err"] < 1e-5 and r["round_trip"] and r["rows_ok"] and r["padding_zero"]


def _agreement_worker(rank, world):
    """Rank 1 fails a phase on the host; every rank must learn of it and leave together."""
    from iris_testing_b200.utils import all_ranks_ok, sync_and_check
    ok = True
    try:
        if rank == 1:
            raise RuntimeError("injected host-side failure")
    except RuntimeError:
        ok = False
    first = sync_and_check(ok)
    second = all_ranks_ok(True)
    return first, second


def test_rank_agreement_on_injected_failure():
    assert run_gloo(_agreement_worker, 2) == [(False, True), (False, True)]


def _late_rank_worker(rank, world):
    """A rank that joins the exchange late: peers block in the collective, nobody hangs,
    and a short process-group timeout would surface a rank that never joins."""
    import torch.distributed as dist
    from iris_testing_b200.parallel import exchange_counts
    if rank == 1:
        time.sleep(0.5)
    t0 = time.time()
    c = exchange_counts(torch.full((world, 2), rank + 1, dtype=torch.int32))
    return c[:, 0].tolist(), time.time() - t0


def test_late_rank_is_waited_for():
    res = run_gloo(_late_rank_worker, 2)
    assert res[0][0] == [1, 2] and res[1][0] == [1, 2]
    assert res[0][1] >= 0.3           # rank 0 really waited for rank 1


def _never_joins_worker(rank, world):
    """Rank 1 never enters the collective: rank 0's next collective must end with an error
    after the (short) process-group timeout instead of hanging."""
    import datetime
    import torch.distributed as dist
    pg = dist.new_group(ranks=list(range(world)), timeout=datetime.timedelta(seconds=2), backend="gloo")
    if rank == 1:
        time.sleep(4.0)
        return "skipped"
    try:
        t = torch.ones(1)
        dist.all_reduce(t, group=pg)
        return "completed"
    except Exception as exc:          # gloo reports the timeout as a RuntimeError
        return "error:" + type(exc).__name__


def test_missing_rank_ends_collective_with_error():
    res = run_gloo(_never_joins_worker, 2)
    assert res[1] == "skipped" and res[0].startswith("error:")
