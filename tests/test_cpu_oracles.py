"""CPU tests of the PyTorch restatements and host helpers (no GPU, no process group)."""
import pytest
import torch

from iris_testing_b200.config import MoEConfig, preset
from iris_testing_b200.models import MoELayer
from iris_testing_b200.ops import cpu_ref, custom_a2a, expert, make_plan, router_topk, shuffle, unshuffle
from iris_testing_b200.ops.combine import padded_return, weighted_gather
from iris_testing_b200.utils import (LocalHeap, alloc_return_buffers, alloc_shmem_buffers,
                                     build_dst_offsets, build_expert_offsets, expected_tiles,
                                     gen_local_tokens, gen_local_weights, gen_router, masked_stats,
                                     route_and_pack, route_and_pack_padding_free, set_seed,
                                     spin_wait_counts_ready, spin_wait_token_sync, WaitTimeout,
                                     zipf_expert_bias)


def slow_pack(tokens, router, topk, world, E):
    """Literal restatement of the reference's bucket loop semantics (utils.py:204-246)."""
    e_local = E // world
    probs = torch.softmax(tokens.float() @ router.float(), dim=-1)
    idx = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :topk]
    buckets = [[[] for _ in range(e_local)] for _ in range(world)]
    for t in range(tokens.shape[0]):
        for s in range(topk):
            ex = int(idx[t, s])
            buckets[ex // e_local][ex % e_local].append(tokens[t])
    counts = torch.tensor([[len(b) for b in row] for row in buckets], dtype=torch.int32)
    rows = [r for row in buckets for b in row for r in b]
    return torch.stack(rows), counts


def test_generators_are_deterministic_and_rank_dependent():
    a = gen_local_tokens(2, 8, 16, torch.float32, "cpu", 42, 0)
    b = gen_local_tokens(2, 8, 16, torch.float32, "cpu", 42, 0)
    c = gen_local_tokens(2, 8, 16, torch.float32, "cpu", 42, 1)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert a.min() >= 0 and a.max() < 1          # uniform like the reference
    r0 = gen_router(16, 8, torch.float32, "cpu", 42)
    r1 = gen_router(16, 8, torch.float32, "cpu", 42)
    assert torch.equal(r0, r1) and r0.abs().max() < 0.01
    w0 = gen_local_weights(2, 16, 32, torch.float32, "cpu", 42, 0)
    w1 = gen_local_weights(2, 16, 32, torch.float32, "cpu", 42, 1)
    assert w0.shape == (2, 16, 32) and not torch.equal(w0, w1)
    set_seed(3, 1)
    x = torch.rand(3)
    set_seed(3, 1)
    assert torch.equal(x, torch.rand(3))
    z = zipf_expert_bias(8, 1.2)
    assert z.shape == (8,) and abs(float(z.mean())) < 1e-5 and len(set(z.tolist())) == 8


def test_config_rules_and_env(monkeypatch):
    with pytest.raises(ValueError):
        MoEConfig(hidden_dim=8, ffn_dim=8, num_experts=6, topk=2, world_size=4)
    monkeypatch.setenv("HIDDEN", "256")
    monkeypatch.setenv("E_LOCAL", "2")
    monkeypatch.setenv("TOPK", "3")
    cfg = MoEConfig.from_env(world_size=4)
    assert (cfg.hidden_dim, cfg.num_experts, cfg.topk, cfg.e_local, cfg.gated) == (256, 8, 3, 2, False)
    assert preset("mixtral-8x7b", 8).e_local == 1


@pytest.mark.parametrize("world,E,topk", [(1, 8, 2), (2, 8, 2), (4, 8, 3), (2, 6, 1)])
def test_route_and_pack_matches_bucket_loop(world, E, topk):
    x = gen_local_tokens(2, 24, 32, torch.float32, "cpu", 0, 0, "normal")
    router = gen_router(32, E, torch.float32, "cpu", 0, std=None)
    payload, counts, dst_off, dst_sizes = route_and_pack_padding_free(x, router, topk, world, E)
    ref_payload, ref_counts = slow_pack(x, router, topk, world, E)
    assert torch.equal(counts, ref_counts) and torch.equal(payload, ref_payload)
    assert torch.equal(dst_sizes, ref_counts.sum(1).to(torch.int32))
    assert torch.equal(dst_off, build_dst_offsets(ref_counts))
    offs = build_expert_offsets(ref_counts)
    assert offs.dtype == torch.int32 and torch.equal(offs[:, 0], torch.zeros(world, dtype=torch.int32))


def test_plan_is_a_stable_permutation():
    idx = torch.randint(0, 5, (50, 3), dtype=torch.int32)
    p = make_plan(idx, 5)
    flat = idx.reshape(-1)
    assert int(p.counts.sum()) == flat.numel()
    assert torch.equal(torch.sort(p.send_order).values, torch.arange(flat.numel(), dtype=torch.int32))
    # inside each bucket the flat (token, slot) index increases
    for e in range(5):
        seg = p.send_order[p.bucket_start[e]:p.bucket_start[e + 1]]
        assert bool((flat[seg.long()] == e).all()) and bool((seg[1:] > seg[:-1]).all())
    assert torch.equal(p.send_order[p.dst_slot.long()], torch.arange(flat.numel(), dtype=torch.int32))


def test_router_tie_break_and_renorm():
    x = torch.zeros(3, 4)
    w = torch.zeros(4, 6)
    idx, wgt = router_topk(x, w, 2)
    assert idx.tolist() == [[0, 1]] * 3 and torch.allclose(wgt, torch.full((3, 2), 1 / 6))
    _, wn = router_topk(x, w, 2, renormalize=True)
    assert torch.allclose(wn.sum(-1), torch.ones(3))


def test_shuffle_roundtrip_and_masked_stats():
    pca = torch.tensor([[3, 0], [1, 4]], dtype=torch.int32)
    buf = torch.zeros(2, 2, 4, 8)
    for e in range(2):
        for s in range(2):
            buf[e, s, :pca[e, s]] = torch.randn(int(pca[e, s]), 8)
    packed, rows = shuffle(buf, pca)
    assert packed.shape == (8, 8) and rows.tolist() == [3, 5]
    assert torch.equal(packed[:3], buf[0, 0, :3]) and torch.equal(packed[4:], buf[1, 1, :4])
    assert torch.equal(unshuffle(packed, pca, 4), buf)
    noisy = buf.clone()
    noisy[0, 1] = 7.0                      # padding only
    mx, sa, sb = masked_stats(buf, noisy, pca)
    assert float(mx) == 0.0 and float(sa) == pytest.approx(float(sb))


def test_custom_a2a_single_rank_contract():
    """World of one: the op must fill token_buf[e, 0, m] / pca / flags exactly (unit_tests.py:126-220)."""
    e_local, H, cap = 2, 16, 8
    heap = LocalHeap()
    bufs = alloc_shmem_buffers(heap, 1, e_local, cap, H, torch.float32)
    counts = torch.tensor([[5, 8]], dtype=torch.int32)
    payload = torch.arange(13 * H, dtype=torch.float32).view(13, H)
    out = custom_a2a(payload, counts, build_dst_offsets(counts), bufs.pca, bufs.token_buf,
                     bufs.counts_ready, bufs.token_sync, bufs.heap_bases, e_local, cap)
    assert out.data_ptr() == bufs.token_buf.data_ptr()
    assert bufs.pca.tolist() == [[5], [8]]
    assert torch.equal(out[0, 0, :5], payload[:5]) and torch.equal(out[1, 0, :8], payload[5:])
    assert float(out[0, 0, 5:].abs().sum()) == 0.0
    spin_wait_counts_ready(bufs.counts_ready, 1, timeout_s=1)
    spin_wait_token_sync(bufs.token_sync, expected_tiles(bufs.pca, 32), timeout_s=1)
    with pytest.raises(WaitTimeout):
        spin_wait_token_sync(bufs.token_sync, [99, 99], timeout_s=0.05)


def test_unfused_pipeline_equals_dense_reference_single_rank():
    """router -> pack -> dispatch -> shuffle -> expert -> unshuffle -> return -> weighted sum."""
    D, E, k, T = 32, 4, 2, 40
    x = gen_local_tokens(1, T, D, torch.float32, "cpu", 1, 0, "normal")
    router = gen_router(D, E, torch.float32, "cpu", 1, std=None)
    w = gen_local_weights(E, D, D, torch.float32, "cpu", 1, 0, std=0.1)
    payload, counts, dst_off, _, idx, wgt, plan = route_and_pack(x, router, k, 1, E)
    cap = int(counts.max())
    heap = LocalHeap()
    b = alloc_shmem_buffers(heap, 1, E, cap, D, torch.float32)
    custom_a2a(payload, counts, dst_off, b.pca, b.token_buf, b.counts_ready, b.token_sync,
               b.heap_bases, E, cap)
    packed, rows = shuffle(b.token_buf, b.pca)
    out = expert(packed, w, rows)
    out_buf = unshuffle(out, b.pca, cap)
    r = alloc_return_buffers(heap, 1, E, cap, D, torch.float32)
    padded_return(out_buf, b.pca, r.ret_buf, r.ret_sync, b.heap_bases)
    y = weighted_gather(r.ret_buf, plan, idx, wgt, None, 1, cap)
    ref = cpu_ref.dense_moe_ref(x, router, k, w_single=w)
    assert torch.allclose(y, ref, atol=1e-5)


def test_moe_layer_cpu_matches_dense_reference_and_state_dict():
    cfg = MoEConfig(hidden_dim=128, ffn_dim=256, num_experts=8, topk=2, dtype=torch.float32)
    layer = MoELayer(cfg, max_tokens=128, router_std=None)
    x = gen_local_tokens(2, 64, 128, torch.float32, "cpu", 0, 0, "normal")
    w1, w3, w2 = layer.reference_weights()
    ref = cpu_ref.dense_moe_ref(x, layer.router, 2, w1=w1, w3=w3, w2=w2)
    assert torch.allclose(layer(x), ref, atol=1e-5)
    other = MoELayer(cfg, max_tokens=128, seed=5, router_std=None)
    assert not torch.allclose(other(x), ref, atol=1e-5)
    other.load_state_dict(layer.state_dict())       # checkpoint / resume comes with nn.Module
    assert torch.allclose(other(x), ref, atol=1e-5)
    # reference-layout round trip
    third = MoELayer(cfg, max_tokens=128, seed=9, router_std=None)
    third.load_reference_weights(w1, w3, w2)
    assert torch.equal(third.w13, layer.w13) and torch.equal(third.w2, layer.w2)


def test_interleave_gate_up_layout():
    w1 = torch.arange(2 * 4 * 256, dtype=torch.float32).view(2, 4, 256)
    w3 = -w1
    w13 = cpu_ref.interleave_gate_up(w1, w3)
    assert w13.shape == (2, 512, 4)
    assert torch.equal(w13[:, :128], w1.transpose(1, 2)[:, :128])
    assert torch.equal(w13[:, 128:256], w3.transpose(1, 2)[:, :128])
    assert torch.equal(w13[:, 256:384], w1.transpose(1, 2)[:, 128:])


def test_capacity_and_heap_sizing():
    from iris_testing_b200.models import default_cap_rows, heap_bytes_needed
    import dataclasses
    tight = preset("mixtral-8x7b", world_size=8)                 # default: 1.25 x the balanced load
    assert tight.capacity_factor == 1.25
    cfg = dataclasses.replace(tight, capacity_factor=None)
    worst = default_cap_rows(cfg, 16384)
    assert worst == 8 * 16384 * 2 and worst % 128 == 0          # every token of every rank
    assert default_cap_rows(tight, 16384) < worst
    assert int(1.25 * 16384 * 2) <= default_cap_rows(tight, 16384) <= int(1.26 * 16384 * 2)
    assert default_cap_rows(preset("mixtral-8x7b", world_size=1), 16384) == 16384 * 2   # one rank: worst = balanced
    need = heap_bytes_needed(cfg, 16384)
    assert need > 2 * worst * 4096 * 2                           # two parity copies of the receive buffer
    assert heap_bytes_needed(cfg, 16384, cap_rows=1024) < need


def test_router_weight_cache_follows_the_tensor_not_its_address():
    from iris_testing_b200.ops.router import router_kmajor
    w = torch.randn(16, 4)
    t = router_kmajor(w)
    assert router_kmajor(w) is t and torch.equal(t, w.t())
    w.mul_(2.0)                                   # in-place update: version changes
    assert torch.equal(router_kmajor(w), w.t())
    ptr = w.data_ptr()
    del w, t
    w2 = torch.randn(16, 4)                       # may reuse the freed block
    assert torch.equal(router_kmajor(w2), w2.t()), (ptr, w2.data_ptr())


def test_reference_module_names_are_importable():
    from iris_testing_b200.compat.baseline import (BaselineBuffers, init_baseline_buffers,
                                                   reorder_flat_to_token_buf, run_baseline_ref)
    from iris_testing_b200.compat.layers.all_to_all import custom_a2a as a2a
    from iris_testing_b200.compat.layers.expert import expert as ex
    from iris_testing_b200.compat.layers.token_shuffle import shuffle as sh
    from iris_testing_b200.compat.utils import gen_local_tokens as glt, route_and_pack_padding_free as rp
    assert all(callable(f) for f in (a2a, ex, sh, glt, rp, run_baseline_ref, reorder_flat_to_token_buf))
    # single-process run of the baseline runner with the reference's argument list
    x = glt(1, 16, 8, torch.float32, "cpu", 0, 0)
    router = gen_router(8, 4, torch.float32, "cpu", 0, std=None)
    payload, counts, _, _ = rp(x, router, 2, 1, 4)
    bufs = init_baseline_buffers(1, 4, 32, 8, torch.float32, "cpu", int(counts.sum()), allocate_token_buf=True)
    assert isinstance(bufs, BaselineBuffers)
    tb, timings, meta = run_baseline_ref(0, 1, 4, 32, 8, payload, counts, bufs, do_reorder=True, barrier=False)
    assert tb.shape == (4, 1, 32, 8) and set(timings) == {"step1_ms", "step2_ms", "reorder_ms"}
    assert meta["total_send"] == meta["total_recv"] == int(counts.sum())
    assert torch.equal(tb[0, 0, :int(counts[0, 0])], payload[:int(counts[0, 0])])


def test_zero_padding_clears_stale_rows_only():
    from iris_testing_b200.ops import zero_padding
    buf = torch.ones(2, 3, 4, 5)
    pca = torch.tensor([[0, 4, 2], [1, 3, 0]], dtype=torch.int32)
    zero_padding(buf, pca)
    for e in range(2):
        for s_ in range(3):
            n = int(pca[e, s_])
            assert bool((buf[e, s_, :n] == 1).all()) and bool((buf[e, s_, n:] == 0).all())


def test_small_token_path_rule():
    """Which batches take the one-launch router + plan: at most 4096 routed copies and at most 16
    load trips per router warp (decided on the host from the shape alone)."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer

    def layer(D, E, k):
        # tiny weights: the rule only reads the configuration
        return MoELayer(MoEConfig(hidden_dim=D, ffn_dim=128, num_experts=E, topk=k), max_tokens=8, router_std=None)

    mixtral = layer(4096, 8, 2)
    assert [mixtral.uses_small_path(T) for T in (0, 1, 64, 2048, 2049, 16384)] == [True, True, True, True, False, False]
    assert mixtral.launches_for(64) == 4 and mixtral.launches_for(16384) == 6
    fine = layer(2048, 64, 8)
    assert not fine.uses_small_path(512) and not fine.uses_small_path(513)     # 8 expert groups x 4 row pieces
    assert layer(256, 64, 8).uses_small_path(512)
    tiny = layer(256, 8, 2)
    assert tiny.uses_small_path(64) and tiny.uses_small_path(2048) and not tiny.uses_small_path(2049)
    mixtral.small_path = False
    assert not mixtral.uses_small_path(64) and mixtral.launches_for(64) == 6
