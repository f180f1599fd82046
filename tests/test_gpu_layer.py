"""GPU tests of the fused MoE layer (single GPU: every "peer" is the local GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


TOL = 1e-2      # of max |reference|, over the tokens whose top-k choice is not a near tie


def _make(cfg, T, **kw):
    """A layer with guard blocks around its symmetric buffers (checked by ``_finish``)."""
    from iris_testing_b200.models import MoELayer, heap_bytes_needed
    from iris_testing_b200.parallel.symm import SymmetricHeap
    torch.cuda.set_device(0)
    heap = SymmetricHeap(heap_bytes_needed(cfg, T, kw.get("cap_rows")) + (16 << 20),
                         wait_budget_ms=kw.pop("budget", 2000.0))
    return MoELayer(cfg, max_tokens=T, heap=heap, router_std=None, debug_canaries=True, **kw), heap


def _finish(layer):
    """End of a layer test: no error status and untouched guard blocks."""
    layer.check_status()
    layer.check_canaries()


def _dense(layer, x):
    from iris_testing_b200.ops import cpu_ref
    cfg = layer.cfg
    w1, w3, w2 = layer.reference_weights()
    if cfg.gated:
        return cpu_ref.dense_moe_ref(x, layer.router, cfg.topk, w1=w1, w3=w3, w2=w2,
                                     bias=layer.router_bias, round_hidden=torch.bfloat16)
    return cpu_ref.dense_moe_ref(x, layer.router, cfg.topk, w_single=w1, bias=layer.router_bias)


def _close(layer, x, y, ref=None):
    """y against the dense oracle within TOL on every token with a clear top-k choice."""
    from iris_testing_b200.ops import cpu_ref
    ref = _dense(layer, x) if ref is None else ref
    clear = cpu_ref.clear_routing_mask(x, layer.router, layer.cfg.topk, layer.router_bias)
    assert clear.float().mean() > 0.95
    scale = float(ref.abs().max())
    err = float((y.float() - ref[: y.shape[0]])[clear[: y.shape[0]]].abs().max()) if bool(clear.any()) else 0.0
    assert err <= TOL * scale, (err, scale)
    return ref


@pytest.mark.parametrize("small", [True, False])
@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("D,F,E,k,gated,T", [
    (256, 512, 8, 2, True, 200), (256, 0, 4, 1, False, 77), (2048, 1408, 32, 4, True, 2048),
    (512, 256, 64, 8, True, 1000), (128, 0, 8, 2, False, 128), (1024, 1024, 2, 2, True, 3000),
    (128, 128, 128, 2, True, 700), (72, 128, 8, 3, True, 333), (200, 0, 16, 4, False, 129)])
def test_fused_layer_matches_dense_reference(D, F, E, k, gated, T, pair, small):
    """``small``: small batches may take the single-launch route+plan kernel; with it off every
    shape goes through the tensor-core router and the two plan kernels."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens
    cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=E, topk=k, gated=gated, cta_pair=pair)
    layer, heap = _make(cfg, T)
    layer.small_path = small
    if small and not layer.uses_small_path(T // 2):
        pytest.skip("this shape never takes the small-token path")
    dev = heap.device
    for i in range(3):                                  # exercises both parity slots and re-arming
        x = gen_local_tokens(1, T, D, torch.bfloat16, dev, i, 0, "normal")
        y = layer(x)
        ref = _close(layer, x, y)
    layer.check_status()
    y_short = layer(x[: T // 2])                        # fewer tokens than max_tokens
    _close(layer, x[: T // 2], y_short, ref)
    layer.check_status()
    y_none = layer(x[:0])                               # a rank with no tokens still takes part
    assert y_none.shape == (0, cfg.out_dim)
    y_again = layer(x[: T // 2])
    assert torch.equal(y_again, y_short)                # deterministic, and state survived the empty step
    _finish(layer)


def test_fused_layer_skewed_routing_and_empty_experts():
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens, zipf_expert_bias
    cfg = MoEConfig(hidden_dim=256, ffn_dim=256, num_experts=16, topk=2)
    layer, heap = _make(cfg, 600)
    layer.router_bias = zipf_expert_bias(16, 1.2, scale=4.0, device=heap.device)
    x = gen_local_tokens(1, 600, 256, torch.bfloat16, heap.device, 3, 0, "normal")
    y = layer(x)
    rows = layer.group_rows.cpu()
    assert int(rows.sum()) == 1200 and int(rows.max()) > 4 * max(int(rows.min()), 1)
    _close(layer, x, y)
    _finish(layer)


def test_capacity_overflow_is_reported_not_written():
    """1024 routed rows against a capacity of 256: the step reports how many rows it needed,
    writes nothing outside its buffers (guard blocks, the other parity's counters, the count
    tables and the iteration table stay as they were) and the layer works again afterwards."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens
    cfg = MoEConfig(hidden_dim=128, ffn_dim=128, num_experts=4, topk=2)
    layer, heap = _make(cfg, 512, cap_rows=256, budget=100.0)
    x = gen_local_tokens(1, 512, 128, torch.bfloat16, heap.device, 0, 0, "normal")
    torch.cuda.synchronize()
    ready_other = layer.ready[1].clone()
    flags_other = layer.counts_flag[1].clone()
    layer(x)                                                           # iteration 0 uses parity 0
    torch.cuda.synchronize()
    with pytest.raises(Exception, match=r"overflow.*rows needed on this rank: 1024"):
        layer.check_status()
    assert torch.equal(layer.ready[1], ready_other) and torch.equal(layer.counts_flag[1], flags_other)
    assert int(layer.ready[0].abs().sum()) == 0 and int(layer.arrived[0]) == 0      # re-armed by the retire
    assert layer.iter_done.tolist() == [1] and int(layer.iter_dev[0]) == 1
    layer.check_canaries()
    # the status was reset by check_status(): a step that fits runs and is correct
    y = layer(x[:100])
    _close(layer, x[:100], y)
    y = layer(x[:120])
    _close(layer, x[:120], y)
    _finish(layer)


def test_forward_checked_grows_the_buffers_and_repeats_the_step():
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer
    from iris_testing_b200.parallel.symm import SymmetricHeap
    from iris_testing_b200.utils import gen_local_tokens
    torch.cuda.set_device(0)
    cfg = MoEConfig(hidden_dim=128, ffn_dim=256, num_experts=4, topk=2, wait_budget_ms=100.0)
    heap = SymmetricHeap(4 << 20, max_bytes=64 << 20, wait_budget_ms=100.0)
    layer = MoELayer(cfg, max_tokens=512, heap=heap, router_std=None, cap_rows=256, debug_canaries=True)
    x = gen_local_tokens(1, 512, 128, torch.bfloat16, heap.device, 0, 0, "normal")
    y = layer.forward_checked(x)                   # needs 1024 rows: overflow, resize, repeat
    assert layer.cap_rows >= 1024
    _close(layer, x, y)
    y2 = layer(x)                                  # later steps run unchecked at the new capacity
    assert torch.equal(y, y2)
    mem = layer.memory_bytes()
    assert mem["capacity_rows"] == layer.cap_rows and mem["symmetric"] > 2 * layer.cap_rows * 128 * 2
    _finish(layer)


@pytest.mark.parametrize("ctas", [8, 37])
@pytest.mark.parametrize("pair", [False, True])
def test_fused_layer_on_a_forced_small_grid(ctas, pair):
    """The persistent kernels stride all work (sender units, tiles) over the CTAs they were
    given: a grid far smaller than the SM count (and an odd one, where CTA pairs use one CTA
    less) still sends every row and computes every tile."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens
    cfg = MoEConfig(hidden_dim=512, ffn_dim=512, num_experts=8, topk=2, cta_pair=pair)
    layer, heap = _make(cfg, 1500, num_ctas=ctas)
    for i in range(2):
        x = gen_local_tokens(1, 1500, 512, torch.bfloat16, heap.device, i, 0, "normal")
        _close(layer, x, layer(x))
    _finish(layer)


def test_dropped_arrival_signal_times_out_with_status():
    """Host-injected fault: the senders skip the tile-arrival signal.  The consumer's wait
    runs out of budget, the kernels drain and return, and the host reads the status."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens
    cfg = MoEConfig(hidden_dim=128, ffn_dim=128, num_experts=4, topk=2, wait_budget_ms=50.0)
    layer, heap = _make(cfg, 256, budget=50.0)
    x = gen_local_tokens(1, 256, 128, torch.bfloat16, heap.device, 0, 0, "normal")
    layer(x)
    layer.check_status()
    layer.drop_signal = True
    layer(x)
    torch.cuda.synchronize()
    with pytest.raises(Exception, match="never arrived"):
        layer.check_status()
    # the context is still usable
    assert float(torch.ones(4, device=heap.device).sum()) == 4.0


@pytest.mark.parametrize("gated", [True, False])
def test_cuda_graph_replay_matches_eager(gated):
    """The forward pass captured once replays correctly for every later step: the iteration
    number and the buffer parity are read from device memory, not baked into the launches."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens
    cfg = MoEConfig(hidden_dim=256, ffn_dim=512 if gated else 0, num_experts=8, topk=2, gated=gated)
    layer, heap = _make(cfg, 300)
    dev = heap.device
    xs = [gen_local_tokens(1, 300, 256, torch.bfloat16, dev, i, 0, "normal") for i in range(5)]
    refs = [_dense(layer, x) for x in xs]
    y0 = layer(xs[0])                                     # eager step before the capture
    _close(layer, xs[0], y0, refs[0])
    layer.capture(300)
    for i in (1, 2, 3):                                   # odd and even iterations
        y = layer.replay(xs[i]).clone()
        _close(layer, xs[i], y, refs[i])
    y4 = layer(xs[4])                                     # eager again after replays
    _close(layer, xs[4], y4, refs[4])
    _finish(layer)


def test_phase_timing_and_arrival_trace():
    """The profiling hooks: per-phase CUDA-event times and the per-tile arrival trace."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens
    cfg = MoEConfig(hidden_dim=256, ffn_dim=512, num_experts=4, topk=2)
    layer, heap = _make(cfg, 1024)
    layer.small_path = False              # time the router and the plan as separate phases
    x = gen_local_tokens(1, 1024, 256, torch.bfloat16, heap.device, 0, 0, "normal")
    layer(x)
    layer.profile = True
    layer.trace_arrivals = True
    y = layer(x)
    phases = layer.phase_times_us()
    assert list(phases) == ["router", "plan", "dispatch+gemm1", "gemm2+combine", "slot_reduce"]
    assert all(v > 0 for v in phases.values())
    rep = layer.arrival_report()
    assert rep["tiles"] == sum((int(r) + 127) // 128 for r in layer.group_rows.tolist())
    assert 0 <= rep["first_us"] <= rep["last_us"] and rep["own_last_published_us"] >= rep["own_first_published_us"]
    _close(layer, x, y)
    _finish(layer)


def test_small_token_path_routes_and_plans_like_the_regular_kernels():
    """The single-launch route+plan kernel must produce the same routing (indices exactly, weights
    to fp32 rounding) and the same plan as the tensor-core router plus the two plan kernels,
    and one launch fewer... two fewer."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens, zipf_expert_bias
    for D, F, E, k, T, bias in [(256, 512, 8, 2, 64, False), (512, 256, 64, 8, 100, True), (4096, 512, 8, 2, 64, False)]:
        cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=E, topk=k)
        layer, heap = _make(cfg, T)
        if bias:
            layer.router_bias = zipf_expert_bias(E, 1.2, device=heap.device)
        x = gen_local_tokens(1, T, D, torch.bfloat16, heap.device, 4, 0, "normal")
        assert layer.uses_small_path(T) and layer.launches_for(T) == 4
        y_small = layer(x)
        idx_s, w_s = (t.clone() for t in layer.last_routing)
        order_s, slot_s = layer._plan.send_order[: T * k].clone(), layer._plan.dst_slot[: T * k].clone()
        counts_s = layer._plan.counts.clone()
        layer.small_path = False
        assert layer.launches_for(T) == 6
        y_reg = layer(x)
        idx_r, w_r = layer.last_routing
        from iris_testing_b200.ops import cpu_ref
        clear = cpu_ref.clear_routing_mask(x, layer.router, k, layer.router_bias)
        assert torch.equal(idx_s[clear], idx_r[clear]) and torch.allclose(w_s[clear], w_r[clear], atol=1e-6, rtol=2e-4)
        if bool(clear.all()):
            assert torch.equal(order_s, layer._plan.send_order[: T * k]) and torch.equal(slot_s, layer._plan.dst_slot[: T * k])
            assert torch.equal(counts_s, layer._plan.counts)
        _close(layer, x, y_small)
        _close(layer, x, y_reg)
        _finish(layer)


@pytest.mark.parametrize("wide", [(1, 1), (0, 1)])
@pytest.mark.parametrize("D,F,E,k,gated,T", [(512, 1024, 4, 2, True, 2100), (768, 0, 2, 2, False, 1500)])
def test_fused_layer_with_wide_tiles(D, F, E, k, gated, T, wide):
    """The optional 512-column tile geometry in the fused kernels (dispatch + GEMM1 and GEMM2 +
    combine): odd numbers of 256-column blocks, ragged groups, both parities."""
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.utils import gen_local_tokens
    cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=E, topk=k, gated=gated, cta_pair=True)
    layer, heap = _make(cfg, T)
    layer.wide_tiles = wide
    for i in range(3):
        x = gen_local_tokens(1, T, D, torch.bfloat16, heap.device, 10 + i, 0, "normal")
        _close(layer, x, layer(x))
    _finish(layer)


def test_random_layer_shapes_match_dense_reference():
    """Seeded sweep over odd shapes: hidden sizes that are no multiple of a k-block, one to 128
    experts, top-1 to top-8, one token to a few thousand, every tile geometry, with and without
    the small-token path, capacity factor and skewed routing.  Each case: two full steps and a
    shorter one through ``forward_checked`` against the dense oracle, then status and guards."""
    import random
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.ops import cpu_ref
    from iris_testing_b200.utils import gen_local_tokens, zipf_expert_bias
    rng = random.Random(20240607)
    for case in range(120):
        gated = rng.random() < 0.6
        D = rng.choice([8, 64, 72, 128, 200, 256, 520, 1024, 2048])
        F = rng.choice([128, 256, 384, 1408]) if gated else rng.choice([0, 8, 64, 200, 256, 1000])
        E = rng.choice([1, 2, 3, 5, 8, 24, 64, 128])
        k = rng.randint(1, min(E, 8))
        T = rng.choice([1, 2, 17, 64, 127, 128, 129, 255, 257, 1000, 2047])
        cfg = MoEConfig(hidden_dim=D, ffn_dim=F, num_experts=E, topk=k, gated=gated,
                        cta_pair=rng.choice([None, True, False]), capacity_factor=rng.choice([None, 1.25]))
        layer, heap = _make(cfg, T)
        layer.small_path = rng.random() < 0.7
        layer.wide_tiles = rng.choice([(0, 0), (0, 0), (1, 1)])
        if rng.random() < 0.3:
            layer.router_bias = zipf_expert_bias(E, 1.2, scale=3.0, device=heap.device)
        what = (case, D, F, E, k, T, gated, cfg.cta_pair, cfg.capacity_factor, layer.small_path, layer.wide_tiles)
        for i in range(2):
            x = gen_local_tokens(1, T, D, torch.bfloat16, heap.device, i, 0, "normal")
            y = layer.forward_checked(x)
            ref = _dense(layer, x)
            clear = cpu_ref.clear_routing_mask(x, layer.router, k, layer.router_bias)
            scale = float(ref.abs().max()) or 1.0
            err = float((y.float() - ref)[clear].abs().max()) if bool(clear.any()) else 0.0
            assert err <= TOL * scale, (what, err, scale)
        half = max(T // 2, 1)
        y = layer.forward_checked(x[:half])
        err = float((y.float() - ref[:half])[clear[:half]].abs().max()) if bool(clear[:half].any()) else 0.0
        assert err <= TOL * scale, (what, err, scale)
        _finish(layer)
        del layer
        heap.close()


def test_layer_close_returns_its_symmetric_buffers():
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer
    from iris_testing_b200.parallel.symm import SymmetricHeap
    from iris_testing_b200.utils import gen_local_tokens
    torch.cuda.set_device(0)
    heap = SymmetricHeap(64 << 20)
    used0 = heap.bytes_in_use
    first = None
    for D, E in ((256, 8), (512, 4), (256, 8)):
        cfg = MoEConfig(hidden_dim=D, ffn_dim=256, num_experts=E, topk=2)
        layer = MoELayer(cfg, max_tokens=300, heap=heap, router_std=None, debug_canaries=True)
        assert heap.bytes_in_use > used0
        if first is None:
            first = layer.counts_all.data_ptr()
        x = gen_local_tokens(1, 300, D, torch.bfloat16, heap.device, 0, 0, "normal")
        _close(layer, x, layer(x))
        _finish(layer)
        layer.close()
        layer.close()                                     # a second call is a no-op
        assert heap.bytes_in_use == used0
        with pytest.raises(RuntimeError, match="closed"):
            layer(x)
    # the space was reused, not appended
    cfg = MoEConfig(hidden_dim=256, ffn_dim=256, num_experts=8, topk=2)
    layer = MoELayer(cfg, max_tokens=300, heap=heap, router_std=None, debug_canaries=True)
    assert layer.counts_all.data_ptr() == first
    layer.close()
    heap.close()
