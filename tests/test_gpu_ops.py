"""GPU tests of the individual sm_100a kernels against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    torch.cuda.set_device(0)
    return torch.device("cuda", 0)


@pytest.fixture(scope="module")
def heap(dev):
    from iris_testing_b200.parallel.symm import SymmetricHeap
    return SymmetricHeap(512 << 20)


def test_native_library_is_loaded():
    from iris_testing_b200 import _native
    lib = _native.lib()
    assert lib.b200_gemm_smem_bytes() <= 232448
    maps = open("/proc/self/maps").read()
    assert "libb200moe.so" in maps


@pytest.mark.parametrize("simple", [False, True])
@pytest.mark.parametrize("T,D,E,k,bias", [(64, 128, 8, 2, False), (1000, 256, 64, 8, False),
                                          (333, 512, 128, 4, True), (5, 64, 3, 1, False),
                                          (4096, 2048, 256, 8, True)])
def test_router_topk(dev, T, D, E, k, bias, simple):
    from iris_testing_b200.ops import cpu_ref, router_topk
    from iris_testing_b200.utils import gen_local_tokens, gen_router, zipf_expert_bias
    x = gen_local_tokens(1, T, D, torch.bfloat16, dev, 0, 0, "normal")
    wr = gen_router(D, E, torch.bfloat16, dev, 0, std=None)
    b = zipf_expert_bias(E, device=dev) if bias else None
    ref_lg = x.float() @ wr.float() + (b if bias else 0)
    if simple:
        idx, w, lg = router_topk(x, wr, k, bias=b, return_logits=True)
        assert torch.allclose(lg, ref_lg, atol=1e-4, rtol=1e-4)
    else:                                   # tensor-core path (softmax + top-k in the epilogue)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        idx, w = router_topk(x, wr, k, bias=b, status=status)
        assert status[0].item() == 0
    ridx, rw = cpu_ref.router_topk_ref(x, wr, k, bias=b)
    # near-ties may legitimately swap: compare where the reference's k-th gap is clear
    probs = torch.softmax(ref_lg, -1)
    srt = torch.sort(probs, -1, descending=True).values
    clear = (srt[:, :k] - srt[:, 1:k + 1]).min(dim=1).values > 1e-6 if E > k else torch.ones(T, dtype=torch.bool, device=dev)
    assert clear.float().mean() > 0.95
    assert torch.equal(idx[clear], ridx[clear])
    assert torch.allclose(w[clear], rw[clear], atol=1e-6, rtol=2e-4)
    _, wn = router_topk(x, wr, k, bias=b, renormalize=True, force_simple=simple)
    assert torch.allclose(wn.sum(-1), torch.ones(T, device=dev), atol=1e-5)


@pytest.mark.parametrize("T,k,E", [(64, 2, 8), (4096, 8, 128), (1, 1, 4), (1000, 4, 64)])
def test_plan_and_pack(dev, T, k, E):
    from iris_testing_b200.ops import cpu_ref, make_plan, pack_rows
    g = torch.Generator(device="cpu").manual_seed(T + k)
    idx = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32).to(dev)
    if T > 100:
        idx[idx == 3] = 0                      # an empty expert and a hot one
    p = make_plan(idx, E)
    r = cpu_ref.plan_ref(idx, E)
    for name in ("counts", "bucket_start", "send_order", "dst_slot", "rank_in_bucket"):
        assert torch.equal(getattr(p, name), getattr(r, name)), name
    x = torch.randn(T, 64, device=dev).to(torch.bfloat16)
    assert torch.equal(pack_rows(x, p.send_order, k), cpu_ref.pack_ref(x, r.send_order, k))


def _gemm_case(dev, rows_list, N, K, gated, pair=False, wide=0):
    from iris_testing_b200 import _native as nv
    from iris_testing_b200.ops import grouped_gemm
    G, M = len(rows_list), max(sum(rows_list), 1)
    g = torch.Generator(device="cpu").manual_seed(N + K)
    a = torch.randn(M, K, generator=g).to(dev, torch.bfloat16)
    w = (torch.randn(G, N, K, generator=g) * 0.05).to(dev, torch.bfloat16)
    rows = torch.tensor(rows_list, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = grouped_gemm(a, w, rows, epilogue=nv.EPI_SILU_GATE if gated else nv.EPI_STORE, status=status,
                       cta_pair=pair, wide_tiles=wide)
    ref = torch.zeros(M, N, device=dev)
    off = 0
    for gi, r in enumerate(rows_list):
        ref[off:off + r] = a[off:off + r].float() @ w[gi].float().t()
        off += r
    if gated:
        v = ref.view(M, N // 256, 2, 128)
        ref = (torch.nn.functional.silu(v[:, :, 0]) * v[:, :, 1]).reshape(M, N // 2)
    n = sum(rows_list)
    assert status[0].item() == 0
    assert torch.allclose(out[:n].float(), ref[:n], atol=2e-2 * float(ref.abs().max()) + 1e-3, rtol=2e-2)


@pytest.mark.parametrize("rows,N,K", [([128], 256, 64), ([100], 256, 512), ([300, 0, 77, 129], 512, 512),
                                      ([37] * 16, 2048, 1408), ([5, 200], 136, 72), ([0, 0, 1], 256, 128),
                                      ([4096], 1024, 4096)])
@pytest.mark.parametrize("pair", [False, True])
def test_grouped_gemm_plain(dev, rows, N, K, pair):
    _gemm_case(dev, rows, N, K, gated=False, pair=pair)


@pytest.mark.parametrize("rows,N,K", [([300, 0, 77, 129], 512, 512), ([1000, 513], 2816, 2048)])
@pytest.mark.parametrize("pair", [False, True])
def test_grouped_gemm_silu_gate(dev, rows, N, K, pair):
    _gemm_case(dev, rows, N, K, gated=True, pair=pair)


@pytest.mark.parametrize("rows,N,K,gated", [([300, 0, 77, 129], 512, 512, False), ([4096], 1024, 4096, False),
                                            ([1000, 513], 2816, 2048, True), ([700], 768, 256, False),
                                            ([37] * 16, 2048, 1408, False), ([256, 255, 257], 1280, 64, True),
                                            ([5000], 136, 72, False)])
def test_grouped_gemm_wide_tiles(dev, rows, N, K, gated):
    """512-column tiles (both TMEM accumulators per tile, second half's MMAs trailing the first):
    also with an odd number of 256-column blocks, where the last tile's second half is past N."""
    _gemm_case(dev, rows, N, K, gated=gated, pair=True, wide=1)


def test_expert_op_reference_signature(dev):
    """Oracle of the reference's dead test_gemm (unit_tests.py:224-237): per-expert matmul, tol 1e-2."""
    from iris_testing_b200.ops import expert
    from iris_testing_b200.utils import gen_local_weights
    g = torch.Generator(device="cpu").manual_seed(0)
    cnt = torch.randint(0, 100, (6,), generator=g, dtype=torch.int32)
    S = int(cnt.sum())
    tokens = torch.randn(S, 128, generator=g).to(dev, torch.bfloat16)
    w = gen_local_weights(6, 128, 256, torch.bfloat16, dev, 0, 0)
    out = expert(tokens, w, cnt.to(dev))
    off = 0
    for e, n in enumerate(cnt.tolist()):
        ref = tokens[off:off + n].float() @ w[e].float()
        assert torch.allclose(out[off:off + n].float(), ref, atol=1e-2, rtol=1e-2)
        off += n


def test_silu_gate(dev):
    from iris_testing_b200.ops import silu_gate
    g, u = torch.randn(513, 256, device=dev).bfloat16(), torch.randn(513, 256, device=dev).bfloat16()
    ref = torch.nn.functional.silu(g.float()) * u.float()
    assert torch.allclose(silu_gate(g, u).float(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("e_local,H,cap", [(2, 128, 32), (4, 256, 16)])
def test_custom_a2a_reference_unit_shapes(dev, heap, e_local, H, cap):
    """The reference's two unit-test shapes (unit_tests.py:84-88) on a world of one: full
    routing, value-encodes-coordinates payload, exact equality per (src, e) block."""
    from iris_testing_b200.ops import custom_a2a, shuffle, unshuffle
    from iris_testing_b200.utils import (alloc_shmem_buffers, build_dst_offsets, expected_tiles,
                                         reset_dispatch_flags, spin_wait_counts_ready,
                                         spin_wait_token_sync)
    world = 1
    counts = torch.full((world, e_local), cap, dtype=torch.int32, device=dev)
    t = torch.arange(cap, device=dev).view(1, cap, 1)
    e = torch.arange(e_local, device=dev).view(e_local, 1, 1)
    payload = (e * 100 + t).expand(e_local, cap, H).reshape(-1, H).to(torch.bfloat16).contiguous()
    b = alloc_shmem_buffers(heap, world, e_local, cap, H, torch.bfloat16)
    for _ in range(2):                      # second call after the reference's flag reset
        reset_dispatch_flags(b)
        out = custom_a2a(payload, counts, build_dst_offsets(counts), b.pca, b.token_buf,
                         b.counts_ready, b.token_sync, b.heap_bases, e_local * world, cap)
        spin_wait_counts_ready(b.counts_ready, world, timeout_s=5)
        spin_wait_token_sync(b.token_sync, expected_tiles(b.pca, 32), timeout_s=5)
        assert torch.equal(b.pca, counts.t())
        assert torch.equal(out.view(-1, H), payload)
    packed, rows = shuffle(b.token_buf, b.pca, b.token_sync, b.counts_ready)
    assert rows.tolist() == [cap] * e_local and torch.equal(packed, payload)
    assert torch.equal(unshuffle(packed, b.pca, cap), b.token_buf)
    heap.check_status()


def test_unfused_pipeline_ragged_single_gpu(dev, heap):
    """Router-driven ragged counts through dispatch -> shuffle -> expert -> unshuffle -> return ->
    weighted sum, against the dense reference; padding rows stay zero; overflow is reported."""
    from iris_testing_b200.ops import cpu_ref, custom_a2a, expert, shuffle, unshuffle
    from iris_testing_b200.ops.combine import padded_return, weighted_gather
    from iris_testing_b200.utils import (alloc_return_buffers, alloc_shmem_buffers, gen_local_tokens,
                                         gen_local_weights, gen_router, route_and_pack)
    D, E, k, T = 256, 8, 2, 300
    x = gen_local_tokens(1, T, D, torch.bfloat16, dev, 1, 0, "normal")
    router = gen_router(D, E, torch.bfloat16, dev, 1, std=None)
    w = gen_local_weights(E, D, D, torch.bfloat16, dev, 1, 0, std=0.05)
    payload, counts, dst_off, _, idx, wgt, plan = route_and_pack(x, router, k, 1, E)
    cap = int(counts.max().item())
    guard_lo = heap.zeros((4096,), torch.int32); guard_lo.fill_(0x5A5A5A5A)     # canaries around the
    b = alloc_shmem_buffers(heap, 1, E, cap, D, torch.bfloat16)                   # symmetric buffers
    guard_hi = heap.zeros((4096,), torch.int32); guard_hi.fill_(0x5A5A5A5A)
    custom_a2a(payload, counts, dst_off, b.pca, b.token_buf, b.counts_ready, b.token_sync,
               b.heap_bases, E, cap)
    packed, rows = shuffle(b.token_buf, b.pca, b.token_sync, b.counts_ready)
    n = int(rows.sum().item())
    assert torch.equal(packed[:n], payload)                 # world of one: same order
    valid = torch.arange(cap, device=dev).view(1, 1, cap) < b.pca.unsqueeze(-1)
    assert float(b.token_buf[~valid].abs().sum()) == 0.0     # padding is zero
    out = expert(packed, w, rows)
    out_buf = unshuffle(out, b.pca, cap)
    r = alloc_return_buffers(heap, 1, E, cap, D, torch.bfloat16)
    padded_return(out_buf, b.pca, r.ret_buf, r.ret_sync, b.heap_bases)
    y = weighted_gather(r.ret_buf, plan, idx, wgt, r.ret_sync, 1, cap, status=heap.status)
    ref = cpu_ref.dense_moe_ref(x, router, k, w_single=w)
    assert torch.allclose(y.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
    heap.check_status()
    assert bool((guard_lo == 0x5A5A5A5A).all()) and bool((guard_hi == 0x5A5A5A5A).all())
    # capacity too small: rows beyond CAP are dropped and the status word says so
    small = alloc_shmem_buffers(heap, 1, E, max(cap // 2, 1), D, torch.bfloat16)
    custom_a2a(payload, counts, dst_off, small.pca, small.token_buf, small.counts_ready,
               small.token_sync, small.heap_bases, E, max(cap // 2, 1))
    torch.cuda.synchronize()
    with pytest.raises(Exception, match="overflow"):
        heap.check_status()


def test_heap_barrier_and_bounded_wait(dev, heap):
    heap.barrier()
    heap.barrier()
    # a wait that nothing satisfies must return with a status, not hang
    from iris_testing_b200.ops import shuffle
    pca = torch.full((2, 1), 4, dtype=torch.int32, device=dev)
    buf = torch.zeros(2, 1, 4, 64, dtype=torch.bfloat16, device=dev)
    never = torch.zeros(2, dtype=torch.int32, device=dev)
    ready = torch.ones(1, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    shuffle(buf, pca, never, ready, status=status, wait_budget_ms=50)
    torch.cuda.synchronize()
    assert status[0].item() == 6     # "a dispatched token tile never arrived"


def test_device_row_counts_beyond_the_buffers_are_reported_not_stored(dev):
    """Row counts are read on the device; counts that add up to more rows than a buffer holds
    must end in a status code, never in a store past the buffer."""
    from iris_testing_b200.ops import check_default_status, default_status, grouped_gemm, shuffle
    a = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    w = torch.randn(2, 256, 128, device=dev).to(torch.bfloat16)
    out = torch.zeros(256 + 64, 256, dtype=torch.bfloat16, device=dev)       # 64 guard rows behind the output
    rows = torch.tensor([200, 200], dtype=torch.int32, device=dev)           # 400 > 256
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    grouped_gemm(a, w, rows, out=out[:256], status=status)
    torch.cuda.synchronize()
    assert status.tolist()[:2] == [10, 400] and float(out.abs().sum()) == 0.0
    # same call without a status tensor: the report lands in the device's default status word
    default_status(dev).zero_()
    grouped_gemm(a, w, rows, out=out[:256])
    with pytest.raises(Exception, match=r"overflow.*rows needed: 400"):
        check_default_status(dev)
    check_default_status(dev)                                                # reset by the failed check
    # shuffle into a packed buffer that is too small: the copy stops at max_rows
    pca = torch.tensor([[6], [5]], dtype=torch.int32, device=dev)
    buf = torch.ones(2, 1, 8, 64, dtype=torch.bfloat16, device=dev)
    st2 = torch.zeros(4, dtype=torch.int32, device=dev)
    packed, _ = shuffle(buf, pca, max_rows=8, status=st2)
    torch.cuda.synchronize()
    assert packed.shape[0] == 8 and st2.tolist()[:2] == [10, 11]


@pytest.mark.parametrize("mode", ["stores", "bulk"])
@pytest.mark.parametrize("e_local,H,T,k,combine", [(2, 128, 100, 2, False), (8, 4096, 1024, 2, True),
                                                   (4, 768, 777, 4, True), (1, 264, 50, 1, True)])
def test_padded_all_to_all_engine_repeats_without_memsets(dev, e_local, H, T, k, combine, mode):
    """``PaddedAllToAll`` on a world of one, three exchanges in a row with changing routing: flags
    re-armed in-kernel, valid rows bit-equal to the payload, padding never written, and with
    the return path the weighted sum of the rows that come home."""
    from iris_testing_b200.parallel.padded_a2a import CapacityProbe, PaddedAllToAll
    from iris_testing_b200.parallel.symm import SymmetricHeap
    from iris_testing_b200.utils import gen_local_tokens, gen_router, route_and_pack
    E = e_local
    heap = SymmetricHeap(64 << 20, max_bytes=1 << 30)
    probe = CapacityProbe(heap, e_local)
    router = gen_router(H, E, torch.bfloat16, dev, 3, std=None)
    xs = [gen_local_tokens(1, T, H, torch.bfloat16, dev, s, 0, "normal") for s in range(3)]
    routed = [route_and_pack(x, router, k, 1, E) for x in xs]
    caps = torch.stack([probe.measure(r[1].contiguous()) for r in routed]).tolist()
    for c, r in zip(caps, routed):
        n = r[1].to(torch.int64)
        assert c == [int(n.max()), int(n.sum()), int(n.sum()), int(n.sum())]     # CAP, M, rows received
    cap = max(c[0] for c in caps)
    a2a = PaddedAllToAll(heap, e_local, cap, H, torch.bfloat16, with_return=combine, copy_mode=mode)
    a2a.token_buf.fill_(7.0)                                  # rows no exchange has used stay as they were
    high = torch.zeros(e_local, dtype=torch.int64)            # most rows each cell has ever held
    for x, (payload, counts, dst_off, _, idx, wgt, plan) in zip(xs, routed):
        out = a2a.dispatch(payload, counts, dst_off)
        a2a.wait()
        torch.cuda.synchronize()
        assert torch.equal(a2a.pca, counts.t()) and int(a2a.counts_ready[0]) == 1
        tiles = ((counts.reshape(-1) + 31) // 32).to(torch.int32)
        assert torch.equal(a2a.token_sync, tiles)
        off = 0
        for e, n in enumerate(counts.reshape(-1).tolist()):
            assert torch.equal(out[e, 0, :n], payload[off:off + n]), e
            high[e] = max(int(high[e]), n)
            assert float((out[e, 0, int(high[e]):].float() - 7.0).abs().sum()) == 0.0   # never written
            off += n
        if combine:
            a2a.send_back()
            y = a2a.reduce(plan, idx, wgt)
            ref = x.float() * wgt.sum(dim=1, keepdim=True)
            assert torch.allclose(y.float(), ref, atol=2e-2 * float(ref.abs().max()), rtol=2e-2)
            torch.cuda.synchronize()
            assert int(a2a.ret.ret_sync.abs().sum()) == 0     # re-armed by the reduce
    heap.check_status()
    del a2a, probe
    heap.close()
