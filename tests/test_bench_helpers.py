"""CPU tests of bench.py's host-side helpers (clock-sample parsing, reference install check)."""
import importlib.util
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_module"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_clock_sampler_parses_samples_inside_the_timed_window(tmp_path):
    bench = _load_bench()
    s = bench.ClockSampler(0)
    now = time.time()

    def stamp(t):
        lt = time.localtime(t)
        return time.strftime("%Y/%m/%d %H:%M:%S", lt) + f".{int((t % 1) * 1000):03d}"

    rows = [
        (now - 10.0, 300, 1965, 120.0, "Not Active"),      # before the window: ignored
        (now + 0.10, 1207, 1965, 621.2, "Active"),
        (now + 0.20, 1350, 1965, 640.0, "Active"),
        (now + 0.30, 1290, 1965, 650.5, "Not Active"),
        (now + 50.0, 1965, 1965, 100.0, "Not Active"),      # after the window: ignored
    ]
    path = tmp_path / "clocks.csv"
    path.write_text("".join(
        f"{stamp(t)}, {sm}, {mx}, {pw}, 0x0000000000000004, Not Active, Not Active, Not Active, {cap}\n"
        for t, sm, mx, pw, cap in rows))

    class Done:
        def terminate(self): pass
        def wait(self, timeout=None): return 0
        def kill(self): pass

    s.proc, s.path = Done(), str(path)
    s.t_begin, s.t_end = now, now + 0.4
    out = s.stop()
    assert out["samples"] == 3 and out["sm_mhz"] == 1290 and out["sm_max_mhz"] == 1965
    assert out["reasons"] == ["sw_power_cap"] and abs(out["power_w_max"] - 650.5) < 1e-6


def test_reference_arm_reports_unavailable_without_a_reference(tmp_path, monkeypatch):
    bench = _load_bench()
    monkeypatch.setattr(bench, "ROOT", tmp_path)            # no baseline/_ref, no reference next to it
    monkeypatch.setenv("REFERENCE_DIR", str(tmp_path / "does_not_exist"))
    err = bench.ensure_reference()
    assert isinstance(err, str) and "missing" in err


def _args(bench, argv):
    import argparse
    ns = argparse.Namespace(gpus=1, steps=3, warmup=3, impl="ours", mode="layer", model="mixtral-8x7b", experts=0,
                            topk=0, batch=0, seq=0, hidden=4096, combine=False, zipf=0.0, zipf_scale=1.0, seed=0,
                            check_tokens=2048, no_check=False, sweep=None, ref_packer="auto")
    for k, v in argv.items():
        setattr(ns, k, v)
    from iris_testing_b200.bench_harness import MODEL_DEFAULTS
    d = MODEL_DEFAULTS["a2a" if ns.mode == "a2a" else ns.model]
    ns.batch = ns.batch or d["batch"]
    ns.seq = ns.seq or d["seq"]
    return ns


def test_both_arms_print_the_same_config_and_nothing_else_in_it():
    """``config`` is built from the arguments alone, so it cannot differ between the arms; prose and
    memory figures live in sibling keys."""
    bench = _load_bench()
    from iris_testing_b200.bench_harness import describe_config, make_config
    for argv in (dict(), dict(model="fine-grained", experts=64, topk=8), dict(model="large", zipf=1.2),
                 dict(mode="a2a", combine=True, batch=16, seq=1024)):
        ours, ref = _args(bench, dict(argv, impl="ours")), _args(bench, dict(argv, impl="reference"))
        c1 = describe_config(ours, make_config(ours, 8), 8)
        c2 = describe_config(ref, make_config(ref, 8), 8)
        assert c1 == c2
        assert "timed" not in c1 and "capacity_rows" not in c1
        assert c1["tokens_per_rank"] == ours.batch * ours.seq and c1["parallelism"] == "ep8"
    cfg = make_config(_args(bench, dict(model="fine-grained", experts=128, topk=2)), 8)
    assert (cfg.num_experts, cfg.topk, cfg.e_local, cfg.hidden_dim, cfg.ffn_dim) == (128, 2, 16, 2048, 1408)


def test_published_sweeps_cover_the_configurations():
    bench = _load_bench()
    c2 = bench.SWEEPS["config2"]
    pts = {(p["batch"], p["seq"], p["combine"]) for p in c2}
    for comb in (False, True):
        assert {(b, 1024, comb) for b in (1, 2, 4, 8, 16)} <= pts
        assert {(4, s, comb) for s in (128, 256, 512, 2048, 4096)} <= pts
    c4 = {(p["experts"], p["topk"]) for p in bench.SWEEPS["config4"]}
    assert {(e, k) for e in (8, 32, 128) for k in (1, 2, 8)} <= c4
    assert [p["zipf"] for p in bench.SWEEPS["config5"]] == [1.2, 0.0]
    small = bench.SWEEPS["small"]
    assert [p["batch"] * p["seq"] for p in small] == [64, 256, 512, 1024, 2048]
    assert all(p["model"] == "mixtral-8x7b" and p["mode"] == "layer" for p in small)


def test_vectorized_reference_packer_builds_the_reference_payload():
    """The tensor-op packer used for large inputs of the reference arm must produce the payload the
    reference's bucket loop produces (rows by destination, then local expert, stable)."""
    import torch
    from iris_testing_b200.bench_harness import reference_pack
    torch.manual_seed(0)
    T, H, E, k, world = 40, 16, 8, 2, 4
    x = torch.randn(T, H)
    router = torch.randn(H, E) * 0.3
    payload, counts, order, vals, idx = reference_pack(None, x, router, k, world, E, None, "vectorized")
    e_local = E // world
    buckets = [[[] for _ in range(e_local)] for _ in range(world)]
    for t in range(T):
        for s in range(k):
            ex = int(idx[t, s])
            buckets[ex // e_local][ex % e_local].append(x[t])
    rows = [r for row in buckets for b in row for r in b]
    assert torch.equal(payload, torch.stack(rows))
    assert counts.tolist() == [[len(b) for b in row] for row in buckets]
    assert torch.equal(x[order // k], payload)
