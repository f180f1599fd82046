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
