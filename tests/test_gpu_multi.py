"""Multi-GPU tests: run the multi-process drivers as child processes on the GPUs present
(skipped on a single-GPU box).  NVLS is off in NCCL; the kernels use plain peer stores."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _run(script, world, extra_env=None, timeout=600):
    env = dict(os.environ, WORLD_SIZE=str(world), NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1",
               MASTER_PORT=str(29600 + world), **(extra_env or {}))
    for k in ("RANK", "LOCAL_RANK"):
        env.pop(k, None)
    return subprocess.run([sys.executable, str(ROOT / script)], env=env, capture_output=True, text=True,
                          timeout=timeout, cwd=str(ROOT))


def _worlds():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return [w for w in (2, 4, 8) if w <= n]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_unit_tests_driver(world):
    if world not in _worlds():
        pytest.skip(f"needs {world} GPUs")
    res = _run("unit_tests.py", world)
    assert res.returncode == 0 and "ALL PASSED" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_benchmark_driver_correctness_report():
    if 2 not in _worlds():
        pytest.skip("needs 2 GPUs")
    res = _run("benchmark.py", 2, dict(BATCH="2", SEQ="512", HIDDEN="1024", E_LOCAL="4", CAPACITY="0",
                                       WARMUP="2", ITERS="3", CHECK="1", TOKEN_DIST="normal"))
    assert res.returncode == 0 and "PASS" in res.stdout and "FAIL" not in res.stdout, \
        res.stdout[-2000:] + res.stderr[-2000:]


def test_rank_leaving_between_steps_is_detected_on_the_host():
    """Failure detection without a GPU fault: a rank exits between steps; the survivor learns of
    it from the host-side monitor (short gloo timeout) before launching its next step."""
    if 2 not in _worlds():
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, WORLD_SIZE="2", NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29655")
    procs = []
    for r in range(2):
        e = dict(env, RANK=str(r), LOCAL_RANK=str(r))
        procs.append(subprocess.Popen([sys.executable, str(ROOT / "tests" / "_rank_leaves_worker.py")], env=e,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=str(ROOT)))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=180)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[killed after timeout]"
        outs.append(out)
    assert "rank1: leaving between steps" in outs[1], outs[1][-1500:]
    assert "peer loss detected on the host before step 2" in outs[0], outs[0][-1500:]
    assert "rank0: steps_done=2" in outs[0] and "rank0: OK" in outs[0], outs[0][-1500:]
