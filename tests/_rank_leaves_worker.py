"""Worker of test_gpu_multi.py::test_rank_leaving_between_steps_is_detected_on_the_host.

Two ranks run fused MoE steps.  After step 2 rank 1 leaves (between steps, nothing in flight).
Rank 0 checks liveness on the host before its next launch, learns that the peer is gone within
the monitor's timeout, launches nothing further and reports.  No GPU wait runs out, no kernel
faults: the failure is made and detected on the host."""
import os
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    from iris_testing_b200.config import MoEConfig
    from iris_testing_b200.models import MoELayer, heap_bytes_needed
    from iris_testing_b200.parallel.health import HealthMonitor
    from iris_testing_b200.parallel.symm import SymmetricHeap
    from iris_testing_b200.utils import gen_local_tokens
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    monitor = HealthMonitor(timeout_s=3.0)
    cfg = MoEConfig(hidden_dim=256, ffn_dim=512, num_experts=8, topk=2, world_size=world)
    heap = SymmetricHeap(heap_bytes_needed(cfg, 256) + (16 << 20))
    layer = MoELayer(cfg, max_tokens=256, heap=heap, router_std=None)
    x = gen_local_tokens(1, 256, 256, torch.bfloat16, dev, 0, rank, "normal")
    steps_done = 0
    for step in range(5):
        if not monitor.all_alive():
            print(f"rank{rank}: peer loss detected on the host before step {step}: "
                  f"{monitor.last_error}", flush=True)
            break
        layer(x)
        torch.cuda.synchronize()
        layer.check_status()
        steps_done += 1
        # "step done on the device" on every rank, agreed on the host: after this handshake no
        # rank has a store into a peer's memory outstanding (the last kernel of a step publishes
        # its retire stamp into the peers' heaps)
        monitor.step_done()
        if rank == 1 and step == 1:
            print("rank1: leaving between steps", flush=True)
            sys.stdout.flush()
            os._exit(0)               # gone without a goodbye: no barrier, no destroy
    print(f"rank{rank}: steps_done={steps_done}", flush=True)
    # the device is still usable and nothing ran out of budget on it
    assert float(torch.ones(8, device=dev).sum()) == 8.0
    assert int(heap.status[0].item()) == 0
    print(f"rank{rank}: OK", flush=True)
    os._exit(0)                       # skip collective teardown with a missing peer


if __name__ == "__main__":
    main()
