"""Turns an Nsight Compute report into the short per-kernel table used under ``profiles/``.

    python -m iris_testing_b200.utils.ncu_summary report.ncu-rep [--kernel regex]

Reads the report with ``ncu -i <file> --page raw --csv`` (works without a GPU) and prints, per
captured launch: duration, tensor-pipe activity, DRAM bytes and throughput, L2 hit rate,
registers, launch shape.  Nothing is disassembled; only counters are read.
"""
from __future__ import annotations

import argparse
import csv
import io
import re
import subprocess
import sys

METRICS = [
    ("time", "gpu__time_duration.sum"),
    ("tensor_active_pct", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active"),
    ("tensor_elapsed_pct", "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed"),
    ("dram_read", "dram__bytes_read.sum"),
    ("dram_write", "dram__bytes_write.sum"),
    ("dram_pct", "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed"),
    ("l2_hit_pct", "lts__t_sector_hit_rate.pct"),
    ("regs", "launch__registers_per_thread"),
    ("block", "launch__block_size"),
    ("grid", "launch__grid_size"),
    ("cluster", "launch__cluster_dim_x"),
    ("smem_kb", "launch__shared_mem_per_block_dynamic"),
    ("warps_active_pct", "sm__warps_active.avg.pct_of_peak_sustained_active"),
    ("stall_long_scoreboard", "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio"),
]


def read_report(path: str):
    res = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"ncu could not read {path}: {res.stderr.strip()[:300]}")
    rows = list(csv.reader(io.StringIO(res.stdout)))
    if len(rows) < 3:
        raise RuntimeError("report holds no captured launches")
    return rows[0], rows[1], rows[2:]


def summarise(path: str, kernel_regex: str | None = None):
    header, units, launches = read_report(path)
    col = {name: i for i, name in enumerate(header)}
    out = []
    for row in launches:
        name = row[col["Kernel Name"]]
        if kernel_regex and not re.search(kernel_regex, name):
            continue
        rec = {"kernel": re.sub(r"\(.*", "", name)}
        for key, metric in METRICS:
            if metric in col:
                rec[key] = f"{row[col[metric]]} {units[col[metric]]}".strip()
        out.append(rec)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("report")
    ap.add_argument("--kernel", default=None, help="only launches whose kernel name matches this regex")
    a = ap.parse_args()
    recs = summarise(a.report, a.kernel)
    if not recs:
        print("no matching launches", file=sys.stderr)
        sys.exit(1)
    keys = ["kernel"] + [k for k, _ in METRICS]
    print("| " + " | ".join(keys) + " |")
    print("|" + "---|" * len(keys))
    for r in recs:
        print("| " + " | ".join(r.get(k, "") for k in keys) + " |")


if __name__ == "__main__":
    main()
