#!/usr/bin/env python
"""Turns an Nsight Compute report into the short text summary kept under ``profiles/``.

    python benchmarks/ncu_summary.py REPORT.ncu-rep [--title "kernel and workload"] [--command "how it was captured"]
                                     [--algorithmic-bytes N] [--flops N]

Reads the report with ``ncu -i REPORT --page raw --csv`` (no GPU needed) and prints, per captured launch: duration,
DRAM bytes read / written and throughput as a fraction of the device's peak, tensor-pipe activity, achieved
occupancy, registers, issue rate and the dominant stall reason.  With ``--algorithmic-bytes`` / ``--flops`` (per
launch) it adds the achieved rate against the measured peaks (``MEASURED_PEAKS.json`` beside the repository root
when present).
"""
from __future__ import annotations

import argparse
import csv
import io
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WANT = {
    "gpu__time_duration.sum": "duration",
    "dram__bytes_read.sum": "dram read",
    "dram__bytes_write.sum": "dram write",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "dram throughput, % of peak",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor pipe active, %",
    "sm__inst_executed_pipe_tensor.sum": "tensor instructions",
    "sm__warps_active.avg.pct_of_peak_sustained_active": "achieved occupancy, %",
    "launch__registers_per_thread": "registers / thread",
    "launch__grid_size": "grid",
    "launch__block_size": "block",
    "launch__waves_per_multiprocessor": "waves / SM",
    "sm__inst_executed.sum.per_cycle_elapsed": "warp instructions / cycle (whole GPU)",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed": "SM throughput, % of peak",
    "lts__t_sectors_op_red.sum": "L2 reduction sectors",
    "lts__t_bytes.sum": "L2 bytes",
    "l1tex__t_bytes.sum": "L1 bytes",
    "smsp__cycles_active.avg": "active cycles / SMSP",
}


def read_report(path: str):
    out = subprocess.run(["ncu", "-i", path, "--page", "raw", "--csv"], capture_output=True, text=True, check=True).stdout
    rows = list(csv.reader(io.StringIO(out)))
    header, units = rows[0], rows[1]
    return header, units, rows[2:]


def stall_reasons(header, row):
    best = []
    for i, h in enumerate(header):
        if h.startswith("smsp__average_warps_issue_stalled_") and h.endswith("_per_issue_active.ratio"):
            try:
                best.append((float(row[i].replace(",", "")), h[len("smsp__average_warps_issue_stalled_"):-len("_per_issue_active.ratio")]))
            except ValueError:
                pass
    return sorted(best, reverse=True)[:3]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("report")
    ap.add_argument("--title", default="")
    ap.add_argument("--command", default="")
    ap.add_argument("--algorithmic-bytes", type=float, default=0.0)
    ap.add_argument("--flops", type=float, default=0.0)
    a = ap.parse_args()
    header, units, launches = read_report(a.report)
    peaks = {}
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as f:
            peaks = json.load(f)
    print(f"# {a.title or os.path.basename(a.report)}\n")
    if a.command:
        print(f"Captured with: `{a.command}`\n")
    col = {h: i for i, h in enumerate(header)}
    for n, row in enumerate(launches):
        name = row[col["Kernel Name"]] if "Kernel Name" in col else "?"
        print(f"## launch {n}: `{name[:120]}`\n")
        for key, label in WANT.items():
            if key in col and row[col[key]] != "":
                print(f"- {label}: {row[col[key]]} {units[col[key]]}".rstrip())
        top = stall_reasons(header, row)
        if top:
            print("- top stall reasons (warps stalled per issue): " + ", ".join(f"{k} {v:.2f}" for v, k in top))
        try:
            dur_s = float(row[col["gpu__time_duration.sum"]].replace(",", "")) * {"ns": 1e-9, "us": 1e-6, "ms": 1e-3, "s": 1.0}[
                units[col["gpu__time_duration.sum"]].replace("second", "s").replace("usecond", "us")]
        except (KeyError, ValueError):
            dur_s = 0.0
        if dur_s and a.algorithmic_bytes:
            gbs = a.algorithmic_bytes / dur_s / 1e9
            frac = f" = {gbs / peaks['hbm_gbs']:.2f} of measured copy bandwidth ({peaks['hbm_gbs']:.0f} GB/s)" if "hbm_gbs" in peaks else ""
            print(f"- algorithmic bytes {a.algorithmic_bytes / 1e6:.1f} MB -> {gbs:.0f} GB/s under the profiler{frac}")
        if dur_s and a.flops:
            tf = a.flops / dur_s / 1e12
            frac = f" = {tf / peaks['bf16_tflops']:.2f} of measured cuBLAS burst ({peaks['bf16_tflops']:.0f} TFLOP/s)" if "bf16_tflops" in peaks else ""
            print(f"- {a.flops / 1e9:.1f} GFLOP -> {tf:.0f} TFLOP/s under the profiler{frac}")
        print()
    print("(Durations under the profiler are with cold caches and serialised launches: use them for shares and "
          "ratios; the timed figures are the CUDA-event numbers of `benchmarks/bench_kernels.py`.)")


if __name__ == "__main__":
    sys.exit(main())
