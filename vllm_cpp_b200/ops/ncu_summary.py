"""Turns the raw CSV page of an ncu report into the short text kept under ``profiles/``.

    ncu -i report.ncu-rep --page raw --csv | python -m vllm_cpp_b200.ops.ncu_summary \\
        --title "kernel, workload" --command "the ncu command" [--plain "plain-run line"] \\
        [--flops F] [--bytes B]

``--flops`` / ``--bytes``: algorithmic work of one launch; the summary then states the achieved
rate under ncu and its fraction of the measured peaks (cuBLAS bf16 burst, copy bandwidth) read
from ``MEASURED_PEAKS.json`` beside the package when present.
"""
from __future__ import annotations

import argparse
import csv
import json
import sys
from pathlib import Path

KEEP = [
    "gpu__time_duration.sum",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",
    "dram__bytes_read.sum",
    "dram__bytes_write.sum",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active",
    "sm__inst_executed_pipe_tensor.sum",
    "sm__warps_active.avg.pct_of_peak_sustained_active",
    "lts__t_sector_hit_rate.pct",
    "launch__registers_per_thread",
    "launch__grid_size",
    "launch__block_size",
    "launch__cluster_size",
    "launch__shared_mem_per_block_dynamic",
    "launch__occupancy_limit_registers",
    "launch__occupancy_limit_shared_mem",
    "smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio",
    "smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio",
    "smsp__average_warps_issue_stalled_sleeping_per_issue_active.ratio",
]


def peaks():
    for base in (Path(__file__).resolve().parents[2], Path.cwd()):
        f = base / "MEASURED_PEAKS.json"
        if f.exists():
            try:
                d = json.loads(f.read_text())
                return float(d.get("bf16_tflops", 0) or 0), float(d.get("hbm_gbs", 0) or 0), "measured"
            except Exception:
                pass
    return 1590.0, 6650.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--title", required=True)
    ap.add_argument("--command", required=True)
    ap.add_argument("--plain", default="")
    ap.add_argument("--flops", type=float, default=0.0)
    ap.add_argument("--bytes", type=float, default=0.0)
    args = ap.parse_args()
    rows = list(csv.reader(sys.stdin))
    hdr = next(i for i, r in enumerate(rows) if "Kernel Name" in r)
    names, units = rows[hdr], rows[hdr + 1]
    col = {n: i for i, n in enumerate(names)}
    tf, gbs, which = peaks()
    out = [args.title, "", "Command (one B200, after the same command exited 0 without ncu):",
           "  " + args.command]
    if args.plain:
        out.append("Plain run of the same command (CUDA events, not under ncu): " + args.plain)
    for li, r in enumerate(rows[hdr + 2:]):
        if len(r) < len(names):
            continue
        out += ["", f"launch {li}: {r[col['Kernel Name']]}"]
        for k in KEEP:
            if k in col and r[col[k]] != "":
                out.append(f"  {k:<82} {r[col[k]]} {units[col[k]]}")
        t = r[col["gpu__time_duration.sum"]].replace(",", "") if "gpu__time_duration.sum" in col else ""
        if t:
            tu = units[col["gpu__time_duration.sum"]]
            sec = float(t) * {"ns": 1e-9, "us": 1e-6, "ms": 1e-3, "s": 1.0}.get(tu, 1e-6)
            if args.flops:
                r_tf = args.flops / sec / 1e12
                out.append(f"  -> {r_tf:.1f} TFLOP/s under ncu = {r_tf / tf:.2f} of {which} cuBLAS bf16 burst ({tf:.1f} TF)")
            if args.bytes:
                r_gb = args.bytes / sec / 1e9
                out.append(f"  -> algorithmic {args.bytes / 1e6:.1f} MB, {r_gb:.0f} GB/s under ncu = "
                           f"{r_gb / gbs:.2f} of {which} copy bandwidth ({gbs:.1f} GB/s)")
    print("\n".join(out))


if __name__ == "__main__":
    main()
