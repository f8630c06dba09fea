#!/usr/bin/env python
"""Counterpart of the reference's perf sweep
(tools/wave-matmul-calibrate/wave-matmul-perf-sweep.py) on B200: the f16 GEMM
K sweep at M=N=4096 (K = 512 ... 16384, `F16_DOC_K_VALUES`, :32), the 8192^3
point, and the flash-attention point B=2 H=64 S=8192 D=128 (:34-37), each timed
with the sweep's defaults (25 warm-ups, 200 launches, 9 repeats, median; :39-41)
by running the drop-in calibrate tools of this directory as child processes and
parsing their `per_launch_us` / `tflops` lines like the reference does
(:659-677).  Writes a CSV with the reference's column names (:798-861; columns
that only exist on AMD are left empty) and prints a Markdown table.
"""
from __future__ import annotations

import argparse
import csv
import math
import os
import re
import shlex
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
F16_DOC_K_VALUES = (512, 1024, 2048, 3072, 4096, 8192, 16384)
COLUMNS = ["kernel", "profile", "m", "n", "k", "variants", "iters", "warmup", "repeats", "us", "tflops", "cycles",
           "check", "returncode", "command", "workload", "batch", "heads", "sequence", "head_dim", "xcds", "waves"]


def run(cmd):
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1200)
    text = proc.stdout
    us = re.search(r"^median_per_launch_us: ([0-9.]+)", text, re.M) or re.search(r"^per_launch_us: ([0-9.]+)", text, re.M)
    tf = re.search(r"^median_tflops: ([0-9.]+)", text, re.M) or re.search(r"^tflops: ([0-9.]+)", text, re.M)
    check = "passed" if "output_check: passed" in text else ("skipped" if "--no-check" in cmd else "failed")
    return (float(us.group(1)) if us else float("nan"), float(tf.group(1)) if tf else float("nan"), check,
            proc.returncode, proc.stderr)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=25)
    ap.add_argument("--repeats", type=int, default=9)
    ap.add_argument("--csv", default=os.path.join(os.getcwd(), "wave_b200_perf_sweep.csv"))
    ap.add_argument("--input-mode", choices=["rand-int", "hpl", "lcg"], default="rand-int")
    ap.add_argument("--check-rows", type=int, default=16)
    ap.add_argument("--fa-qk-max-abs", type=float, default=1.0,
                    help="fixed-reference |Q|,|K| bound for the bounded attention rows (wave-matmul-perf-sweep.py:887-892)")
    ap.add_argument("--quick", action="store_true", help="fewer repeats and launches, for a smoke run")
    args = ap.parse_args()
    if not math.isfinite(args.fa_qk_max_abs) or args.fa_qk_max_abs <= 0:
        raise SystemExit("--fa-qk-max-abs must be finite and positive")  # wave-matmul-perf-sweep.py:1046-1047
    if args.quick:
        args.iters, args.warmup, args.repeats = 20, 5, 3
    timing = ["--iters", str(args.iters), "--warmup", str(args.warmup), "--repeats", str(args.repeats)]
    mode = [] if args.input_mode == "lcg" else ["--" + args.input_mode]
    big = ["--bm", "4", "--bn", "4", "--wave-m-tiles", "4", "--wave-n-tiles", "4"]
    rows = []

    def gemm(label, profile, m, n, k, in_type, c_type):
        cmd = [sys.executable, os.path.join(HERE, "wave_matmul_calibrate.py"), "--m", str(m), "--n", str(n), "--k", str(k),
               *big, "--input-type", in_type, "--c-type", c_type, *mode, "--check-rows", str(args.check_rows), *timing]
        us, tf, check, rc, err = run(cmd)
        if rc:
            sys.stderr.write(err)
        rows.append([label, profile, m, n, k, "scheduled", args.iters, args.warmup, args.repeats, us, tf, "", check, rc,
                     shlex.join(cmd), "matmul", "", "", "", "", "", ""])

    for k in F16_DOC_K_VALUES:
        gemm("f16-gemm", "b200-f16-auto", 4096, 4096, k, "f16", "f16")
    gemm("f16-gemm", "b200-f16-pair256", 8192, 8192, 8192, "f16", "f16")
    gemm("bf16-gemm", "b200-bf16-pair256", 8192, 8192, 8192, "bf16", "bf16")
    # The reference times its attention kernel with the fixed softmax reference
    # (bounded) and with the running maximum (adaptive):
    # integrations/tlx/workloads/run_wave_perf_sweeps.py:428.
    for mode, causal in (("bounded", False), ("adaptive", False), ("bounded", True), ("adaptive", True)):
        cmd = [sys.executable, os.path.join(HERE, "wave_fa_gfx950.py"), "--batch", "2", "--heads", "64", "--sequence", "8192",
               "--check", *timing] + (["--qk-max-abs", f"{args.fa_qk_max_abs:g}"] if mode == "bounded" else []) + (
                   ["--causal"] if causal else [])
        us, tf, check, rc, err = run(cmd)
        if rc:
            sys.stderr.write(err)
        rows.append(["fa-bf16-" + mode + ("-causal" if causal else ""), "b200-fa-256x128", "", "", "", "scheduled",
                     args.iters, args.warmup, args.repeats, us, tf, "", check, rc, shlex.join(cmd), "flash-attention", 2,
                     64, 8192, 128, "", ""])
    with open(args.csv, "w", newline="", encoding="utf-8") as f:
        w = csv.writer(f)
        w.writerow(COLUMNS)
        w.writerows(rows)
    print("| kernel | shape | us | TFLOP/s | check |")
    print("|---|---|---:|---:|---|")
    for r in rows:
        shape = f"{r[2]}x{r[3]}x{r[4]}" if r[15] == "matmul" else f"B={r[16]} H={r[17]} S={r[18]} D={r[19]}"
        print(f"| {r[0]} | {shape} | {r[9]:.1f} | {r[10]:.1f} | {r[12]} |")
    return 1 if any(r[13] for r in rows) else 0


if __name__ == "__main__":
    raise SystemExit(main())
