#!/usr/bin/env python
"""Counterpart of the reference's perf sweep
(tools/wave-matmul-calibrate/wave-matmul-perf-sweep.py) on B200.

Selectors as in the reference (:864-992): --kernels picks the kernel families
(f16, f16-streamk, fa-8wave, all, with the reference's aliases; bf16 is an
addition; the mxfp4 / v9 families belong to the AMD compiler and are refused),
--m / --n / --k-values the GEMM shapes (default: the documented K sweep
512 ... 16384 at M=N=4096, `F16_DOC_K_VALUES`, :32), --streamk-workers the
Stream-K grid, --fa-batch / --fa-heads / --fa-sequence / --fa-qk-max-abs the
attention point (default B=2 H=64 S=8192 D=128, :34-37), --variants, --check,
--all-ones / --rand-int / --hpl, --seed, --keep-going, --dry-run, --csv,
--extra-calibrator-arg / --extra-fa-calibrator-arg.  Timing defaults are the
sweep's (25 warm-ups, 200 launches, 9 repeats, median; :39-41).  Every point
runs one of the drop-in calibrate tools of this directory as a child process
and is parsed from its `per_launch_us` / `tflops` lines like the reference does
(:659-677).  Writes a CSV with the reference's column names (:798-861; columns
that only exist on AMD are left empty) and prints a Markdown table.  With
--kernels=all (the default) the two 8192^3 points (f16 and bf16) that sit
beside the reference's published numbers are added to the K sweep.
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
from dataclasses import dataclass

HERE = os.path.dirname(os.path.abspath(__file__))
F16_DOC_K_VALUES = (512, 1024, 2048, 3072, 4096, 8192, 16384)
FA_DEFAULT_BATCH, FA_DEFAULT_HEADS, FA_DEFAULT_SEQUENCE, FA_HEAD_DIM = 2, 64, 8192, 128
DEFAULT_ITERS, DEFAULT_WARMUP, DEFAULT_REPEATS = 200, 25, 9
DEFAULT_STREAMK_WORKERS = 148  # one worker per SM of a B200 (the reference: 256, its part's CU count)
COLUMNS = ["kernel", "profile", "m", "n", "k", "variants", "iters", "warmup", "repeats", "us", "tflops", "cycles",
           "check", "returncode", "command", "workload", "batch", "heads", "sequence", "head_dim", "xcds", "waves"]


@dataclass(frozen=True)
class KernelSpec:
    key: str
    label: str
    workload: str  # "matmul" | "flash-attention"
    profile: str
    input_type: str = "f16"
    streamk: bool = False


KERNELS = {
    "f16": KernelSpec("f16", "f16-gemm", "matmul", "b200-f16-auto"),
    "bf16": KernelSpec("bf16", "bf16-gemm", "matmul", "b200-bf16-auto", input_type="bf16"),
    "f16-streamk": KernelSpec("f16-streamk", "f16-gemm-streamk", "matmul", "b200-f16-streamk", streamk=True),
    "fa-8wave": KernelSpec("fa-8wave", "fa-bf16", "flash-attention", "b200-fa"),
}
ALIASES = {"f16-8wave": "f16", "f16-4wave": "f16", "f16-spatial": "f16", "fa": "fa-8wave"}
AMD_ONLY = ("mxfp4", "mxfp4-4wave", "mxfp4-aiter", "mxfp", "mxfp4-8wave", "v9", "v9-transposed")


def parse_kernel_csv(text: str):
    keys = []
    for raw in (t.strip() for t in text.split(",")):
        if not raw:
            continue
        if raw == "all":
            keys += ["f16", "bf16", "fa-8wave"]
            continue
        key = ALIASES.get(raw, raw)
        if key in AMD_ONLY:
            raise argparse.ArgumentTypeError(f"kernel family '{raw}' belongs to the AMD compiler and is outside this backend")
        if key not in KERNELS:
            raise argparse.ArgumentTypeError(f"unknown kernel '{raw}'")
        keys.append(key)
    if not keys:
        raise argparse.ArgumentTypeError("at least one kernel is required")
    return [KERNELS[k] for k in dict.fromkeys(keys)]


def parse_int_csv(text: str):
    try:
        values = [int(t) for t in text.split(",") if t.strip()]
    except ValueError as err:
        raise argparse.ArgumentTypeError(str(err)) from None
    if not values or any(v <= 0 for v in values):
        raise argparse.ArgumentTypeError("expected a comma-separated list of positive integers")
    return values


def build_argparser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernels", type=parse_kernel_csv, default=None,
                    help="comma-separated f16,bf16,f16-streamk,fa-8wave,all; f16-8wave/f16-4wave/f16-spatial alias f16, "
                         "fa aliases fa-8wave")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--streamk-workers", type=int, help=f"Stream-K workers; default {DEFAULT_STREAMK_WORKERS}")
    ap.add_argument("--fa-batch", type=int, default=FA_DEFAULT_BATCH)
    ap.add_argument("--fa-heads", type=int, default=FA_DEFAULT_HEADS)
    ap.add_argument("--fa-sequence", type=int, default=FA_DEFAULT_SEQUENCE)
    ap.add_argument("--fa-xcds", type=int, default=8, help="AMD-only; accepted and ignored")
    ap.add_argument("--fa-qk-max-abs", type=float, default=1.0, help="fixed-reference |Q|,|K| bound for FA")
    ap.add_argument("--k-values", type=parse_int_csv, default=None,
                    help="comma-separated K override for the GEMM kernels; FA uses --fa-sequence")
    ap.add_argument("--iters", type=int, default=DEFAULT_ITERS, help="timed launches per repeat")
    ap.add_argument("--warmup", type=int, default=DEFAULT_WARMUP)
    ap.add_argument("--repeats", type=int, default=DEFAULT_REPEATS)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--variants", default="", help="override variants for every kernel (baseline, scheduled)")
    ap.add_argument("--check", action="store_true", help="enable CPU output checks (sampled rows for the GEMMs)")
    ap.add_argument("--check-rows", type=int, default=16, help="rows a GEMM check samples (0 = all)")
    mode = ap.add_mutually_exclusive_group()
    mode.add_argument("--all-ones", action="store_true")
    mode.add_argument("--rand-int", action="store_true")
    mode.add_argument("--hpl", action="store_true")
    ap.add_argument("--keep-going", action="store_true")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--csv", default=None, help="write summary CSV")
    ap.add_argument("--extra-calibrator-arg", action="append", default=[],
                    help="append one raw argument to wave_matmul_calibrate.py")
    ap.add_argument("--extra-fa-calibrator-arg", action="append", default=[],
                    help="append one raw argument to wave_fa_gfx950.py")
    ap.add_argument("--fa-modes", default="bounded,adaptive",
                    help="attention softmax modes to time: bounded (fixed reference), adaptive "
                         "(integrations/tlx/workloads/run_wave_perf_sweeps.py:428 times both)")
    ap.add_argument("--fa-causal", choices=["no", "yes", "both"], default="both",
                    help="also time the causal mask (an addition: the reference's kernel is non-causal)")
    ap.add_argument("--quick", action="store_true", help="fewer repeats and launches, for a smoke run")
    for flag in ("--chip", "--build-dir", "--sim-trip-count", "--build-jobs", "--compile-jobs", "--artifact-dir",
                 "--hipcc", "--rocm-lib", "--hip-visible-devices"):
        ap.add_argument(flag, default=None, help="AMD build plumbing; accepted and ignored")
    for flag in ("--skip-rebuild", "--multi-wave-specialize"):
        ap.add_argument(flag, action="store_true", help="AMD build plumbing; accepted and ignored")
    return ap


def validate_args(args) -> None:
    """wave-matmul-perf-sweep.py:994-1058."""
    for name in ("m", "n", "fa_batch", "fa_heads", "fa_sequence", "iters", "warmup", "repeats"):
        if getattr(args, name) <= 0:
            raise SystemExit(f"--{name.replace('_', '-')} must be positive")
    has_fa = any(k.workload == "flash-attention" for k in args.kernels)
    if (args.all_ones or args.rand_int or args.hpl) and has_fa and args.kernels_given:
        raise SystemExit("FA sweep supports random floating-point inputs only")
    if args.streamk_workers is not None and args.streamk_workers <= 0:
        raise SystemExit("--streamk-workers must be positive")
    if args.streamk_workers is not None and not any(k.key == "f16-streamk" for k in args.kernels):
        raise SystemExit("--streamk-workers requires --kernels=f16-streamk")
    if has_fa and (not math.isfinite(args.fa_qk_max_abs) or args.fa_qk_max_abs <= 0):
        raise SystemExit("--fa-qk-max-abs must be finite and positive")
    if args.variants:
        variants = [v.strip() for v in args.variants.split(",") if v.strip()]
        if any(v not in ("baseline", "scheduled") for v in variants):
            raise SystemExit("--variants takes baseline and/or scheduled")
        if has_fa and args.kernels_given and variants != ["scheduled"]:
            raise SystemExit("FA sweep supports only --variants=scheduled")


def run(cmd, dry_run):
    if dry_run:
        return float("nan"), float("nan"), "dry-run", 0, ""
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=1200)
    text = proc.stdout
    us = re.search(r"^median_per_launch_us: ([0-9.]+)", text, re.M) or re.search(r"^per_launch_us: ([0-9.]+)", text, re.M)
    tf = re.search(r"^median_tflops: ([0-9.]+)", text, re.M) or re.search(r"^tflops: ([0-9.]+)", text, re.M)
    # the GEMM tool checks unless told not to; the attention tool checks when asked
    asked = "--check" in cmd if any("wave_fa_gfx950" in c for c in cmd) else "--no-check" not in cmd
    check = "passed" if "output_check: passed" in text else ("failed" if asked else "skipped")
    return (float(us.group(1)) if us else float("nan"), float(tf.group(1)) if tf else float("nan"), check,
            proc.returncode, proc.stderr)


def main(argv=None) -> int:
    args = build_argparser().parse_args(sys.argv[1:] if argv is None else argv)
    args.kernels_given = args.kernels is not None
    if args.kernels is None:
        args.kernels = parse_kernel_csv("all")
    validate_args(args)
    if args.quick:
        args.iters, args.warmup, args.repeats = 20, 5, 3
    timing = ["--iters", str(args.iters), "--warmup", str(args.warmup), "--repeats", str(args.repeats)]
    # the published numbers this sweep sits beside were taken with rand_int inputs; that is the default here
    mode = ["--all-ones"] if args.all_ones else ["--hpl"] if args.hpl else ["--rand-int"]
    big = ["--bm", "4", "--bn", "4", "--wave-m-tiles", "4", "--wave-n-tiles", "4"]
    variants = args.variants or "scheduled"
    rows = []
    failed = False

    def record(row, rc, err, cmd):
        nonlocal failed
        if rc:
            failed = True
            sys.stderr.write(err)
            if not args.keep_going:
                raise SystemExit(f"command failed ({rc}): {shlex.join(cmd)}")
        rows.append(row)

    def gemm(spec: KernelSpec, m, n, k, profile=None):
        cmd = [sys.executable, os.path.join(HERE, "wave_matmul_calibrate.py"), "--m", str(m), "--n", str(n), "--k", str(k),
               *big, "--input-type", spec.input_type, "--c-type", spec.input_type, *mode, "--seed", str(args.seed), *timing]
        cmd += ["--check-rows", str(args.check_rows)] if args.check else ["--no-check"]
        if spec.streamk:
            cmd += ["--kernel-abi", "streamk", "--streamk-workers", str(args.streamk_workers or DEFAULT_STREAMK_WORKERS)]
        cmd += args.extra_calibrator_arg
        us, tf, check, rc, err = run(cmd, args.dry_run)
        record([spec.label, profile or spec.profile, m, n, k, variants, args.iters, args.warmup, args.repeats, us, tf, "",
                check, rc, shlex.join(cmd), "matmul", "", "", "", "", "", ""], rc, err, cmd)

    for spec in args.kernels:
        if spec.workload == "matmul":
            for k in (args.k_values or F16_DOC_K_VALUES):
                gemm(spec, args.m, args.n, k)
            if not args.kernels_given and spec.key in ("f16", "bf16") and args.k_values is None:
                gemm(spec, 8192, 8192, 8192, profile=f"b200-{spec.input_type}-pair256")
            continue
        # The reference times its attention kernel with the fixed softmax reference
        # (bounded) and with the running maximum (adaptive):
        # integrations/tlx/workloads/run_wave_perf_sweeps.py:428.
        causal_set = {"no": (False,), "yes": (True,), "both": (False, True)}[args.fa_causal]
        for fa_mode in [m.strip() for m in args.fa_modes.split(",") if m.strip()]:
            if fa_mode not in ("bounded", "adaptive"):
                raise SystemExit("--fa-modes takes bounded and/or adaptive")
            for causal in causal_set:
                cmd = [sys.executable, os.path.join(HERE, "wave_fa_gfx950.py"), "--batch", str(args.fa_batch), "--heads",
                       str(args.fa_heads), "--sequence", str(args.fa_sequence), "--seed", str(args.seed), *timing]
                cmd += ["--check"] if (args.check or not args.kernels_given) else []
                cmd += ["--qk-max-abs", f"{args.fa_qk_max_abs:g}"] if fa_mode == "bounded" else []
                cmd += ["--causal"] if causal else []
                cmd += args.extra_fa_calibrator_arg
                us, tf, check, rc, err = run(cmd, args.dry_run)
                record([spec.label + "-" + fa_mode + ("-causal" if causal else ""), spec.profile, "", "", "", variants,
                        args.iters, args.warmup, args.repeats, us, tf, "", check, rc, shlex.join(cmd), "flash-attention",
                        args.fa_batch, args.fa_heads, args.fa_sequence, FA_HEAD_DIM, "", ""], rc, err, cmd)
    csv_path = args.csv or os.path.join(os.getcwd(), "wave_b200_perf_sweep.csv")
    if not args.dry_run or args.csv:
        with open(csv_path, "w", newline="", encoding="utf-8") as f:
            w = csv.writer(f)
            w.writerow(COLUMNS)
            w.writerows(rows)
    print("| kernel | shape | us | TFLOP/s | check |")
    print("|---|---|---:|---:|---|")
    for r in rows:
        shape = f"{r[2]}x{r[3]}x{r[4]}" if r[15] == "matmul" else f"B={r[16]} H={r[17]} S={r[18]} D={r[19]}"
        print(f"| {r[0]} | {shape} | {r[9]:.1f} | {r[10]:.1f} | {r[12]} |")
    if args.dry_run:
        for r in rows:
            print(r[14])
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
