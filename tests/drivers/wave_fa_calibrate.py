#!/usr/bin/env python
"""Drop-in for the reference's toy flash-attention calibrate tool
(tools/wave-fa-calibrate/wave-fa-calibrate.py:298-342 and its timed runner
wave-fa-calibrate-runner.cpp) on B200: --block-m --block-n --head-dim --seq-n
--seed --iters --warmup --repeats --variants --no-check --skip-hw, with the
runner's argument rules (runner:142-161: block-m = block-n = 16, head-dim a
power of two and a multiple of 16, seq-n a multiple of block-n) and exit code 2
when they are broken.  The kernel is looked up by the reference's name,
`flash_attention_f32` (python/mlir/dialects/wave_attention.py:18), through the
C ABI's name-based launch facade and launched with the runner's argument block
{&Q, &K, &V, &O}.  Prints the runner's keys (`kernel:`, `shape:`, `grid:`,
`iters:`, `total_ms:`, `per_launch_us:`, `per_launch_cycles_wallclock:`,
`output_check: passed max_abs_diff=... index=...`; runner:263-292) and, with
--repeats, `median_per_launch_us:`.  The check is the runner's: every output
element against the f64 exp2 reference, max-abs <= 3e-3 (runner:250-273).
"""
from __future__ import annotations

import argparse
import ctypes as C
import importlib
import math
import sys

import numpy as np

from _common import add_ignored_flags, dev_bits, load, median, note_ignored, time_launches

KERNEL_NAME = "flash_attention_f32"
VARIANTS = ("baseline", "scheduled")


def parse_variants(text: str):
    names = [v.strip() for v in text.split(",") if v.strip()]
    for v in names:
        if v not in VARIANTS:
            raise argparse.ArgumentTypeError(f"unknown variant '{v}' (expected one of: {', '.join(VARIANTS)})")
    if not names:
        raise argparse.ArgumentTypeError("at least one variant is required")
    return names


def parse(argv):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--block-m", type=int, default=16)
    p.add_argument("--block-n", type=int, default=16)
    p.add_argument("--head-dim", type=int, default=32)
    p.add_argument("--seq-n", type=int, default=16)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--iters", type=int, default=1000)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--repeats", type=int, default=1, help="hardware timing repeats per variant; reports median")
    p.add_argument("--variants", type=parse_variants, default=parse_variants("baseline,scheduled"),
                   help="comma-separated variants: baseline, scheduled (one kernel serves both here)")
    p.add_argument("--skip-hw", action="store_true", help="validate the arguments and print the launch geometry only")
    p.add_argument("--no-check", action="store_true")
    for flag in ("--print-candidates", "--print-score", "--print-regions", "--keep-tmp"):
        p.add_argument(flag, action="store_true", help="scheduler diagnostics of the AMD compiler; accepted and ignored")
    for flag in ("--calibration-file", "--tile-loop-unroll", "--build-dir", "--hipcc", "--rocm-lib"):
        p.add_argument(flag, default=None, help="AMD build plumbing; accepted and ignored")
    add_ignored_flags(p)
    return p.parse_args(argv)


def validate(args) -> str | None:
    """wave-fa-calibrate.py:345-361 and wave-fa-calibrate-runner.cpp:142-161."""
    for name in ("block_m", "block_n", "head_dim", "seq_n", "iters", "repeats"):
        if getattr(args, name) <= 0:
            return f"--{name.replace('_', '-')} must be positive"
    if args.warmup < 0:
        return "--warmup must be non-negative"
    if args.head_dim & (args.head_dim - 1):
        return "head-dim must be a power of two"
    if args.block_m != 16 or args.block_n != 16:
        return "MMA FA kernel requires block-m=16 and block-n=16"
    if args.seq_n % args.block_n:
        return "seq-n must be a multiple of block-n"
    if args.head_dim % 16:
        return "head-dim must be a multiple of 16"
    return None


def main(argv=None) -> int:
    args = parse(sys.argv[1:] if argv is None else argv)
    problem = validate(args)
    if problem:
        sys.stderr.write(problem + "\n")
        return 2
    note_ignored(args)
    torch, wc, oracle = load()
    wa = importlib.import_module("7_b200.wave_attention")
    q, k, v = wa.generate_flash_attention_f32_inputs(args.block_m, args.head_dim, args.seq_n, random_seed=args.seed)
    # The toy kernel's probabilities are 2^(q.k - max) with q already scaled
    # (wave_attention.py:271); a softmax scale of ln 2 makes exp2(scale*log2(e)*s) exactly that.
    desc = wc.fa_desc(1, 1, args.block_m, args.seq_n, args.head_dim, scale=math.log(2.0), io_type=wc.F16, out_f32=True)
    fn = C.c_void_p()
    rc = wc.lib().wave_cuda_module_get_function(KERNEL_NAME.encode(), C.byref(desc), C.byref(fn))
    if rc != wc.OK:
        sys.stderr.write(wc.lib().wave_cuda_last_error().decode() + "\n")
        return 2 if rc in (wc.E_INVALID, wc.E_UNSUPPORTED) else 1
    dq, dk, dv = (dev_bits(torch, x) for x in (q, k, v))
    o = torch.full((args.block_m, args.head_dim), float("nan"), dtype=torch.float32, device="cuda")
    ptrs = [C.c_void_p(t.data_ptr()) for t in (dq, dk, dv, o)]
    block = (C.c_void_p * 4)(*[C.cast(C.pointer(x), C.c_void_p) for x in ptrs])
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        wc.check(wc.lib().wave_cuda_launch(fn, block, stream))

    props = torch.cuda.get_device_properties(0)
    clock_mhz = float(torch.cuda.clock_rate()) if hasattr(torch.cuda, "clock_rate") else 0.0
    status = 0
    try:
        for variant in args.variants:
            print(f"variant: {variant}")
            print(f"device: {props.name} (sm_{props.major}{props.minor}a) shader_clock_mhz={clock_mhz:.0f}")
            print(f"kernel: {KERNEL_NAME}")
            print(f"shape: block_m={args.block_m} block_n={args.block_n} seq_n={args.seq_n} head_dim={args.head_dim} "
                  f"seed={args.seed} threads=384")
            print("grid: 1,1,1 block: 384,1,1 waves_per_workgroup=12")
            if args.skip_hw:
                continue
            times = [time_launches(torch, launch, args.warmup, args.iters) for _ in range(args.repeats)]
            wc.check_device_status()
            us = [t * 1e3 / args.iters for t in times]
            print(f"iters: {args.iters}")
            print(f"total_ms: {times[-1]:.3f}")
            for t in us:
                print(f"per_launch_us: {t:.3f}")
                print(f"per_launch_cycles_wallclock: {t * clock_mhz:.0f}")
            if args.repeats > 1:
                print(f"median_per_launch_us: {median(us):.3f}")
            if not args.no_check:
                want = oracle.fa_ref(q[None], k[None], v[None], oracle.F16, 1.0, exp2_mode=True)[0]
                got = o.cpu().numpy().astype(np.float64)
                diff = np.abs(got - want).reshape(-1)
                worst = int(np.nanargmax(np.where(np.isnan(diff), np.inf, diff)))
                if not diff[worst] <= 3.0e-3:
                    sys.stderr.write(f"output_check: failed index={worst} expected={want.reshape(-1)[worst]:.8f} "
                                     f"got={got.reshape(-1)[worst]:.8f} abs_diff={diff[worst]:.8f}\n")
                    status = 1
                    break
                print(f"output_check: passed max_abs_diff={diff[worst]:.8f} index={worst}")
    except wc.WaveCudaError as err:
        sys.stderr.write(err.message + "\n")
        status = 1
    finally:
        wc.lib().wave_cuda_function_release(fn)
    return status


if __name__ == "__main__":
    raise SystemExit(main())
