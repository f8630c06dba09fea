#!/usr/bin/env python
"""Drop-in for the reference's GEMM calibrate runner
(tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp, driven by
wave-matmul-calibrate.py) on B200: same shape/tiling/input-mode/timing flags
(runner.cpp:36-64, 71-102), same stdout keys (`kernel:`, `shape:`, `grid:`,
`iters:`, `total_ms:`, `per_launch_us:`, `output_check: passed mode=strict ...`,
`streamk_counter_check: passed`; runner.cpp:1881-1908, 918-954, 1732) so the
reference's regex parsers (tools/wave_calibration.py:262-271) keep working,
plus `tflops:` and `roofline_fraction:`.  Exit codes as in the runner: 1 on a
failed check or CUDA error, 2 on bad arguments.
"""
from __future__ import annotations

import argparse
import sys
import time

import numpy as np

from _common import time_sustained, add_ignored_flags, dev_bits, load, median, note_ignored, time_launches

MODE_NAMES = {0: "lcg", 1: "all_ones", 2: "rand_int", 3: "hpl"}


def parse(argv):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--kernel", default=None)
    p.add_argument("--m", type=int, default=32)
    p.add_argument("--n", type=int, default=32)
    p.add_argument("--k", type=int, default=32)
    p.add_argument("--bm", type=int, default=1)
    p.add_argument("--bn", type=int, default=2)
    p.add_argument("--wave-m-tiles", type=int, default=1)
    p.add_argument("--wave-n-tiles", type=int, default=1)
    p.add_argument("--wave-k-tiles", type=int, default=1)
    p.add_argument("--input-type", choices=["f16", "bf16"], default="f16")
    p.add_argument("--c-type", choices=["f32", "f16", "bf16"], default="f32")
    p.add_argument("--output-layout", choices=["automatic", "row-major", "column-major", "tile-packed"],
                   default="automatic")
    p.add_argument("--accumulator-layout", choices=["automatic", "mfma", "wmma"], default="automatic",
                   help="fragment order inside a tile of tile-packed output (runner.cpp:765-769)")
    p.add_argument("--wave-size", type=int, choices=[32, 64], default=32)
    p.add_argument("--kernel-abi", choices=["matmul", "streamk"], default="matmul")
    p.add_argument("--streamk-workers", type=int, default=1)
    p.add_argument("--cta-group-m", type=int, default=1)
    p.add_argument("--iters", type=int, default=1000)
    p.add_argument("--warmup", type=int, default=10)
    p.add_argument("--repeats", type=int, default=1)
    p.add_argument("--sustained-seconds", type=float, default=0.0,
                   help="also time a back-to-back loop of at least this long (the clock the power cap allows)")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--all-ones", action="store_true")
    p.add_argument("--rand-int", action="store_true")
    p.add_argument("--hpl", action="store_true")
    p.add_argument("--no-check", action="store_true")
    p.add_argument("--check-rows", type=int, default=0,
                   help="check only this many evenly spaced rows (0 = all); large shapes take minutes on the CPU")
    add_ignored_flags(p)
    return p.parse_args(argv)


def main(argv=None) -> int:
    args = parse(sys.argv[1:] if argv is None else argv)
    note_ignored(args, handled=("--wave-size",))
    if sum([args.all_ones, args.rand_int, args.hpl]) > 1:
        sys.stderr.write("--all-ones, --rand-int and --hpl are mutually exclusive\n")
        return 2
    if args.iters <= 0 or args.warmup < 0 or args.repeats <= 0:
        sys.stderr.write("--iters and --repeats must be positive, --warmup non-negative\n")
        return 2
    torch, wc, oracle = load()
    layout = "row-major" if args.output_layout == "automatic" else args.output_layout
    if layout == "tile-packed":
        # getEffectiveAccumulatorLayout (runner.cpp:765-769): MFMA on wave64, WMMA on wave32 unless told otherwise
        acc = args.accumulator_layout
        if acc == "automatic":
            acc = "mfma" if args.wave_size == 64 else "wmma"
        if acc == "wmma" and args.wave_size != 32:
            sys.stderr.write("WMMA output check requires wave32\n")
            return 2
        layout = f"tile-packed-{acc}{args.wave_size}"
    streamk = args.streamk_workers if args.kernel_abi == "streamk" else 1
    desc = wc.gemm_desc(args.m, args.n, args.k, bm=args.bm, bn=args.bn, wave_m_tiles=args.wave_m_tiles,
                        wave_n_tiles=args.wave_n_tiles, wave_k_tiles=args.wave_k_tiles,
                        in_type=wc.TYPE_BY_NAME[args.input_type], out_type=wc.TYPE_BY_NAME[args.c_type],
                        out_layout=wc.LAYOUT_BY_NAME[layout], cta_group_m=args.cta_group_m, streamk_workers=streamk)
    try:
        wc.gemm_validate(desc)
        scratch, counters = wc.gemm_workspace_bytes(desc)
        plan = wc.gemm_plan(desc)
    except wc.WaveCudaError as err:
        sys.stderr.write(err.message + "\n")
        return 2 if err.code in (wc.E_INVALID, wc.E_UNSUPPORTED) else 1
    mode = 1 if args.all_ones else 2 if args.rand_int else 3 if args.hpl else 0
    t = oracle.F16 if args.input_type == "f16" else oracle.BF16
    a_bits = oracle.make_input_bits(args.m, args.k, t, args.seed, 0, mode)
    b_bits = oracle.make_input_bits(args.n, args.k, t, args.seed, 1, mode)
    a, b = dev_bits(torch, a_bits), dev_bits(torch, b_bits)
    out_dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[args.c_type]
    c = torch.zeros(args.m * args.n, dtype=out_dt, device="cuda")  # runner.cpp:1659: C zero-filled before launch
    ws = torch.zeros(scratch + counters, dtype=torch.uint8, device="cuda") if scratch + counters else None
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        wc.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), ws.data_ptr() if ws is not None else 0, stream)

    try:
        times = [time_launches(torch, launch, args.warmup, args.iters) for _ in range(args.repeats)]
        wc.check_device_status()
    except wc.WaveCudaError as err:
        sys.stderr.write(err.message + "\n")
        return 1
    total_ms = median(times)
    per_launch_us = total_ms * 1e3 / args.iters
    tflops = 2.0 * args.m * args.n * args.k / per_launch_us * 1e-6
    name = args.kernel or ("gfx950_f16_streamk_gemm" if args.kernel_abi == "streamk" else "wmma_f16_matmul_tiled")
    props = torch.cuda.get_device_properties(0)
    print(f"device: {props.name} (sm_{props.major}{props.minor}a) sms={props.multi_processor_count}")
    print(f"kernel: {name}")
    print(f"shape: m={args.m} n={args.n} k={args.k} bm={args.bm} bn={args.bn} wave_m_tiles={args.wave_m_tiles} "
          f"wave_n_tiles={args.wave_n_tiles} wave_k_tiles={args.wave_k_tiles} wave_size={args.wave_size} input_type={args.input_type} "
          f"c_type={args.c_type} kernel_abi={args.kernel_abi} output_layout={layout} scale_layout=canonical "
          f"mxfp4_input_layout=canonical input_mode={MODE_NAMES[mode]}")
    print(f"output_contract: kernel={layout} final={layout} conversion=none")
    print(f"grid: {plan['grid']},1,1 block: 192,1,1 tile={plan['tile_m']}x{plan['tile_n']} "
          f"streamk_workers={plan['streamk_workers']} swapped={int(plan['swapped'])}")
    print(f"loop_trip_count: {args.k // (16 * args.wave_k_tiles) - 1}")
    print(f"iters: {args.iters}")
    print("timing_scope: gemm")
    print(f"total_ms: {total_ms:.3f}")
    print(f"per_launch_us: {per_launch_us:.3f}")
    if args.repeats > 1:
        print(f"median_per_launch_us: {per_launch_us:.3f}")
        print(f"best_per_launch_us: {min(times) * 1e3 / args.iters:.3f}")
    print(f"tflops: {tflops:.3f}")
    print(f"roofline_fraction: {tflops / 2250.0:.4f} (of 2250 TFLOP/s nominal dense bf16/f16)")
    if args.sustained_seconds > 0:
        sus_ms, sus_n = time_sustained(torch, launch, args.sustained_seconds)
        print(f"sustained_per_launch_us: {sus_ms * 1e3:.3f}")
        print(f"sustained_tflops: {2.0 * args.m * args.n * args.k / (sus_ms * 1e3) * 1e-6:.3f}")
        print(f"sustained_launches: {sus_n}")
    if not args.no_check:
        rows = None
        if args.check_rows and args.check_rows < args.m:
            rows = np.unique(np.linspace(0, args.m - 1, args.check_rows).astype(np.int32))
        t0 = time.perf_counter()
        exp = oracle.round_output(oracle.gemm_ref(a_bits, b_bits, t, rows=rows), args.c_type)
        cpu_s = time.perf_counter() - t0
        got = c.float().cpu().numpy()
        if layout in oracle.FRAGMENT_LAYOUTS:
            # reorderTilePackedOutput (runner.cpp:874-886): back to row-major through the index map
            wmma, wave = oracle.FRAGMENT_LAYOUTS[layout]
            mm, nn = oracle.tile_packed_fragment_coordinate(np.arange(args.m * args.n), args.m, args.n, args.bm, args.bn,
                                                            args.wave_m_tiles, args.wave_n_tiles, wmma, wave)
            logical = np.empty((args.m, args.n), got.dtype)
            logical[mm, nn] = got
            got = logical
        else:
            got = got.reshape(args.m, args.n) if layout == "row-major" else got.reshape(args.n, args.m).T
        if rows is not None:
            got = got[rows]
        diff = np.abs(got.astype(np.float64) - exp.astype(np.float64))
        rel = 2.0 ** -7 if args.c_type == "bf16" else 1.0e-3  # one bf16 ulp; the reference never stores bf16
        limit = 1.0e-2 + rel * np.abs(exp.astype(np.float64))
        bad = np.argwhere(~(diff <= limit))
        if bad.size:
            r, col = bad[0]
            m = int(rows[r]) if rows is not None else int(r)
            sys.stderr.write(f"output_check: failed m={m} n={int(col)} expected={exp[r, col]:.6f} got={got[r, col]:.6f} "
                             f"abs_diff={diff[r, col]:.6f} tolerance={limit[r, col]:.6f}\n")
            return 1
        worst = int(np.argmax(diff))
        print(f"output_check: passed mode=strict layout={layout} elements={diff.size} "
              f"max_abs_diff={float(diff.reshape(-1)[worst]):.6f} index={worst}")
        print(f"cpu_reference_s: {cpu_s:.3f}")
        print(f"cpu_cores: {oracle.host_threads()}")
    if plan["streamk_workers"] > 0:
        left = ws[scratch:].cpu().numpy().view(np.int32)
        nz = np.flatnonzero(left)
        if nz.size:
            sys.stderr.write(f"Stream-K counter {int(nz[0])} did not reset: {int(left[nz[0]])}\n")
            return 2
        print("streamk_counter_check: passed")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
