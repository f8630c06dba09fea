#!/usr/bin/env python
"""Drop-in for the reference's flash-attention calibrate tool
(tools/wave-fa-calibrate/wave-fa-gfx950.py + wave-fa-gfx950-runner.cpp) on B200:
--batch --heads --sequence --qk-max-abs --seed --input-scale --check --zero-qk
--iters --warmup --repeats (wave-fa-gfx950.py:95-128), plus --causal, --scale and --head-dim, which
the reference's Wave kernel does not have.  Prints the runner's keys (`shape:`,
`grid:`, `per_launch_us:`, `tflops:`, `output_check: passed max_abs_diff=...`,
`median_per_launch_us:`, `median_tflops:`; wave-fa-gfx950-runner.cpp:465-481,
392; wave-fa-gfx950.py:297-298).  --check samples heads and rows exactly as the
runner does (runner:204-232) against the f64 reference, max-abs <= 3e-2.
"""
from __future__ import annotations

import argparse
import importlib
import math
import sys

import numpy as np

from _common import dev_bits, load, median, time_launches, time_sustained


def parse(argv):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--heads", type=int, default=1)
    p.add_argument("--sequence", type=int, default=256)
    p.add_argument("--qk-max-abs", type=float, default=None, help="use fixed softmax reference for |Q|,|K| <= VALUE")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--input-scale", type=int, default=1)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--repeats", type=int, default=1)
    p.add_argument("--sustained-seconds", type=float, default=0.0,
                   help="also time a back-to-back loop of at least this long (the clock the power cap allows)")
    p.add_argument("--check", action="store_true")
    p.add_argument("--zero-qk", action="store_true")
    p.add_argument("--causal", action="store_true")
    p.add_argument("--scale", type=float, default=0.0, help="softmax scale; 0 = 1/sqrt(head_dim)")
    p.add_argument("--head-dim", type=int, default=128, help="a multiple of 16 up to 128 (the reference: 128 only)")
    p.add_argument("--waves", type=int, default=None, help="AMD-only; accepted and ignored")
    p.add_argument("--threads", type=int, default=None, help="AMD-only; accepted and ignored")
    args = p.parse_args(argv)
    if args.qk_max_abs is not None:  # wave-fa-gfx950.py:70-78
        if not math.isfinite(args.qk_max_abs) or args.qk_max_abs <= 0:
            p.error("--qk-max-abs must be finite and positive")
        if args.qk_max_abs < args.input_scale:
            p.error("--qk-max-abs must cover the generated input range")
    return args


def main(argv=None) -> int:
    args = parse(sys.argv[1:] if argv is None else argv)
    if args.batch <= 0 or args.heads <= 0 or args.sequence <= 0 or args.sequence % 256:
        sys.stderr.write("batch and heads must be positive; sequence a positive multiple of 256\n")  # runner:142-161
        return 2
    torch, wc, oracle = load()
    wa = importlib.import_module("7_b200.wave_attention")
    D = args.head_dim
    q, k, v = wa.make_runner_inputs(args.batch, args.heads, args.sequence, seed=args.seed, input_scale=args.input_scale,
                                    head_dim=D)
    if args.zero_qk:
        q[:] = 0
        k[:] = 0
    dq, dk, dv = (dev_bits(torch, x) for x in (q, k, v))
    o = torch.zeros(q.shape, dtype=torch.bfloat16, device="cuda")
    desc = wc.fa_desc(args.batch, args.heads, args.sequence, args.sequence, D, scale=args.scale, causal=args.causal,
                      qk_max_abs=args.qk_max_abs or 0.0)
    try:
        wc.fa_validate(desc)
    except wc.WaveCudaError as err:  # the reference's builder raises here (wave-fa-gfx950.py:176-177)
        raise SystemExit(err.message) from err
    stream = torch.cuda.current_stream().cuda_stream

    def launch():
        wc.flash_attention_fwd(desc, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), o.data_ptr(), 0, stream)

    try:
        times = [time_launches(torch, launch, args.warmup, args.iters) for _ in range(args.repeats)]
        wc.check_device_status()
    except wc.WaveCudaError as err:
        sys.stderr.write(err.message + "\n")
        return 1
    us = [t * 1e3 / args.iters for t in times]
    full = wa.flops(args.batch, args.heads, args.sequence, D)  # the reference's formula, 4*B*H*S^2*D
    done = wa.flops(args.batch, args.heads, args.sequence, D, causal=args.causal)
    print(f"shape: B={args.batch} H={args.heads} N={args.sequence} D={D} causal={int(args.causal)}")
    print(f"grid: {args.sequence // 256},{args.batch * args.heads},1 block: 384,1,1 dynamic_lds=197888")
    for t in us:
        print(f"per_launch_us: {t:.3f}")
        print(f"tflops: {done / t * 1e-6:.3f}")
    if args.causal:
        print(f"tflops_full_square_formula: {full / median(us) * 1e-6:.3f}")
    if args.sustained_seconds > 0:
        sus_ms, sus_n = time_sustained(torch, launch, args.sustained_seconds, batch=10)
        print(f"sustained_per_launch_us: {sus_ms * 1e3:.3f}")
        print(f"sustained_tflops: {done / (sus_ms * 1e3) * 1e-6:.3f}")
        print(f"sustained_launches: {sus_n}")
    if args.check:
        heads, rows = oracle.fa_sample_heads(args.batch * args.heads), oracle.fa_sample_rows(args.sequence)
        scale = args.scale if args.scale > 0 else 1.0 / np.sqrt(float(D))
        want = oracle.fa_ref(q, k, v, oracle.BF16, scale, causal=args.causal, heads=heads, rows=rows)
        got = o.float().cpu().numpy()[np.ix_(heads, rows)]
        diff = np.abs(got.astype(np.float64) - want)
        worst = int(np.argmax(diff))
        if not diff.reshape(-1)[worst] <= 3.0e-2:
            sys.stderr.write(f"output_check: failed max_abs_diff={diff.reshape(-1)[worst]:.8f} index={worst}\n")
            return 1
        print(f"output_check: passed max_abs_diff={diff.reshape(-1)[worst]:.8f} index={worst}")
    print(f"median_per_launch_us: {median(us):.3f}")
    print(f"median_tflops: {done / median(us) * 1e-6:.3f}")
    print(f"roofline_fraction: {done / median(us) * 1e-6 / 2250.0:.4f} (of 2250 TFLOP/s nominal dense bf16)")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
