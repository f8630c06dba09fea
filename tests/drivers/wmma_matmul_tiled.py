#!/usr/bin/env python
"""Drop-in for the reference's examples/wave/wmma_matmul_tiled.py on B200.

Same flags for the part of the surface this backend carries
(examples/wave/wmma_matmul_tiled.py:271-341, 406-411): --m/--n/--k, --bm/--bn,
--wave-m-tiles/--wave-n-tiles/--wave-k-tiles, --input-type, --output-type,
--output-layout, --cta-group-m, --random-data, --seed, --compare-cpu,
--atol/--rtol.  Without --compare-cpu the C buffer is printed the way
mlir-runner prints a memref (`data = [...]`, examples/wave/common.py:300-306);
with it the buffer is compared element by element with the CPU reference
(math.isclose, atol = rtol = 1e-3, wmma_matmul_tiled.py:267-268, 580-597) and
the tool prints `CPU comparison passed: ...` or exits 1.
"""
from __future__ import annotations

import argparse
import math
import sys

import numpy as np

from _common import add_ignored_flags, load, note_ignored


def parse(argv):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--m", type=int, default=32)
    p.add_argument("--n", type=int, default=32)
    p.add_argument("--k", type=int, default=32)
    p.add_argument("--bm", type=int, default=1)
    p.add_argument("--bn", type=int, default=1)
    p.add_argument("--wave-m-tiles", type=int, default=1)
    p.add_argument("--wave-n-tiles", type=int, default=1)
    p.add_argument("--wave-k-tiles", type=int, default=1)
    p.add_argument("--input-type", choices=["f16", "bf16", "mxfp4"], default="f16")
    p.add_argument("--output-type", choices=["f32", "f16", "bf16"], default="f32")
    p.add_argument("--output-layout", choices=["automatic", "row-major", "column-major", "tile-packed"],
                   default="automatic")
    p.add_argument("--cta-group-m", type=int, default=1)
    p.add_argument("--streamk-workers", type=int, default=1)
    p.add_argument("--random-data", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--run", action="store_true")
    p.add_argument("--compare-cpu", action="store_true")
    p.add_argument("--atol", type=float, default=1e-3)
    p.add_argument("--rtol", type=float, default=1e-3)
    add_ignored_flags(p)
    return p.parse_args(argv)


def main(argv=None) -> int:
    args = parse(sys.argv[1:] if argv is None else argv)
    note_ignored(args)
    if args.input_type == "mxfp4":
        sys.stderr.write("mxfp4 inputs are outside this backend\n")
        return 2
    torch, wc, oracle = load()
    import importlib
    wm = importlib.import_module("7_b200.wave_matmul")
    layout = "row-major" if args.output_layout == "automatic" else args.output_layout
    random_data = args.random_data or args.compare_cpu  # wmma_matmul_tiled.py:620
    try:
        cfg = wm.MatmulConfig(args.m, args.n, args.k, BM=args.bm, BN=args.bn, wave_m_tiles=args.wave_m_tiles,
                              wave_n_tiles=args.wave_n_tiles, wave_k_tiles=args.wave_k_tiles,
                              input_type=args.input_type, output_type=args.output_type, output_layout=layout,
                              cta_group_m=args.cta_group_m,
                              streamk_workers=1)
    except ValueError as err:
        sys.stderr.write(f"{err}\n")
        return 2
    a, b = wm.generate_wmma_f16_matmul_inputs(args.m, args.n, args.k, input_type=args.input_type,
                                              random_data=random_data, random_seed=args.seed)
    out = wm.run_matmul(cfg, a, b)
    t = oracle.F16 if args.input_type == "f16" else oracle.BF16
    if args.output_type == "bf16":
        actual = oracle.from_bits(out, oracle.BF16)
    else:
        actual = out.astype(np.float32)
    if not args.compare_cpu:
        sys.stdout.write("data = \n[" + ",  ".join(repr(float(v)) for v in actual) + "]\n")
        return 0
    expected = oracle.layout_output(oracle.round_output(oracle.gemm_ref(a, b, t), args.output_type), layout, args.bm,
                                    args.bn, args.wave_m_tiles, args.wave_n_tiles)
    if actual.size != expected.size:
        sys.stderr.write(f"CPU comparison failed: length mismatch: gpu={actual.size} cpu={expected.size}\n")
        return 1
    worst = (0.0, 0, 0.0, 0.0)
    for index, (got, exp) in enumerate(zip(actual.tolist(), expected.tolist())):
        diff = abs(got - exp)
        if diff > worst[0]:
            worst = (diff, index, got, exp)
        if not math.isclose(got, exp, rel_tol=args.rtol, abs_tol=args.atol):
            sys.stderr.write(f"CPU comparison failed: element {index}: gpu={got} cpu={exp} abs_diff={diff}\n")
            return 1
    diff, index, got, exp = worst
    sys.stdout.write(f"CPU comparison passed: elements={actual.size} max_abs_diff={diff} at {index} ({got}, {exp})\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
