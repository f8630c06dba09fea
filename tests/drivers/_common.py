"""Shared plumbing of the command-line checkers in this directory.

These tools mirror the reference's example driver and calibrate tools flag for
flag, run the kernels through libwave_cuda.so (C ABI) and check the result with
the CPU oracle.  They are checkers: they live under tests/ because they import
the oracle, which product code never does.  torch provides device memory only.
"""
from __future__ import annotations

import importlib
import os
import statistics
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load():
    import torch
    if not torch.cuda.is_available():
        sys.stderr.write("no CUDA device: this backend has no CPU fallback\n")
        raise SystemExit(1)
    from oracle import oracle
    oracle.build()
    wc = importlib.import_module("7_b200").wave_cuda
    wc.lib()
    return torch, wc, oracle


def dev_bits(torch, bits: np.ndarray):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def time_launches(torch, fn, warmup: int, iters: int) -> float:
    """Warm-up launches, then `iters` back-to-back launches between two events
    (the runner's loop, wave-matmul-calibrate-runner.cpp:1863-1879).  Returns
    total milliseconds."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def time_sustained(torch, fn, seconds: float, batch: int = 50):
    """Back-to-back launches for at least `seconds` of GPU time (the part
    settles at the clock its power cap allows only after a fraction of a
    second, so a short loop overstates what it holds); batches of launches
    between two events, the first quarter of the batches left out.  Returns
    (milliseconds per launch, launches timed)."""
    per = []
    total_ms = 0.0
    while total_ms < seconds * 1e3:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(batch):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        per.append(ms / batch)
        total_ms += ms
    kept = per[len(per) // 4:]
    return statistics.median(kept), len(kept) * batch


def median(values):
    return statistics.median(values)


IGNORED_AMD_FLAGS = [
    ("--cta-swizzle-xcds", 1), ("--use-buffer", 0), ("--use-dma-lds", 0), ("--matrix-intrinsic", 1),
    ("--target-waves", 1), ("--enable-split-barriers", 1), ("--multi-wave-specialize", 0),
    ("--coalesced-mfma-output", 0), ("--output-store-cache", 1), ("--kernel-profile", 1), ("--chip", 1),
    ("--wave-size", 1), ("--dynamic-lds-bytes", 1),
]


def add_ignored_flags(parser):
    """AMD-only controls of the reference tools: accepted so that existing
    command lines run, ignored with a one-line notice.  A flag the tool already
    defines for itself is left alone."""
    for flag, nargs in IGNORED_AMD_FLAGS:
        if flag in parser._option_string_actions:
            continue
        if nargs:
            parser.add_argument(flag, default=None, help="AMD-only; accepted and ignored")
        else:
            parser.add_argument(flag, action="store_true", help="AMD-only; accepted and ignored")


def note_ignored(args, handled=()):
    used = [flag for flag, _ in IGNORED_AMD_FLAGS if getattr(args, flag[2:].replace("-", "_")) not in (None, False)]
    used = [f for f in used if f != "--chip" and f not in handled]
    if used:
        sys.stderr.write("note: ignoring AMD-only flags on sm_100a: " + " ".join(used) + "\n")
