"""Helpers shared by the GPU parity tests: device buffers come from torch
(plumbing only); every compute call goes through the C ABI."""
from __future__ import annotations

import contextlib
import os

import numpy as np


@contextlib.contextmanager
def env_knobs(wc, **knobs):
    """Sets WAVE_CUDA_* measurement knobs for the enclosed calls.  The library
    reads its environment once, so it is told to read it again on the way in
    and on the way out."""
    old = {k: os.environ.get(k) for k in knobs}
    os.environ.update({k: str(v) for k, v in knobs.items()})
    wc.reload_env()
    try:
        yield
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
        wc.reload_env()


def to_device_bits(torch, bits: np.ndarray):
    """uint16 bit patterns -> device int16 tensor holding the same bytes."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def device_out(torch, count: int, out_type: str):
    dt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[out_type]
    # poison so that unwritten elements are caught (the reference's ctypes
    # runner does the same: test/Integration/Inputs/wavec_wmma_matmul_ctypes_runner.py:80)
    return torch.full((count,), float("nan"), dtype=dt, device="cuda")


def out_to_f32(torch, t) -> np.ndarray:
    return t.float().cpu().numpy()


def runner_tolerance_ok(got: np.ndarray, exp: np.ndarray, out_type: str = "f32"):
    """|got-exp| <= 1e-2 + 1e-3*|exp| for every element
    (tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp:907).

    The reference only stores f32 or f16.  A bf16 result keeps 8 significant
    bits, so two correct f32 accumulations that differ in their last bits can
    round to neighbouring bf16 values; for bf16 the relative term is therefore
    one bf16 unit in the last place (2**-7), still inside the 1e-2 maximum
    relative error this backend is specified to."""
    diff = np.abs(got.astype(np.float64) - exp.astype(np.float64))
    rel = 2.0 ** -7 if out_type == "bf16" else 1.0e-3
    limit = 1.0e-2 + rel * np.abs(exp.astype(np.float64))
    bad = ~(diff <= limit)  # catches NaN too
    return not bad.any(), float(np.nanmax(diff)) if diff.size else 0.0, int(bad.sum())
