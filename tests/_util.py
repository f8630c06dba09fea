"""Helpers shared by the GPU parity tests: device buffers come from torch
(plumbing only); every compute call goes through the C ABI."""
from __future__ import annotations

import numpy as np


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


def runner_tolerance_ok(got: np.ndarray, exp: np.ndarray):
    """|got-exp| <= 1e-2 + 1e-3*|exp| for every element
    (tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp:907)."""
    diff = np.abs(got.astype(np.float64) - exp.astype(np.float64))
    limit = 1.0e-2 + 1.0e-3 * np.abs(exp.astype(np.float64))
    bad = ~(diff <= limit)  # catches NaN too
    return not bad.any(), float(np.nanmax(diff)) if diff.size else 0.0, int(bad.sum())
