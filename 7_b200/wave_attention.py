"""Host-side mirror of the reference's attention interfaces on top of the CUDA
backend: the operator-level signature of
integrations/tlx/workloads/amd_fa_wave.py:1671-1682
(`attention(q, k, v, sm_scale=None, causal=False, *, out=None)`, rank-4
contiguous (B, H, N, D) tensors) and the input generators of the calibrate
runners (tools/wave-fa-calibrate/wave-fa-gfx950-runner.cpp:188-202,
python/mlir/dialects/wave_attention.py:225-245).

There is no CPU implementation of attention here.
"""
from __future__ import annotations

import math

import numpy as np

from . import wave_cuda as wc
from .wave_matmul import deterministic_random_values, input_bits

HEAD_DIM = 128   # wave_flash_attention.py: the production kernel's only head dimension (others run zero-padded)
BLOCK_M = 256    # query rows per workgroup (wave_flash_attention.py:23)


def make_runner_inputs(batch: int, heads: int, sequence: int, *, seed: int = 0, input_scale: int = 1,
                       io_type: str = "bf16", head_dim: int = HEAD_DIM):
    """Q, K (x0.125*input_scale) and V (x0.25) from LCG streams 0, 1, 2, rounded
    to the I/O type, shaped [B*H, S, 128] (wave-fa-gfx950-runner.cpp:410-413);
    `head_dim` other than the reference's 128 is an extension."""
    n = batch * heads * sequence * head_dim
    shape = (batch * heads, sequence, head_dim)
    q = deterministic_random_values(n, seed=seed, stream=0, scale=0.125 * input_scale)
    k = deterministic_random_values(n, seed=seed, stream=1, scale=0.125 * input_scale)
    v = deterministic_random_values(n, seed=seed, stream=2, scale=0.25)
    return tuple(input_bits(x, io_type).reshape(shape) for x in (q, k, v))


def generate_flash_attention_f32_inputs(block_m: int, head_dim: int, seq_n: int, *, random_seed: int = 0):
    """Inputs of the toy kernel `flash_attention_f32` as f16 bit patterns
    (python/mlir/dialects/wave_attention.py:225-245; C++ twin
    tools/wave-fa-calibrate/wave-fa-calibrate-runner.cpp:183-206): Q [block_m, d]
    from LCG stream 0 x0.0625, multiplied by log2(e)/sqrt(d) in double precision
    and rounded straight to f16; K and V [seq_n, d] from streams 1 (x0.0625) and
    2 (x0.125)."""
    q = deterministic_random_values(block_m * head_dim, seed=random_seed, stream=0, scale=0.0625)
    k = deterministic_random_values(seq_n * head_dim, seed=random_seed, stream=1, scale=0.0625)
    v = deterministic_random_values(seq_n * head_dim, seed=random_seed, stream=2, scale=0.125)
    scale = math.log2(math.e) / math.sqrt(head_dim)
    f16 = lambda x: np.asarray(x, np.float64).astype(np.float16).view(np.uint16)
    return (f16(q.astype(np.float64) * scale).reshape(block_m, head_dim), f16(k).reshape(seq_n, head_dim),
            f16(v).reshape(seq_n, head_dim))


def flops(batch: int, heads: int, sequence: int, head_dim: int = HEAD_DIM, causal: bool = False) -> float:
    """4*B*H*S^2*D (wave_flash_attention.py:138-139); for causal, the unmasked pairs only."""
    pairs = sequence * (sequence + 1) / 2 if causal else float(sequence) * sequence
    return 4.0 * batch * heads * head_dim * pairs


_F32_MIN_NORMAL = 1.1754943508222875e-38


def attention(q, k, v, sm_scale: float | None = None, causal: bool = False, *, qk_max_abs: float | None = None,
              out=None, lse=None):
    """Flash-attention forward on CUDA tensors of shape (B, H, N, D), bf16 or
    f16, contiguous, same device.  `sm_scale` defaults to 1/sqrt(D) and may be
    any finite number, as in the reference.
    `qk_max_abs`, a bound on the absolute values in q and k, selects the
    fixed-reference softmax of the reference's operator
    (integrations/tlx/workloads/amd_fa_wave.py:1671-1696): no running row
    maximum; None keeps the adaptive one.  `out` may alias `q` only in the sense
    of being a distinct tensor of the same shape; returns `out`."""
    import torch

    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k and v must be rank-4 (B, H, N, D) tensors")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("q, k and v must be CUDA tensors: this backend has no CPU path")
    if k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[3] != k.shape[3]:
        raise ValueError("q, k and v must agree on batch, heads and head_dim; k and v on sequence")
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k and v must share dtype bf16 or f16")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("q, k and v must be contiguous")
    B, H, Nq, D = q.shape
    Nk = k.shape[2]
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must match q in shape and dtype and be contiguous")
    # amd_fa_wave.py:1582-1611 (_resolve_softmax_reference): any finite scale,
    # the bound checked against |scale|.
    scale = 1.0 / math.sqrt(D) if sm_scale is None else float(sm_scale)
    if not math.isfinite(scale):
        raise ValueError("sm_scale must be finite")
    if qk_max_abs is not None and not (math.isfinite(qk_max_abs) and qk_max_abs > 0):
        raise ValueError("qk_max_abs must be finite and greater than zero")
    bound = 0.0 if qk_max_abs is None else float(qk_max_abs)
    # The kernels take a positive scale.  softmax(-|s| q.k) is softmax(|s| (-q).k),
    # and negating 16-bit floats is exact; with scale 0 every visible key weighs
    # the same, which is what zero queries give at any scale (the bound then has
    # nothing left to bound).
    if abs(scale) < _F32_MIN_NORMAL:  # zero, or a scale the f32 arithmetic would flush to zero
        q, scale, bound = torch.zeros_like(q), 1.0, 0.0
    elif scale < 0.0:
        q, scale = -q, -scale
    desc = wc.fa_desc(B, H, Nq, Nk, D, scale=scale, causal=causal,
                      io_type=wc.BF16 if q.dtype == torch.bfloat16 else wc.F16, qk_max_abs=bound)
    try:
        wc.fa_validate(desc)
    except wc.WaveCudaError as err:
        raise ValueError(err.message) from None
    wc.flash_attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                           lse.data_ptr() if lse is not None else 0, torch.cuda.current_stream().cuda_stream)
    return out


def run_toy_attention_f32(q_bits: np.ndarray, k_bits: np.ndarray, v_bits: np.ndarray) -> np.ndarray:
    """The reference's toy kernel `flash_attention_f32`
    (python/mlir/dialects/wave_attention.py:18, 225-278): one [block_m, d] f16
    Q tile already multiplied by log2(e)/sqrt(d), [seq_n, d] f16 K and V, f32
    output, probabilities 2^(s - max).  A softmax scale of ln 2 turns the
    backend's exp2(scale*log2(e)*s) into exactly that."""
    q, k, v = (np.ascontiguousarray(x, np.uint16) for x in (q_bits, k_bits, v_bits))
    desc = wc.fa_desc(1, 1, q.shape[-2], k.shape[-2], q.shape[-1], scale=math.log(2.0), io_type=wc.F16, out_f32=True)
    out = np.zeros(q.shape[-2:], np.float32)
    wc.flash_attention_fwd_host(desc, q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data)
    wc.check_device_status()
    return out


def run_attention_host(q_bits: np.ndarray, k_bits: np.ndarray, v_bits: np.ndarray, batch: int, heads: int, *,
                       sm_scale: float | None = None, causal: bool = False, io_type: str = "bf16") -> np.ndarray:
    """Host-buffer form: [B*H, S, D] 16-bit patterns in, the same out."""
    q, k, v = (np.ascontiguousarray(x, np.uint16) for x in (q_bits, k_bits, v_bits))
    BH, Sq, D = q.shape
    if BH != batch * heads:
        raise ValueError("leading dimension must be batch*heads")
    desc = wc.fa_desc(batch, heads, Sq, k.shape[1], D, scale=float(sm_scale or 0.0), causal=causal,
                      io_type=wc.TYPE_BY_NAME[io_type])
    out = np.zeros_like(q)
    wc.flash_attention_fwd_host(desc, q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data)
    wc.check_device_status()
    return out
