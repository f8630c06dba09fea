"""Host-side mirror of the reference's GEMM builder/driver interface
(python/mlir/dialects/wave_matmul.py, examples/wave/wmma_matmul_tiled.py) on
top of the CUDA backend: the same configuration fields, validation rules and
messages, deterministic input generators and Stream-K partition arithmetic,
with the kernel launch going through the C ABI instead of MLIR + ROCm.

There is no CPU implementation of the GEMM here: `run_matmul` needs a CUDA
device and raises without one.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import wave_cuda as wc

STREAMK_PARTIAL_SLOTS_PER_WORKER = 2  # wave_matmul.py:156-159


# --------------------------------------------------------------------------
# deterministic inputs (wave_matmul.py:828-852, 966-994; runner.cpp:681-716)
# --------------------------------------------------------------------------
def deterministic_random_values(count: int, *, seed: int, stream: int, scale: float = 0.25) -> np.ndarray:
    """state0 = seed ^ ((stream+1)*0x9E3779B9); state = 1664525*state + 1013904223
    (mod 2**32); value = (((state >> 24) % 17) - 8) * scale.  Vectorised through
    the closed form state_i = a^i * state0 + c * (1 + a + ... + a^(i-1))."""
    a, c = np.uint32(1664525), np.uint32(1013904223)
    state0 = np.uint32((seed ^ ((stream + 1) * 0x9E3779B9)) & 0xFFFFFFFF)
    with np.errstate(over="ignore"):
        powers = np.multiply.accumulate(np.full(count, a, dtype=np.uint32), dtype=np.uint32)  # a^1 .. a^count
        geo = np.empty(count, np.uint32)                                           # 1 + a + ... + a^(i-1)
        geo[0] = 1
        if count > 1:
            geo[1:] = np.uint32(1) + np.add.accumulate(powers[:-1], dtype=np.uint32)
        states = powers * state0 + geo * c
    buckets = ((states >> np.uint32(24)) % np.uint32(17)).astype(np.int32) - 8
    return buckets.astype(np.float32) * np.float32(scale)


def round_bf16_bits(values) -> np.ndarray:
    """wave_matmul.py:843-846: add 0x7FFF + lsb, keep the top 16 bits."""
    bits = np.ascontiguousarray(values, np.float32).view(np.uint32)
    return ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def round_f16_bits(values) -> np.ndarray:
    """wave_matmul.py:839-840 (struct 'e' packing is round-to-nearest-even)."""
    return np.ascontiguousarray(values, np.float32).astype(np.float16).view(np.uint16)


def input_bits(values, input_type: str) -> np.ndarray:
    if input_type == "bf16":
        return round_bf16_bits(values)
    if input_type == "f16":
        return round_f16_bits(values)
    raise ValueError(f"input_type must be one of f16, bf16; got {input_type}")


def generate_wmma_f16_matmul_inputs(M: int, N: int, K: int, *, input_type: str = "f16", random_data: bool = False,
                                    random_seed: int = 0) -> tuple[np.ndarray, np.ndarray]:
    """A (M x K, stream 0) and B (N x K, stream 1) as 16-bit patterns.  Without
    `random_data` the first half of each buffer is 1.0 and the second 2.0
    (wave_matmul.py:985-989)."""
    if random_data:
        a = deterministic_random_values(M * K, seed=random_seed, stream=0)
        b = deterministic_random_values(N * K, seed=random_seed, stream=1)
    else:
        a = np.where(np.arange(M * K) < (M * K) // 2, 1.0, 2.0).astype(np.float32)
        b = np.where(np.arange(N * K) < (N * K) // 2, 1.0, 2.0).astype(np.float32)
    return input_bits(a, input_type).reshape(M, K), input_bits(b, input_type).reshape(N, K)


# --------------------------------------------------------------------------
# Stream-K partition arithmetic (wave_matmul.py:88-165)
# --------------------------------------------------------------------------
def streamk_worker_interval(total_iterations: int, workers: int, worker: int) -> tuple[int, int]:
    if total_iterations <= 0:
        raise ValueError("total_iterations must be positive")
    if not 1 <= workers <= total_iterations:
        raise ValueError("workers must be in [1, total_iterations]")
    if not 0 <= worker < workers:
        raise ValueError("worker must be in [0, workers)")
    q, r = divmod(total_iterations, workers)
    begin = worker * q + min(worker, r)
    return begin, begin + q + int(worker < r)


def streamk_owner_for_iteration(total_iterations: int, workers: int, iteration: int) -> int:
    if not 0 <= iteration < total_iterations:
        raise ValueError("iteration must be in [0, total_iterations)")
    q, r = divmod(total_iterations, workers)
    if q == 0:
        raise ValueError("workers must not exceed total_iterations")
    large_end = r * (q + 1)
    if iteration < large_end:
        return iteration // (q + 1)
    return r + (iteration - large_end) // q


def streamk_tile_contributors(tile: int, k_iterations: int, total_iterations: int, workers: int) -> tuple[int, int]:
    if k_iterations <= 0 or total_iterations % k_iterations:
        raise ValueError("k_iterations must divide total_iterations")
    if not 0 <= tile < total_iterations // k_iterations:
        raise ValueError("tile must be in [0, tile_count)")
    return (streamk_owner_for_iteration(total_iterations, workers, tile * k_iterations),
            streamk_owner_for_iteration(total_iterations, workers, (tile + 1) * k_iterations - 1))


def streamk_worker_segments(tile_count: int, k_iterations: int, workers: int, worker: int):
    """(tile, k_begin, k_end, scratch_slot or None) for each tile the worker
    touches; a contiguous interval has at most two partial tiles."""
    if tile_count <= 0 or k_iterations <= 0:
        raise ValueError("tile_count and k_iterations must be positive")
    begin, end = streamk_worker_interval(tile_count * k_iterations, workers, worker)
    segments, slot = [], 0
    for tile in range(begin // k_iterations, (end - 1) // k_iterations + 1):
        tb = tile * k_iterations
        kb, ke = max(begin, tb) - tb, min(end, tb + k_iterations) - tb
        whole = kb == 0 and ke == k_iterations
        segments.append((tile, kb, ke, None if whole else slot))
        slot += int(not whole)
    if slot > STREAMK_PARTIAL_SLOTS_PER_WORKER:
        raise AssertionError("contiguous worker interval has more than two boundaries")
    return tuple(segments)


def streamk_scratch_elements(workers: int, tile_elements: int = 256 * 256) -> int:
    if workers <= 0:
        raise ValueError("workers must be positive")
    return workers * STREAMK_PARTIAL_SLOTS_PER_WORKER * tile_elements


# --------------------------------------------------------------------------
# configuration
# --------------------------------------------------------------------------
@dataclass(frozen=True)
class MatmulConfig:
    """Fields of the reference's _MatmulConfig (wave_matmul.py:288-530) that
    this backend honours.  AMD-only controls (XCD swizzle, LDS DMA, MFMA
    variants, target waves) have no meaning here and are not carried."""
    M: int
    N: int
    K: int
    BM: int = 1
    BN: int = 1
    wave_m_tiles: int = 1
    wave_n_tiles: int = 1
    wave_k_tiles: int = 1
    input_type: str = "f16"
    output_type: str = "f32"
    output_layout: str = "row-major"
    cta_group_m: int = 1
    streamk_workers: int = 1
    ldc: int = 0

    def __post_init__(self):
        for name, table in (("input_type", ("f16", "bf16")), ("output_type", ("f32", "f16", "bf16")),
                            ("output_layout", ("row-major", "column-major", "tile-packed"))):
            if getattr(self, name) not in table:
                raise ValueError(f"{name} must be one of {', '.join(table)}; got {getattr(self, name)}")
        try:
            wc.gemm_validate(self.desc())
        except wc.WaveCudaError as err:
            raise ValueError(err.message) from None

    def desc(self) -> wc.GemmDesc:
        return wc.gemm_desc(self.M, self.N, self.K, bm=self.BM, bn=self.BN, wave_m_tiles=self.wave_m_tiles,
                            wave_n_tiles=self.wave_n_tiles, wave_k_tiles=self.wave_k_tiles,
                            in_type=wc.TYPE_BY_NAME[self.input_type], out_type=wc.TYPE_BY_NAME[self.output_type],
                            out_layout=wc.LAYOUT_BY_NAME[self.output_layout], cta_group_m=self.cta_group_m,
                            streamk_workers=self.streamk_workers, ldc=self.ldc)

    # geometry as the reference derives it (wave_matmul.py:426-444)
    @property
    def M_blocks(self) -> int:
        return (self.M // 16) // (self.BM * self.wave_m_tiles)

    @property
    def N_blocks(self) -> int:
        return (self.N // 16) // (self.BN * self.wave_n_tiles)

    @property
    def waves_per_workgroup(self) -> int:
        return self.BM * self.BN

    @property
    def total_elements(self) -> int:
        return self.M * self.N

    @property
    def trip_count(self) -> int:
        """The reference kernel's i32 argument: K/(k_tile*wave_k_tiles) - 1 (wave_matmul.py:6964)."""
        return self.K // (16 * self.wave_k_tiles) - 1

    def plan(self) -> dict:
        """Launch geometry chosen by the B200 backend (needs a CUDA device)."""
        return wc.gemm_plan(self.desc())

    def workspace_bytes(self) -> tuple[int, int]:
        return wc.gemm_workspace_bytes(self.desc())


_OUT_DTYPES = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}


def run_matmul(cfg: MatmulConfig, a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Runs the GEMM on the current CUDA device from host buffers and returns
    the flat output buffer in its physical layout (row-major m*N+n or
    column-major n*M+m, wave_matmul.py:1040); bf16 outputs come back as raw
    16-bit patterns."""
    a = np.ascontiguousarray(a_bits, np.uint16)
    b = np.ascontiguousarray(b_bits, np.uint16)
    if a.shape != (cfg.M, cfg.K) or b.shape != (cfg.N, cfg.K):
        raise ValueError(f"A must be {cfg.M}x{cfg.K} and B {cfg.N}x{cfg.K} (B is stored transposed)")
    ld = cfg.ldc or (cfg.M if cfg.output_layout == "column-major" else cfg.N)
    outer = cfg.N if cfg.output_layout == "column-major" else cfg.M
    out = np.zeros(ld * outer, _OUT_DTYPES[cfg.output_type])
    wc.gemm_host(cfg.desc(), a.ctypes.data, b.ctypes.data, out.ctypes.data)
    wc.check_device_status()
    return out
