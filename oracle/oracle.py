"""ctypes front end of the CPU oracle (``wave_oracle.c``) and of the compiled
reference (``_ref/libwave_ref.so``), plus small NumPy restatements.

TEST INFRASTRUCTURE ONLY.  Only the test suite, the smoke test and the
benchmark's CPU-baseline leg may import this module; the product path (the
wave_cuda library and its Python host mirror) never does and has no CPU
fallback.

Parity status: pinned -- see the header of ``wave_oracle.c`` for the reference
functions each routine restates and how they are checked.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
F16, BF16 = 0, 1
MODE_LCG, MODE_ALL_ONES, MODE_RAND_INT, MODE_HPL, MODE_HALVES = range(5)

_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def reference_root() -> str:
    """Where the reference checkout lies, if there is one: the
    WAVE_REFERENCE_ROOT environment variable, else a directory named
    `reference` beside this repository (the Makefile uses the same rule)."""
    return os.environ.get("WAVE_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference shim when a checkout is present)."""
    lib = os.path.join(HERE, "libwave_oracle.so")
    src = os.path.join(HERE, "wave_oracle.c")
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B"], check=True, capture_output=True)
    elif os.path.isdir(reference_root()) and not os.path.exists(
        os.path.join(HERE, "_ref", "libwave_ref.so")
    ):
        subprocess.run(["make", "-C", HERE, "ref"], check=True, capture_output=True)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "libwave_oracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.wo_f32_to_bf16.argtypes = [C.c_float]
        L.wo_f32_to_bf16.restype = C.c_uint16
        L.wo_f32_to_f16.argtypes = [C.c_float]
        L.wo_f32_to_f16.restype = C.c_uint16
        L.wo_bf16_to_f32.argtypes = [C.c_uint16]
        L.wo_bf16_to_f32.restype = C.c_float
        L.wo_f16_to_f32.argtypes = [C.c_uint16]
        L.wo_f16_to_f32.restype = C.c_float
        L.wo_round_array.argtypes = [_f32p, _u16p, C.c_size_t, C.c_int]
        L.wo_widen_array.argtypes = [_u16p, _f32p, C.c_size_t, C.c_int]
        L.wo_lcg_values.argtypes = [_f32p, C.c_size_t, C.c_int, C.c_int, C.c_float]
        L.wo_make_input_bits.argtypes = [_u16p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.wo_make_input_bits.restype = C.c_int
        L.wo_fa_input_bits.argtypes = [_u16p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_float]
        L.wo_gemm_element.argtypes = [_u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.wo_gemm_element.restype = C.c_float
        L.wo_gemm_ref.argtypes = [_u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_void_p, C.c_int, _f32p, C.c_int]
        L.wo_gemm_ref.restype = C.c_int
        L.wo_fa_ref.argtypes = [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                C.c_double, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                C.c_int, _f32p, C.c_void_p, C.c_int]
        L.wo_fa_ref.restype = C.c_int
        L.wo_fa_sample_heads.argtypes = [C.c_int, _i32p]
        L.wo_fa_sample_heads.restype = C.c_int
        L.wo_fa_sample_rows.argtypes = [C.c_int, _i32p]
        L.wo_fa_sample_rows.restype = C.c_int
        _lib = L
    return _lib


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:  # pragma: no cover
        return os.cpu_count() or 1


# --------------------------------------------------------------------------
# conversions
# --------------------------------------------------------------------------

def to_bits(values, dtype: int) -> np.ndarray:
    """f32 array -> uint16 bit patterns (RNE), f16 or bf16."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(v.shape, np.uint16)
    lib().wo_round_array(v.reshape(-1), out.reshape(-1), v.size, dtype)
    return out


def from_bits(bits, dtype: int) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(b.shape, np.float32)
    lib().wo_widen_array(b.reshape(-1), out.reshape(-1), b.size, dtype)
    return out


def np_to_bits(values, dtype: int) -> np.ndarray:
    """NumPy-only restatement of the two roundings (cross-check of the C code)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    if dtype == F16:
        return v.astype(np.float16).view(np.uint16)
    b = v.view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def np_from_bits(bits, dtype: int) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np.uint16)
    if dtype == F16:
        return b.view(np.float16).astype(np.float32)
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_output(values, out_type: str) -> np.ndarray:
    """Final rounding of the f32 accumulators to the C element type, returned
    as f32 values (wave_matmul.py:1142-1143, runner.cpp:738-744)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    if out_type == "f32":
        return v
    t = F16 if out_type == "f16" else BF16
    return from_bits(to_bits(v, t), t)


# --------------------------------------------------------------------------
# generators
# --------------------------------------------------------------------------

def lcg_values(count: int, seed: int, stream: int, scale: float = 0.25) -> np.ndarray:
    out = np.empty(count, np.float32)
    lib().wo_lcg_values(out, count, seed, stream, scale)
    return out


def np_lcg_values(count: int, seed: int, stream: int, scale: float = 0.25) -> np.ndarray:
    """Pure-Python loop restating wave_matmul.py:828-836 (small counts only)."""
    state = (seed ^ ((stream + 1) * 0x9E3779B9)) & 0xFFFFFFFF
    vals = []
    for _ in range(count):
        state = (1664525 * state + 1013904223) & 0xFFFFFFFF
        vals.append((((state >> 24) % 17) - 8) * scale)
    return np.asarray(vals, np.float64)


def make_input_bits(rows: int, k: int, dtype: int, seed: int, stream: int, mode: int) -> np.ndarray:
    out = np.empty((rows, k), np.uint16)
    rc = lib().wo_make_input_bits(out.reshape(-1), rows * k, k, dtype, seed, stream, mode)
    if rc != 0:
        raise ValueError("bad generator arguments")
    return out


def fa_input_bits(count: int, dtype: int, seed: int, stream: int, scale: float) -> np.ndarray:
    out = np.empty(count, np.uint16)
    lib().wo_fa_input_bits(out, count, dtype, seed, stream, scale)
    return out


def baseline_inputs(shape, dist: str, seed: int, stream: int, dtype: int, scale: float = 1.0) -> np.ndarray:
    """Seeded synthetic inputs with the distributions the benchmark configs
    name (uniform[-1,1) or N(0,1)*scale), from a counter-based Philox stream,
    rounded to f16/bf16.  Not a reference generator: the reference only has the
    LCG / rand_int / HPL modes above."""
    rng = np.random.Generator(np.random.Philox(key=[seed, stream]))
    if dist == "uniform":
        v = rng.random(shape, dtype=np.float32) * 2.0 - 1.0
    elif dist == "normal":
        v = rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)
    else:
        raise ValueError(dist)
    return to_bits(v, dtype)


# --------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------

def gemm_ref(a_bits, b_bits, dtype: int, rows=None, threads: int | None = None) -> np.ndarray:
    """f32-accumulate, k-ascending reference.  a_bits [M,K], b_bits [N,K]
    (B stored as its transpose, as the reference does).  Returns f32
    [nrows, N] -- unrounded accumulators."""
    a = np.ascontiguousarray(a_bits, np.uint16)
    b = np.ascontiguousarray(b_bits, np.uint16)
    M, K = a.shape
    N, K2 = b.shape
    assert K == K2
    if rows is None:
        rp, nrows = None, M
    else:
        rows = np.ascontiguousarray(rows, np.int32)
        rp, nrows = rows.ctypes.data_as(C.c_void_p), rows.size
    out = np.empty((nrows, N), np.float32)
    rc = lib().wo_gemm_ref(a.reshape(-1), b.reshape(-1), M, N, K, dtype, rp, nrows,
                           out.reshape(-1), threads or host_threads())
    if rc != 0:
        raise RuntimeError(f"wo_gemm_ref failed: {rc}")
    return out


def gemm_element(a_bits, b_bits, dtype: int, m: int, n: int) -> float:
    a = np.ascontiguousarray(a_bits, np.uint16)
    b = np.ascontiguousarray(b_bits, np.uint16)
    return float(lib().wo_gemm_element(a.reshape(-1), b.reshape(-1), a.shape[1], dtype, m, n))


def np_gemm_ref(a_bits, b_bits, dtype: int) -> np.ndarray:
    """NumPy restatement: one f32 multiply and one f32 add per k, k ascending."""
    a = np_from_bits(a_bits, dtype)
    b = np_from_bits(b_bits, dtype)
    acc = np.zeros((a.shape[0], b.shape[0]), np.float32)
    for k in range(a.shape[1]):
        acc += a[:, k, None] * b[None, :, k]
    return acc


def layout_output(c_rowmajor: np.ndarray, layout: str, BM: int = 1, BN: int = 1, wave_m_tiles: int = 1,
                  wave_n_tiles: int = 1) -> np.ndarray:
    """Logical [M,N] -> the flat physical buffer (wave_matmul.py:1025-1041).
    Tile-packed: 16x16 tiles appended in the loop order of
    compute_wmma_f16_matmul_reference_buffer (wave_matmul.py:1106-1139):
    workgroup rows, workgroup columns, waves (m_wave = id // BN, n_wave = id % BN),
    per-wave tile rows, per-wave tile columns; row-major inside a tile."""
    if layout == "row-major":
        return np.ascontiguousarray(c_rowmajor).reshape(-1)
    if layout == "column-major":
        return np.ascontiguousarray(c_rowmajor.T).reshape(-1)
    if layout == "tile-packed":
        M, N = c_rowmajor.shape
        m_blocks = (M // 16) // (BM * wave_m_tiles)
        n_blocks = (N // 16) // (BN * wave_n_tiles)
        out = []
        for wg_m in range(m_blocks):
            for wg_n in range(n_blocks):
                for wave in range(BM * BN):
                    m_wave, n_wave = wave // BN, wave % BN
                    for i in range(wave_m_tiles):
                        for j in range(wave_n_tiles):
                            mt = wg_m * BM * wave_m_tiles + m_wave * wave_m_tiles + i
                            nt = wg_n * BN * wave_n_tiles + n_wave * wave_n_tiles + j
                            out.append(c_rowmajor[mt * 16:(mt + 1) * 16, nt * 16:(nt + 1) * 16].reshape(-1))
        return np.concatenate(out)
    if layout in FRAGMENT_LAYOUTS:
        M, N = c_rowmajor.shape
        wmma, wave_size = FRAGMENT_LAYOUTS[layout]
        idx = np.arange(M * N)
        m, n = tile_packed_fragment_coordinate(idx, M, N, BM, BN, wave_m_tiles, wave_n_tiles, wmma, wave_size)
        return np.ascontiguousarray(c_rowmajor)[m, n]
    raise ValueError(layout)


# layout name -> (WMMA accumulator layout?, wave size) of the reference runner
FRAGMENT_LAYOUTS = {"tile-packed-mfma64": (False, 64), "tile-packed-wmma32": (True, 32),
                    "tile-packed-mfma32": (False, 32)}


def tile_packed_fragment_coordinate(index, M: int, N: int, BM: int, BN: int, wave_m_tiles: int, wave_n_tiles: int,
                                    wmma: bool, wave_size: int):
    """Packed index -> logical (m, n) of the timed runner's tile-packed output,
    restating getOutputCoordinate / getAccumulatorRow / makeTilePackedOutputPlan
    (wave-matmul-calibrate-runner.cpp:771-836): tiles in workgroup -> wave ->
    per-wave-tile order, the 256 values of a tile as lane * values_per_lane + v
    with column lane % 16 and row (lane // 16) + 2 v (WMMA, wave32) or
    (lane // 16) * values_per_lane + v (MFMA).  `index` may be an array."""
    index = np.asarray(index)
    values_per_lane = 256 // wave_size
    m_tiles_per_block = BM * wave_m_tiles
    n_tiles_per_block = BN * wave_n_tiles
    n_blocks = N // (16 * n_tiles_per_block)
    wave_elements = wave_m_tiles * wave_n_tiles * 256
    cta_elements = BM * BN * wave_elements
    cta, cta_rem = index // cta_elements, index % cta_elements
    wg_m, wg_n = cta // n_blocks, cta % n_blocks
    wave_id, wave_rem = cta_rem // wave_elements, cta_rem % wave_elements
    tile_id, slot = wave_rem // 256, wave_rem % 256
    m_wave, n_wave = wave_id // BN, wave_id % BN
    lane, lane_value = slot // values_per_lane, slot % values_per_lane
    if wmma:
        m_lane = lane // 16 + 2 * lane_value
    else:
        m_lane = (lane // 16) * values_per_lane + lane_value
    m_tile = wg_m * m_tiles_per_block + m_wave * wave_m_tiles + tile_id // wave_n_tiles
    n_tile = wg_n * n_tiles_per_block + n_wave * wave_n_tiles + tile_id % wave_n_tiles
    return m_tile * 16 + m_lane, n_tile * 16 + lane % 16


# --------------------------------------------------------------------------
# flash attention
# --------------------------------------------------------------------------

def fa_ref(q_bits, k_bits, v_bits, dtype: int, scale: float, causal: bool = False,
           exp2_mode: bool = False, heads=None, rows=None, threads: int | None = None,
           want_lse: bool = False):
    """f64 attention rows.  q [BH,Sq,D], k/v [BH,Sk,D] bit patterns.
    Returns f32 [nheads, nrows, D] (and the f64 log-sum-exp when asked)."""
    q = np.ascontiguousarray(q_bits, np.uint16)
    k = np.ascontiguousarray(k_bits, np.uint16)
    v = np.ascontiguousarray(v_bits, np.uint16)
    BH, Sq, D = q.shape
    Sk = k.shape[1]
    hp = rp = None
    nh, nr = BH, Sq
    if heads is not None:
        heads = np.ascontiguousarray(heads, np.int32)
        hp, nh = heads.ctypes.data_as(C.c_void_p), heads.size
    if rows is not None:
        rows = np.ascontiguousarray(rows, np.int32)
        rp, nr = rows.ctypes.data_as(C.c_void_p), rows.size
    out = np.empty((nh, nr, D), np.float32)
    lse = np.empty((nh, nr), np.float64) if want_lse else None
    rc = lib().wo_fa_ref(q.reshape(-1), k.reshape(-1), v.reshape(-1), dtype, BH, Sq, Sk, D,
                         float(scale), int(causal), int(exp2_mode), hp, nh, rp, nr,
                         out.reshape(-1), lse.ctypes.data_as(C.c_void_p) if want_lse else None,
                         threads or host_threads())
    if rc != 0:
        raise RuntimeError(f"wo_fa_ref failed: {rc}")
    return (out, lse) if want_lse else out


def fa_sample_heads(total_heads: int) -> np.ndarray:
    out = np.empty(4, np.int32)
    n = lib().wo_fa_sample_heads(total_heads, out)
    return out[:n].copy()


def fa_sample_rows(sequence: int) -> np.ndarray:
    out = np.empty(max(512, 8), np.int32)
    n = lib().wo_fa_sample_rows(sequence, out)
    return out[:n].copy()


# --------------------------------------------------------------------------
# compiled reference (present only when built from a reference checkout)
# --------------------------------------------------------------------------

_ref = None


def ref_lib():
    """The reference's own runner code as a shared object, or None."""
    global _ref
    if _ref is None:
        path = os.path.join(HERE, "_ref", "libwave_ref.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.wave_ref_make_input_bits.argtypes = [_u16p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        R.wave_ref_make_input_bits.restype = C.c_int
        R.wave_ref_gemm_rows.argtypes = [_u16p, _u16p, C.c_int, C.c_int, C.c_int, C.c_int,
                                         C.c_void_p, C.c_int, _f32p, C.c_int]
        R.wave_ref_round_output.argtypes = [C.c_double, C.c_int]
        R.wave_ref_round_output.restype = C.c_double
        R.wave_ref_streamk_scratch_bytes.argtypes = [C.c_int]
        R.wave_ref_streamk_scratch_bytes.restype = C.c_size_t
        R.wave_ref_streamk_counter_elements.argtypes = [C.c_int, C.c_int]
        R.wave_ref_streamk_counter_elements.restype = C.c_size_t
        R.wave_ref_output_coordinate.argtypes = [C.c_int] * 9 + [_i32p]
        R.wave_ref_fa_input_bits.argtypes = [_u16p, C.c_size_t, C.c_int, C.c_int, C.c_float]
        R.wave_ref_fa_rows.argtypes = [_u16p, _u16p, _u16p, C.c_int, C.c_int, C.c_int, _i32p, C.c_int,
                                       _i32p, C.c_int, _f32p, C.c_int]
        R.wave_ref_fa_sample_heads.argtypes = [C.c_int, C.c_int, _i32p]
        R.wave_ref_fa_sample_heads.restype = C.c_int
        R.wave_ref_fa_sample_rows.argtypes = [C.c_int, _i32p]
        R.wave_ref_fa_sample_rows.restype = C.c_int
        _ref = R
    return _ref


def ref_make_input_bits(rows: int, k: int, dtype: int, seed: int, stream: int, mode: int) -> np.ndarray:
    out = np.empty((rows, k), np.uint16)
    ref_lib().wave_ref_make_input_bits(out.reshape(-1), rows, k, dtype, seed, stream, mode)
    return out


def ref_output_coordinate(M: int, N: int, BM: int, BN: int, wave_m_tiles: int, wave_n_tiles: int, wmma: bool,
                          wave_size: int, index: int):
    out = np.zeros(2, np.int32)
    ref_lib().wave_ref_output_coordinate(M, N, BM, BN, wave_m_tiles, wave_n_tiles, int(wmma), wave_size, index, out)
    return int(out[0]), int(out[1])


def ref_gemm_rows(a_bits, b_bits, dtype: int, rows=None, threads: int | None = None) -> np.ndarray:
    a = np.ascontiguousarray(a_bits, np.uint16)
    b = np.ascontiguousarray(b_bits, np.uint16)
    M, K = a.shape
    N = b.shape[0]
    if rows is None:
        rp, nrows = None, M
    else:
        rows = np.ascontiguousarray(rows, np.int32)
        rp, nrows = rows.ctypes.data_as(C.c_void_p), rows.size
    out = np.empty((nrows, N), np.float32)
    ref_lib().wave_ref_gemm_rows(a.reshape(-1), b.reshape(-1), M, N, K, dtype, rp, nrows,
                                 out.reshape(-1), threads or host_threads())
    return out


def ref_fa_rows(q_bits, k_bits, v_bits, batch: int, heads: int, sequence: int, head_list, row_list,
                threads: int | None = None) -> np.ndarray:
    hl = np.ascontiguousarray(head_list, np.int32)
    rl = np.ascontiguousarray(row_list, np.int32)
    out = np.empty((hl.size, rl.size, 128), np.float32)
    ref_lib().wave_ref_fa_rows(np.ascontiguousarray(q_bits, np.uint16).reshape(-1),
                               np.ascontiguousarray(k_bits, np.uint16).reshape(-1),
                               np.ascontiguousarray(v_bits, np.uint16).reshape(-1),
                               batch, heads, sequence, hl, hl.size, rl, rl.size,
                               out.reshape(-1), threads or host_threads())
    return out
