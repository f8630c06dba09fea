"""GPU parity of the tiled GEMM against the CPU oracle, through the C ABI.

Mirrors the reference's integration strategy (``--compare-cpu`` runs over a
shape/tiling/dtype/seed matrix, e.g. test/Integration/wave_mfma_per_wave_tiles.mlir:3-11
and wave_wmma_per_wave_tiles.mlir:10-48, and calibrate-runner runs that must
print ``output_check: passed``).
"""
import json
import os

import numpy as np
import pytest

from _util import device_out, env_knobs, out_to_f32, runner_tolerance_ok, to_device_bits

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def run_gemm(torch, wc, a_bits, b_bits, in_name, out_name, layout="row-major", streamk=1, ldc=0, kernel="pair",
             **knobs):
    # small shapes must still exercise the CTA-pair kernel when their knobs ask for 256 x 256 tiles
    with env_knobs(wc, WAVE_CUDA_GEMM_KERNEL=kernel):
        return _run_gemm(torch, wc, a_bits, b_bits, in_name, out_name, layout, streamk, ldc, **knobs)


def _run_gemm(torch, wc, a_bits, b_bits, in_name, out_name, layout="row-major", streamk=1, ldc=0, **knobs):
    M, K = a_bits.shape
    N = b_bits.shape[0]
    desc = wc.gemm_desc(M, N, K, in_type=wc.TYPE_BY_NAME[in_name], out_type=wc.TYPE_BY_NAME[out_name],
                        out_layout=wc.LAYOUT_BY_NAME[layout], streamk_workers=streamk, ldc=ldc, **knobs)
    a = to_device_bits(torch, a_bits)
    b = to_device_bits(torch, b_bits)
    ld = ldc or (N if layout == "row-major" else M)
    outer = M if layout == "row-major" else N
    c = device_out(torch, ld * outer, out_name)
    scratch, counters = wc.gemm_workspace_bytes(desc)
    ws = None
    if scratch + counters:
        ws = torch.zeros(scratch + counters, dtype=torch.uint8, device="cuda")
    wc.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), ws.data_ptr() if ws is not None else 0,
            torch.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    got = out_to_f32(torch, c).reshape(outer, ld)
    inner = N if layout == "row-major" else M
    got = got[:, :inner]
    logical = got if layout == "row-major" else got.T
    counters_np = None
    if ws is not None:
        counters_np = ws[scratch:].cpu().numpy().view(np.int32)
    return np.ascontiguousarray(logical), counters_np


def expected(oracle, a_bits, b_bits, in_name, out_name):
    t = oracle.F16 if in_name == "f16" else oracle.BF16
    return oracle.round_output(oracle.gemm_ref(a_bits, b_bits, t), out_name)


def lcg_inputs(oracle, M, N, K, in_name, seed):
    t = oracle.F16 if in_name == "f16" else oracle.BF16
    return (oracle.make_input_bits(M, K, t, seed, 0, oracle.MODE_LCG),
            oracle.make_input_bits(N, K, t, seed, 1, oracle.MODE_LCG))


def test_config1_matches_reference_golden(cuda, wc, oracle):
    """32x32x64 f16 -> f32, seed 7, bm=bn=2, wave-k-tiles=2: the reference's own
    --compare-cpu case.  LCG inputs make every partial sum exact, so the match
    is bit-for-bit against the reference's Python output."""
    with open(os.path.join(GOLDEN, "gemm_golden.json")) as f:
        cases = json.load(f)["cases"]
    case = next(c for c in cases if c["case"].get("M") == 32 and c["case"].get("K") == 64
                and c["case"].get("input_type", "f16") == "f16")
    a, b = lcg_inputs(oracle, 32, 32, 64, "f16", 7)
    got, _ = run_gemm(cuda, wc, a, b, "f16", "f32", bm=2, bn=2, wave_k_tiles=2)
    want = np.asarray(case["out"], np.float32).reshape(32, 32)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("M,N,K,in_name,out_name,layout,knobs", [
    (16, 16, 16, "f16", "f32", "row-major", dict(bn=1)),
    (32, 32, 64, "bf16", "f32", "row-major", dict(bm=2, bn=2, wave_k_tiles=2)),
    (32, 48, 32, "f16", "f32", "column-major", dict(wave_m_tiles=2, wave_n_tiles=3, wave_k_tiles=2, bn=1)),
    (128, 256, 64, "f16", "f16", "row-major", dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),
    (256, 512, 256, "bf16", "bf16", "row-major", dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),
    (144, 80, 48, "f16", "f32", "row-major", dict(bn=1)),
    (144, 80, 48, "bf16", "bf16", "column-major", dict(bn=1)),
    (400, 272, 208, "f16", "f16", "column-major", dict(bn=1, wave_n_tiles=17)),
    (1024, 1024, 512, "bf16", "f32", "row-major", dict(bm=4, bn=8, wave_m_tiles=2, wave_n_tiles=2)),
    (512, 384, 1040, "f16", "f32", "row-major", dict(bm=2, bn=4, wave_n_tiles=2, wave_k_tiles=5)),
    (16, 1024, 512, "bf16", "f32", "row-major", dict(bn=1)),
    (16, 1024, 512, "bf16", "bf16", "column-major", dict(bn=1)),
    (64, 4096, 256, "f16", "f16", "row-major", dict(bm=4, bn=1)),
    # CTA-pair kernel (256 x 256 tiles): requested tile >= 256 in both directions
    (256, 256, 64, "f16", "f32", "row-major", dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)),
    (512, 768, 256, "bf16", "bf16", "row-major", dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)),
    (1024, 1024, 1040, "bf16", "f32", "column-major", dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)),
    (400, 272, 208, "f16", "f16", "row-major", dict(bm=1, bn=1, wave_m_tiles=25, wave_n_tiles=17)),
    (2304, 2048, 512, "f16", "f32", "row-major", dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4, cta_group_m=3)),
])
def test_lcg_inputs_bit_exact(cuda, wc, oracle, M, N, K, in_name, out_name, layout, knobs):
    """Reference LCG inputs are multiples of 0.25 in [-2, 2]: all partial sums
    are exact in f32, so any summation order must give the oracle's bits."""
    a, b = lcg_inputs(oracle, M, N, K, in_name, seed=M + N + K)
    got, _ = run_gemm(cuda, wc, a, b, in_name, out_name, layout, **knobs)
    want = expected(oracle, a, b, in_name, out_name)
    assert got.shape == want.shape
    assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"


@pytest.mark.parametrize("M,N,K,in_name,out_name,dist,scale", [
    (256, 256, 512, "f16", "f16", "uniform", 1.0),
    (512, 768, 2048, "bf16", "bf16", "normal", 2048 ** -0.5),
    (1024, 512, 4096, "f16", "f32", "uniform", 1.0),
    (16, 2048, 8192, "bf16", "f32", "normal", 8192 ** -0.5),
])
def test_random_inputs_within_runner_tolerance(cuda, wc, oracle, M, N, K, in_name, out_name, dist, scale):
    """Tolerance of the reference runner, |d| <= 1e-2 + 1e-3*|exp|
    (wave-matmul-calibrate-runner.cpp:907), plus mean absolute error <= 1e-3."""
    t = oracle.F16 if in_name == "f16" else oracle.BF16
    a = oracle.baseline_inputs((M, K), dist, 11, 0, t, scale=1.0 if dist == "uniform" else 1.0)
    b = oracle.baseline_inputs((N, K), dist, 11, 1, t, scale=scale)
    knobs = dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4) if M % 128 == 0 and N % 256 == 0 else dict(bn=1)
    got, _ = run_gemm(cuda, wc, a, b, in_name, out_name, **knobs)
    want = expected(oracle, a, b, in_name, out_name)
    ok, worst, nbad = runner_tolerance_ok(got, want, out_name)
    assert ok, f"{nbad} elements out of tolerance, worst abs diff {worst}"
    assert float(np.mean(np.abs(got - want))) <= 1e-3


@pytest.mark.parametrize("M,N,K,workers,knobs", [
    (256, 256, 1024, 3, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),
    (512, 512, 2048, 5, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),
    (384, 640, 1536, 37, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=2)),
    (16, 4096, 4096, 148, dict(bn=1)),
    (16, 28672, 8192, 0, dict(bn=1)),
    # auto mode, several full rounds of tiles plus a thin last one: whole tiles, then a Stream-K tail
    (2560, 4096, 512, 0, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),
    (2688, 1920, 1024, 0, dict(bm=4, bn=4, wave_m_tiles=1, wave_n_tiles=2)),
])
def test_streamk_matches_oracle_and_resets_counters(cuda, wc, oracle, M, N, K, workers, knobs):
    """Stream-K: fixed-order reduction makes two launches bit-identical, and the
    arrival counters are back to zero afterwards (the reference runner's
    streamk_counter_check, runner.cpp:1718-1733)."""
    a, b = lcg_inputs(oracle, M, N, K, "bf16", seed=5)
    got1, counters1 = run_gemm(cuda, wc, a, b, "bf16", "f32", streamk=workers, **knobs)
    want = expected(oracle, a, b, "bf16", "f32")
    assert np.array_equal(got1, want)
    assert counters1 is not None and not counters1.any()
    t = oracle.BF16
    a = oracle.baseline_inputs((M, K), "normal", 3, 0, t)
    b = oracle.baseline_inputs((N, K), "normal", 3, 1, t, scale=K ** -0.5)
    r1, _ = run_gemm(cuda, wc, a, b, "bf16", "f32", streamk=workers, **knobs)
    r2, _ = run_gemm(cuda, wc, a, b, "bf16", "f32", streamk=workers, **knobs)
    assert np.array_equal(r1, r2)
    ok, worst, nbad = runner_tolerance_ok(r1, expected(oracle, a, b, "bf16", "f32"))
    assert ok, f"{nbad} elements out of tolerance, worst {worst}"


PAIR_KNOBS = dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)


@pytest.mark.parametrize("M,N,K,out_name,layout,knobs", [
    (2560, 2560, 1024, "bf16", "row-major", PAIR_KNOBS),     # 100 tiles on 74 CTA pairs: 74 whole, 26 split over all pairs
    (2560, 2560, 1024, "f32", "row-major", PAIR_KNOBS),
    (768, 1024, 512, "bf16", "row-major", PAIR_KNOBS),       # 12 tiles, less than one round: every tile split
    (2560, 2560, 640, "bf16", "column-major", PAIR_KNOBS),   # computed as C^T, Stream-K tail on the swapped problem
    (2576, 2448, 576, "f16", "row-major", dict(bm=1, bn=1, wave_m_tiles=23, wave_n_tiles=17)),  # ragged edges on split tiles
    (8192, 1024, 1024, "bf16", "row-major", PAIR_KNOBS),     # an eighth of the 8192-column problem: 128 tiles, 54 in the tail
])
def test_pair_kernel_streamk_tail(cuda, wc, oracle, M, N, K, out_name, layout, knobs):
    """With streamk_workers = 0 and a workspace, the CTA-pair kernel deals the K
    iterations of a partly filled last round of tiles over all pairs.  LCG
    inputs: the oracle's bits whatever the grouping of the sum; the arrival
    counters are zero afterwards; two runs on random inputs are bit-identical
    (fixed reduction order); and the same with the tail treatment switched off."""
    in_name = "f16" if out_name == "f16" else "bf16"
    t = oracle.F16 if in_name == "f16" else oracle.BF16
    # the planner takes this treatment only where its cost model says it pays; here it is forced
    with env_knobs(wc, WAVE_CUDA_GEMM_STREAMK_TAIL="force", WAVE_CUDA_GEMM_PAIR_TILE_N="256"):
        with env_knobs(wc, WAVE_CUDA_GEMM_KERNEL="pair"):
            desc = wc.gemm_desc(M, N, K, in_type=wc.TYPE_BY_NAME[in_name], out_type=wc.TYPE_BY_NAME[out_name],
                                out_layout=wc.LAYOUT_BY_NAME[layout], streamk_workers=0, **knobs)
            plan = wc.gemm_plan(desc)
            assert (plan["tile_m"], plan["tile_n"]) == (256, 256) and plan["streamk_workers"] == plan["grid"] // 2 > 1, plan
        a, b = lcg_inputs(oracle, M, N, K, in_name, seed=M + 7)
        got, counters = run_gemm(cuda, wc, a, b, in_name, out_name, layout, streamk=0, **knobs)
        want = expected(oracle, a, b, in_name, out_name)
        assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"
        assert counters is not None and counters.size > 0 and not counters.any()
        a = oracle.baseline_inputs((M, K), "normal", 9, 0, t)
        b = oracle.baseline_inputs((N, K), "normal", 9, 1, t, scale=K ** -0.5)
        r1, _ = run_gemm(cuda, wc, a, b, in_name, out_name, layout, streamk=0, **knobs)
        r2, _ = run_gemm(cuda, wc, a, b, in_name, out_name, layout, streamk=0, **knobs)
    assert np.array_equal(r1, r2)
    ok, worst, nbad = runner_tolerance_ok(r1, expected(oracle, a, b, in_name, out_name), out_name)
    assert ok, f"{nbad} elements out of tolerance, worst {worst}"
    with env_knobs(wc, WAVE_CUDA_GEMM_STREAMK_TAIL="0"):
        whole, _ = run_gemm(cuda, wc, a, b, in_name, out_name, layout, streamk=0, **knobs)
    ok, worst, nbad = runner_tolerance_ok(r1, whole, out_name)
    assert ok, f"tail on/off differ beyond rounding: {nbad} elements, worst {worst}"


@pytest.mark.parametrize("width", [224, 192, 160])
@pytest.mark.parametrize("M,N,K,out_name,layout,knobs", [
    (512, 1280, 192, "bf16", "row-major", PAIR_KNOBS),
    (768, 1024, 128, "f32", "row-major", PAIR_KNOBS),          # last column tile narrower than the rest
    (1024, 768, 256, "bf16", "column-major", PAIR_KNOBS),      # computed as C^T
    (400, 464, 208, "f16", "row-major", dict(bm=1, bn=1, wave_m_tiles=25, wave_n_tiles=29)),  # ragged both ways
])
def test_pair_kernel_tile_widths(cuda, wc, oracle, width, M, N, K, out_name, layout, knobs):
    """The CTA-pair kernel's tiles may be any multiple of 32 columns in
    (128, 256] (the planner narrows them where that fills the last round of
    tiles); widths that are not a multiple of 64 end in a 32-column chunk that
    leaves by per-thread stores.  LCG inputs, bit-exact."""
    in_name = "f16" if out_name == "f16" else "bf16"
    a, b = lcg_inputs(oracle, M, N, K, in_name, seed=width + M)
    with env_knobs(wc, WAVE_CUDA_GEMM_PAIR_TILE_N=width):
        with env_knobs(wc, WAVE_CUDA_GEMM_KERNEL="pair"):
            plan = wc.gemm_plan(wc.gemm_desc(M, N, K, in_type=wc.TYPE_BY_NAME[in_name],
                                             out_type=wc.TYPE_BY_NAME[out_name],
                                             out_layout=wc.LAYOUT_BY_NAME[layout], **knobs))
            assert (plan["tile_m"], plan["tile_n"]) == (256, width), plan
        got, _ = run_gemm(cuda, wc, a, b, in_name, out_name, layout, **knobs)
    want = expected(oracle, a, b, in_name, out_name)
    assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"


def test_planner_narrows_tiles_for_column_shards(cuda, wc):
    """An eighth of the 8192-column problem (column-major C, so the kernel sees
    C^T: 1024 rows by 8192 columns) is 1.73 rounds of 256-column tiles on 74 CTA
    pairs but exactly two full rounds of 224-column ones; a quarter keeps 256
    (its sparse last round runs as half-width items), and so do half of it and
    the whole problem."""
    if cuda.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the expected plans are those of a 148-SM part")
    for n_local, want in ((1024, 224), (2048, 256), (4096, 256), (8192, 256)):
        d = wc.gemm_desc(8192, n_local, 8192, in_type=wc.BF16, out_type=wc.BF16, out_layout=wc.COL_MAJOR,
                         streamk_workers=0, **PAIR_KNOBS)
        plan = wc.gemm_plan(d)
        assert (plan["tile_m"], plan["tile_n"], plan["swapped"]) == (256, want, True), (n_local, plan)


@pytest.mark.parametrize("kernel", ["pair", "single"])
@pytest.mark.parametrize("M,N,K,out_name,ldc,knobs", [
    (512, 768, 256, "bf16", 0, PAIR_KNOBS),
    (1024, 256, 320, "f16", 0, PAIR_KNOBS),
    (400, 272, 208, "f16", 0, dict(bm=1, bn=1, wave_m_tiles=25, wave_n_tiles=17)),   # ragged in both directions
    (1024, 512, 128, "bf16", 1536, PAIR_KNOBS),                                       # a column shard of a wider C
    (256, 2048, 192, "bf16", 0, dict(bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4)),
])
def test_column_major_16bit_runs_as_transposed_row_major(cuda, wc, oracle, M, N, K, out_name, ldc, knobs, kernel):
    """Column-major 16-bit C is computed as C^T = B * A^T so that it leaves
    through the TMA-store epilogue; the bits must be the oracle's, the same as
    without the operand swap, and a shard written with ldc must leave the rest
    of the wider C untouched."""
    in_name = "f16" if out_name == "f16" else "bf16"
    a, b = lcg_inputs(oracle, M, N, K, in_name, seed=M + N)
    want = expected(oracle, a, b, in_name, out_name)
    got, _ = run_gemm(cuda, wc, a, b, in_name, out_name, "column-major", ldc=ldc, kernel=kernel, **knobs)
    assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"
    with env_knobs(wc, WAVE_CUDA_GEMM_COL_SWAP="0"):
        plain, _ = run_gemm(cuda, wc, a, b, in_name, out_name, "column-major", ldc=ldc, kernel=kernel, **knobs)
    assert np.array_equal(plain, want)
    if ldc:
        desc = wc.gemm_desc(M, N, K, in_type=wc.TYPE_BY_NAME[in_name], out_type=wc.TYPE_BY_NAME[out_name],
                            out_layout=wc.COL_MAJOR, ldc=ldc, **knobs)
        da, db = to_device_bits(cuda, a), to_device_bits(cuda, b)
        c = device_out(cuda, ldc * N, out_name)
        with env_knobs(wc, WAVE_CUDA_GEMM_KERNEL=kernel):
            wc.gemm(desc, da.data_ptr(), db.data_ptr(), c.data_ptr(), 0, cuda.cuda.current_stream().cuda_stream)
        wc.check_device_status()
        full = out_to_f32(cuda, c).reshape(N, ldc)
        assert np.array_equal(full[:, :M].T, want) and np.isnan(full[:, M:]).all()


@pytest.mark.parametrize("layout", ["tile-packed-mfma64", "tile-packed-wmma32", "tile-packed-mfma32"])
@pytest.mark.parametrize("M,N,K,out_name,streamk,knobs", [
    (64, 96, 32, "f32", 1, dict(bm=2, bn=2, wave_m_tiles=2, wave_n_tiles=3)),
    (256, 512, 128, "bf16", 1, dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)),   # CTA-pair kernel
    (384, 256, 1024, "f16", 7, dict(bm=2, bn=4, wave_m_tiles=3, wave_n_tiles=4)),   # Stream-K
])
def test_tile_packed_fragment_layouts(cuda, wc, oracle, layout, M, N, K, out_name, streamk, knobs):
    """Tile-packed C with each tile in the AMD accumulator-fragment order the
    reference's timed runner validates (wave-matmul-calibrate-runner.cpp:809-836,
    888-988); LCG inputs, bit-exact."""
    a_bits, b_bits = lcg_inputs(oracle, M, N, K, "f16", seed=K + 1)
    desc = wc.gemm_desc(M, N, K, out_type=wc.TYPE_BY_NAME[out_name], out_layout=wc.LAYOUT_BY_NAME[layout],
                        streamk_workers=streamk, **knobs)
    a, b = to_device_bits(cuda, a_bits), to_device_bits(cuda, b_bits)
    c = device_out(cuda, M * N, out_name)
    scratch, counters = wc.gemm_workspace_bytes(desc)
    ws = cuda.zeros(scratch + counters, dtype=cuda.uint8, device="cuda") if scratch + counters else None
    with env_knobs(wc, WAVE_CUDA_GEMM_KERNEL="pair"):
        wc.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), ws.data_ptr() if ws is not None else 0,
                cuda.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    got = out_to_f32(cuda, c)
    want = oracle.layout_output(expected(oracle, a_bits, b_bits, "f16", out_name), layout, knobs.get("bm", 1),
                                knobs.get("bn", 1), knobs.get("wave_m_tiles", 1), knobs.get("wave_n_tiles", 1))
    assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"


def test_pair_kernel_is_selected_for_large_tiles(cuda, wc):
    plan = wc.gemm_plan(wc.gemm_desc(8192, 8192, 8192, bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4, in_type=wc.BF16))
    assert (plan["tile_m"], plan["tile_n"]) == (256, 256) and plan["grid"] % 2 == 0
    plan = wc.gemm_plan(wc.gemm_desc(8192, 8192, 8192, bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4, in_type=wc.BF16))
    assert (plan["tile_m"], plan["tile_n"]) == (128, 256)
    # equal fill of the last round either way (3.46 rounds): the pair kernel's higher rate wins
    plan = wc.gemm_plan(wc.gemm_desc(4096, 4096, 4096, bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4))
    assert (plan["tile_m"], plan["tile_n"]) == (256, 256) and plan["grid"] % 2 == 0
    # one round of tiles either way: the one-CTA kernel
    plan = wc.gemm_plan(wc.gemm_desc(2048, 2048, 4096, bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4))
    assert (plan["tile_m"], plan["tile_n"]) == (128, 256)


@pytest.mark.parametrize("M,N,K,in_name,out_name,layout", [
    (256, 256, 64, "f16", "f32", "row-major"),
    (512, 768, 256, "bf16", "bf16", "row-major"),
    (1024, 1152, 1040, "bf16", "f32", "column-major"),
    (400, 272, 208, "f16", "f16", "row-major"),
    (2304, 2048, 512, "f16", "f32", "row-major"),
])
def test_narrow_pair_tile_bit_exact(cuda, wc, oracle, M, N, K, in_name, out_name, layout):
    """The 256 x 128 tile of the CTA-pair kernel (only on request: WAVE_CUDA_GEMM_KERNEL=pair128)."""
    a, b = lcg_inputs(oracle, M, N, K, in_name, seed=M + N + K)
    knobs = dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4) if M % 256 == 0 and N % 256 == 0 else \
        dict(bm=1, bn=1, wave_m_tiles=M // 16, wave_n_tiles=N // 16)
    if N == 1152:  # ragged against the wide tile, whole against the narrow one
        knobs = dict(bm=1, bn=1, wave_m_tiles=16, wave_n_tiles=72)
    got, _ = run_gemm(cuda, wc, a, b, in_name, out_name, layout, kernel="pair128", **knobs)
    want = expected(oracle, a, b, in_name, out_name)
    assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"


@pytest.mark.parametrize("split", ["1", "0"])
@pytest.mark.parametrize("M,N,K,layout", [
    (2560, 2560, 128, "row-major"),     # 100 tiles on 74 CTA pairs: the last 26 run as 52 half-width items
    (768, 1024, 192, "column-major"),   # 12 tiles: all of them split
    (2304, 2048, 64, "row-major"),      # 72 tiles: one well-filled round, nothing to split
    (2576, 2448, 80, "row-major"),      # ragged edges in both directions on split tiles
])
def test_pair_kernel_split_tail(cuda, wc, oracle, M, N, K, layout, split):
    """A sparsely filled last round of 256 x 256 tiles runs as half-width work
    items; the result must be the oracle's bits with the split on and off."""
    a, b = lcg_inputs(oracle, M, N, K, "bf16", seed=M + K)
    knobs = dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4) if M % 256 == 0 and N % 256 == 0 else \
        dict(bm=1, bn=1, wave_m_tiles=23 if M == 2576 else 16, wave_n_tiles=17 if N == 2448 else 16)
    with env_knobs(wc, WAVE_CUDA_GEMM_SPLIT_TAIL=split):
        got, _ = run_gemm(cuda, wc, a, b, "bf16", "f32", layout, **knobs)
    want = expected(oracle, a, b, "bf16", "f32")
    assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"


def test_pair_kernel_random_inputs(cuda, wc, oracle):
    t = oracle.BF16
    M, N, K = 1024, 768, 4096
    a = oracle.baseline_inputs((M, K), "normal", 21, 0, t, scale=K ** -0.5)
    b = oracle.baseline_inputs((N, K), "normal", 21, 1, t, scale=1.0)
    got, _ = run_gemm(cuda, wc, a, b, "bf16", "bf16", bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)
    ok, worst, nbad = runner_tolerance_ok(got, expected(oracle, a, b, "bf16", "bf16"), "bf16")
    assert ok, f"{nbad} elements out of tolerance, worst abs diff {worst}"


@pytest.mark.parametrize("M,N,K,out_name,streamk,knobs", [
    (64, 96, 32, "f32", 1, dict(bm=2, bn=2, wave_m_tiles=2, wave_n_tiles=3)),
    (32, 32, 64, "f16", 1, dict(bm=2, bn=2, wave_k_tiles=2)),
    (256, 512, 128, "bf16", 1, dict(bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4)),   # CTA-pair kernel
    (384, 256, 1024, "f32", 7, dict(bm=2, bn=4, wave_m_tiles=3, wave_n_tiles=4)),   # Stream-K
    (16, 256, 64, "f32", 1, dict(bn=1, wave_n_tiles=2)),                            # skinny M, not swapped
])
def test_tile_packed_output(cuda, wc, oracle, M, N, K, out_name, streamk, knobs):
    """Tile-packed C in the order the reference's Python reference emits it
    (wave_matmul.py:1025-1028, 1106-1139); LCG inputs, bit-exact."""
    a_bits, b_bits = lcg_inputs(oracle, M, N, K, "f16", seed=K)
    desc = wc.gemm_desc(M, N, K, out_type=wc.TYPE_BY_NAME[out_name], out_layout=wc.TILE_PACKED,
                        streamk_workers=streamk, **knobs)
    a, b = to_device_bits(cuda, a_bits), to_device_bits(cuda, b_bits)
    c = device_out(cuda, M * N, out_name)
    scratch, counters = wc.gemm_workspace_bytes(desc)
    ws = cuda.zeros(scratch + counters, dtype=cuda.uint8, device="cuda") if scratch + counters else None
    with env_knobs(wc, WAVE_CUDA_GEMM_KERNEL="pair"):
        wc.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), ws.data_ptr() if ws is not None else 0,
                cuda.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    want = oracle.layout_output(expected(oracle, a_bits, b_bits, "f16", out_name), "tile-packed", knobs.get("bm", 1),
                                knobs.get("bn", 2), knobs.get("wave_m_tiles", 1), knobs.get("wave_n_tiles", 1))
    assert np.array_equal(out_to_f32(cuda, c), want)


def test_ldc_writes_column_shard_in_place(cuda, wc, oracle):
    """A rank's N-column shard written straight into a wider row-major C."""
    M, N, K, ldc = 128, 64, 128, 256
    a, b = lcg_inputs(oracle, M, N, K, "f16", seed=1)
    got, _ = run_gemm(cuda, wc, a, b, "f16", "f32", ldc=ldc, bn=1)
    assert np.array_equal(got, expected(oracle, a, b, "f16", "f32"))


def test_host_buffer_call(cuda, wc, oracle):
    M, N, K = 256, 128, 320
    a, b = lcg_inputs(oracle, M, N, K, "bf16", seed=9)
    c = np.full((M, N), np.nan, np.float32)
    desc = wc.gemm_desc(M, N, K, in_type=wc.BF16, out_type=wc.F32)
    wc.gemm_host(desc, a.ctypes.data, b.ctypes.data, c.ctypes.data)
    wc.check_device_status()
    assert np.array_equal(c, expected(oracle, a, b, "bf16", "f32"))


@pytest.mark.parametrize("layout,out_name", [("row-major", "f32"), ("column-major", "bf16")])
def test_host_buffer_call_pipelined(cuda, wc, oracle, layout, out_name):
    """Large host-buffer calls are pipelined by column blocks of C (B blocks in,
    C blocks out, overlapped with compute); the result must not depend on it."""
    M, N, K = 2048, 8192, 2048 if out_name == "f32" else 4096
    a, b = lcg_inputs(oracle, M, N, K, "bf16", seed=17)
    dt = np.float32 if out_name == "f32" else np.uint16
    c = np.zeros(M * N, dt)
    desc = wc.gemm_desc(M, N, K, bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=4, in_type=wc.BF16,
                        out_type=wc.TYPE_BY_NAME[out_name], out_layout=wc.LAYOUT_BY_NAME[layout])
    wc.gemm_host(desc, a.ctypes.data, b.ctypes.data, c.ctypes.data)
    wc.check_device_status()
    got = c if out_name == "f32" else oracle.from_bits(c, oracle.BF16)
    got = got.reshape(M, N) if layout == "row-major" else got.reshape(N, M).T
    assert np.array_equal(got, expected(oracle, a, b, "bf16", out_name))


@pytest.mark.parametrize("M,N,K", [(512, 768, 256), (2048, 8192, 4096)])
def test_host_buffer_call_with_device_resident_a(cuda, wc, oracle, pkg, M, N, K):
    """One rank's part of an N-column-sharded GEMM whose operands live in host
    memory: the replicated A is already on the device (on more than one GPU it
    arrives by an all-gather of row blocks; one rank here), B and the
    column-major bf16 C block travel through the host-buffer call, one-piece and
    pipelined sizes."""
    import importlib
    sh = importlib.import_module("7_b200.sharding")
    a, b = lcg_inputs(oracle, M, N, K, "bf16", seed=23)
    a_host = cuda.from_numpy(a.view(np.int16)).pin_memory()
    b_host = cuda.from_numpy(b.view(np.int16)).pin_memory()
    c_host = cuda.zeros(N * M, dtype=cuda.int16).pin_memory()
    a_dev = cuda.empty((M, K), dtype=cuda.int16, device="cuda")
    desc = wc.gemm_desc(M, N, K, bm=4, bn=4, wave_m_tiles=4, wave_n_tiles=4, in_type=wc.BF16, out_type=wc.BF16,
                        out_layout=wc.COL_MAJOR, streamk_workers=0)
    sh.sharded_gemm_host(wc, desc, a_dev, a_host, b_host, c_host, None, 0, 1, cuda.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    got = oracle.from_bits(c_host.numpy().view(np.uint16), oracle.BF16).reshape(N, M).T
    assert np.array_equal(got, expected(oracle, a, b, "bf16", "bf16"))


@pytest.mark.parametrize("M,N,K,out_name,layout,ldc,width", [
    (512, 768, 256, "bf16", "row-major", 0, 0),
    (1024, 512, 320, "bf16", "column-major", 0, 0),       # computed as C^T
    (2048, 512, 128, "f16", "column-major", 2304, 0),     # a column block inside a wider C
    (400, 464, 208, "f16", "row-major", 0, 0),            # ragged edges: the copies clip like the TMA store
    (768, 1024, 192, "bf16", "row-major", 0, 224),        # 224-column tiles: the 32-column remainder chunk
])
def test_multi_output_writes_every_target(cuda, wc, oracle, M, N, K, out_name, layout, ldc, width):
    """wave_cuda_gemm_multi_output: the result lands in every target buffer (on
    one GPU: three local buffers stand in for peer GPUs' copies of C), bit for
    bit what wave_cuda_gemm writes, and nothing outside the block is touched."""
    in_name = "f16" if out_name == "f16" else "bf16"
    a_bits, b_bits = lcg_inputs(oracle, M, N, K, in_name, seed=M + 3)
    knobs = PAIR_KNOBS if M % 256 == 0 and N % 256 == 0 else dict(bm=1, bn=1, wave_m_tiles=M // 16, wave_n_tiles=N // 16)
    desc = wc.gemm_desc(M, N, K, in_type=wc.TYPE_BY_NAME[in_name], out_type=wc.TYPE_BY_NAME[out_name],
                        out_layout=wc.LAYOUT_BY_NAME[layout], ldc=ldc, **knobs)
    a, b = to_device_bits(cuda, a_bits), to_device_bits(cuda, b_bits)
    ld = ldc or (N if layout == "row-major" else M)
    outer = M if layout == "row-major" else N
    inner = N if layout == "row-major" else M
    targets = [device_out(cuda, ld * outer, out_name) for _ in range(3)]
    env = dict(WAVE_CUDA_GEMM_KERNEL="pair")
    if width:
        env["WAVE_CUDA_GEMM_PAIR_TILE_N"] = width
    with env_knobs(wc, **env):
        wc.gemm_multi_output(desc, a.data_ptr(), b.data_ptr(), [t.data_ptr() for t in targets],
                             cuda.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    want = expected(oracle, a_bits, b_bits, in_name, out_name)
    for t in targets:
        full = out_to_f32(cuda, t).reshape(outer, ld)
        got = full[:, :inner] if layout == "row-major" else full[:, :inner].T
        assert np.array_equal(got, want), f"max abs diff {np.nanmax(np.abs(got - want))}"
        assert np.isnan(full[:, inner:]).all()


def test_multi_output_refuses_what_it_cannot_do(cuda, wc):
    x = cuda.zeros(256 * 256, dtype=cuda.float16, device="cuda")
    c = cuda.zeros(256 * 256, dtype=cuda.float32, device="cuda")
    with pytest.raises(wc.WaveCudaError) as err:  # f32 output has no TMA-store epilogue
        wc.gemm_multi_output(wc.gemm_desc(256, 256, 256, **PAIR_KNOBS), x.data_ptr(), x.data_ptr(),
                             [c.data_ptr(), c.data_ptr()])
    assert err.value.code == wc.E_UNSUPPORTED
    with pytest.raises(wc.WaveCudaError) as err:
        wc.gemm_multi_output(wc.gemm_desc(256, 256, 256, out_type=wc.F16, **PAIR_KNOBS), x.data_ptr(), x.data_ptr(), [])
    assert err.value.code == wc.E_INVALID


def test_name_based_launch_facade(cuda, wc, oracle):
    """Same call shape as the reference runner: look a kernel up by name, then
    launch with an array of pointers to the argument values
    (wave-matmul-calibrate-runner.cpp:1790-1791, 1846-1862)."""
    import ctypes as C
    M, N, K = 64, 64, 128
    a_bits, b_bits = lcg_inputs(oracle, M, N, K, "f16", seed=2)
    a, b = to_device_bits(cuda, a_bits), to_device_bits(cuda, b_bits)
    c = device_out(cuda, M * N, "f32")
    desc = wc.gemm_desc(M, N, K, wave_k_tiles=2)
    fn = C.c_void_p()
    wc.check(wc.lib().wave_cuda_module_get_function(b"wmma_f16_matmul_tiled", C.byref(desc), C.byref(fn)))
    pa, pb, pc = C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()), C.c_void_p(c.data_ptr())
    trip = C.c_int(K // (16 * 2) - 1)
    args = (C.c_void_p * 4)(C.addressof(pa), C.addressof(pb), C.addressof(pc), C.addressof(trip))
    wc.check(wc.lib().wave_cuda_launch(fn, args, None))
    wc.check_device_status()
    wc.lib().wave_cuda_function_release(fn)
    assert np.array_equal(out_to_f32(cuda, c).reshape(M, N), expected(oracle, a_bits, b_bits, "f16", "f32"))
