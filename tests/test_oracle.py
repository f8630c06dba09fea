"""Pins the CPU oracle: against the known-answer vectors of the reference's own
tests, against golden vectors produced by running the reference's Python
references (tests/golden/make_golden.py), against the reference's C++ runner
code compiled as a shared object (when built), and against an independent
NumPy restatement."""
import hashlib
import json
import os
import struct

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    with open(os.path.join(GOLDEN, name)) as f:
        return json.load(f)


def _sha(values32: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(values32, "<f4").tobytes()).hexdigest()


# ---------------------------------------------------------------- conversions
def test_f16_roundtrip_exhaustive(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    finite = ((bits >> 10) & 0x1F) != 0x1F
    vals = oracle.from_bits(bits, oracle.F16)
    assert np.array_equal(vals[finite], bits[finite].view(np.float16).astype(np.float32))
    assert np.array_equal(oracle.to_bits(vals[finite], oracle.F16), bits[finite])


def test_rounding_matches_numpy_restatement(oracle):
    rng = np.random.default_rng(0)
    v = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5, 6.0975e-5,
                  np.inf, -np.inf, 1.0009765625, 1.00048828125, 1.00146484375], np.float32)])
    for t in (oracle.F16, oracle.BF16):
        with np.errstate(over="ignore"):
            assert np.array_equal(oracle.to_bits(v, t), oracle.np_to_bits(v, t))
        b = oracle.to_bits(v, t)
        assert np.array_equal(oracle.from_bits(b, t), oracle.np_from_bits(b, t), equal_nan=True)


# ------------------------------------------------- reference C++ test vectors
# test/Integration/Inputs/wave_matmul_rand_int_test.cpp:29-49
RAND_INT_A = [-2, -2, 0, 0, 1, 0, 1, 2, -1, -2, 0, -1, -2, -2, 0]
RAND_INT_B = [2, -2, -0.0, 0, -1, 0, -1, 2, 1, -2, -0.0, -1, 2, -2, -0.0]
# test/Integration/Inputs/wave_matmul_rand_int_test.cpp:467-472
HPL_F16 = [0xb5dc, 0x33a1, 0xb028, 0xb61c, 0x2a95, 0x3581, 0xb509, 0xb583, 0xb537, 0xaaa8, 0x365c, 0xb48d, 0xa801,
           0x2b96, 0x304a]
HPL_BF16 = [0xbebb, 0x3e74, 0xbe05, 0xbec3, 0x3d53, 0x3eb0, 0xbea1, 0xbeb0, 0xbea7, 0xbd55, 0x3ecb, 0xbe92, 0xbd00,
            0x3d73, 0x3e09]


@pytest.mark.parametrize("t", ["F16", "BF16"])
def test_rand_int_known_answers(oracle, t):
    T = getattr(oracle, t)
    a = oracle.make_input_bits(3, 5, T, 0, 0, oracle.MODE_RAND_INT)
    again = oracle.make_input_bits(3, 5, T, 91, 0, oracle.MODE_RAND_INT)
    b = oracle.make_input_bits(3, 5, T, 0, 1, oracle.MODE_RAND_INT)
    assert np.array_equal(a, again), "rand_int must not depend on the seed"
    assert not np.array_equal(a, b), "A and B streams must differ"
    for bits, want in ((a, RAND_INT_A), (b, RAND_INT_B)):
        got = oracle.from_bits(bits, T).reshape(-1)
        want = np.asarray(want, np.float32)
        assert np.array_equal(got, want)
        assert np.array_equal(np.signbit(got), np.signbit(want))


@pytest.mark.parametrize("t,want", [("F16", HPL_F16), ("BF16", HPL_BF16)])
def test_hpl_known_answers(oracle, t, want):
    T = getattr(oracle, t)
    a = oracle.make_input_bits(3, 5, T, 0, 0, oracle.MODE_HPL)
    assert np.array_equal(a, oracle.make_input_bits(3, 5, T, 91, 0, oracle.MODE_HPL))
    assert np.array_equal(a, oracle.make_input_bits(3, 5, T, 0, 1, oracle.MODE_HPL)), "HPL A and B streams are equal"
    assert a.reshape(-1).tolist() == want


@pytest.mark.parametrize("t", ["F16", "BF16"])
def test_cpu_reference_known_answers(oracle, t):
    """wave_matmul_rand_int_test.cpp:70-105."""
    T = getattr(oracle, t)
    a = oracle.make_input_bits(2, 4, T, 0, 0, oracle.MODE_RAND_INT)
    b = oracle.make_input_bits(2, 4, T, 0, 1, oracle.MODE_RAND_INT)
    assert oracle.gemm_ref(a, b, T).reshape(-1).tolist() == [0, -2, 2, -2]
    a = oracle.make_input_bits(2, 4, T, 0, 0, oracle.MODE_HPL)
    b = oracle.make_input_bits(2, 4, T, 0, 1, oracle.MODE_HPL)
    c = oracle.gemm_ref(a, b, T)
    assert c[0, 0] > 0 and c[1, 1] > 0 and c[0, 1] == c[1, 0]


def test_all_ones_fill_pattern(oracle):
    """test/Integration/wave_wmma_tiled.mlir:19-46: with the non-random fill
    (first half 1.0, second half 2.0) C = K * a(i) * b(j): 32, 64 and 128 at K=32."""
    M = N = K = 32
    a = oracle.make_input_bits(M, K, oracle.F16, 0, 0, oracle.MODE_HALVES)
    b = oracle.make_input_bits(N, K, oracle.F16, 0, 1, oracle.MODE_HALVES)
    c = oracle.gemm_ref(a, b, oracle.F16)
    assert c[0, 0] == 32 and c[0, N - 1] == 64 and c[M - 1, 0] == 64 and c[M - 1, N - 1] == 128


# ----------------------------------------- values printed by the Python tests
def test_python_test_printed_values(oracle):
    """test/python/dialects/wave_matmul.py: `bf16-ref 256 32.0` (:1075) and
    `f16-ref-rounding -132.5625 -132.5` (:1080, first element where the f16
    result differs from the f32 one at 16x16x512, seed 91)."""
    a = oracle.make_input_bits(16, 32, oracle.BF16, 0, 0, oracle.MODE_HALVES)
    b = oracle.make_input_bits(16, 32, oracle.BF16, 0, 1, oracle.MODE_HALVES)
    c = oracle.gemm_ref(a, b, oracle.BF16)
    assert c.size == 256 and c.reshape(-1)[0] == 32.0
    a = oracle.make_input_bits(16, 512, oracle.F16, 91, 0, oracle.MODE_LCG)
    b = oracle.make_input_bits(16, 512, oracle.F16, 91, 1, oracle.MODE_LCG)
    f32 = oracle.gemm_ref(a, b, oracle.F16).reshape(-1)
    f16 = oracle.round_output(f32, "f16")
    first = int(np.flatnonzero(f32 != f16)[0])
    assert (float(f32[first]), float(f16[first])) == (-132.5625, -132.5)


# ------------------------------------ golden vectors from the Python reference
def test_gemm_golden_vectors(oracle):
    data = _load("gemm_golden.json")
    assert len(data["cases"]) >= 10
    for entry in data["cases"]:
        case = dict(entry["case"])
        M, N, K = case["M"], case["N"], case["K"]
        t = oracle.BF16 if case.get("input_type", "f16") == "bf16" else oracle.F16
        mode = oracle.MODE_LCG if case.get("random_data") else oracle.MODE_HALVES
        seed = case.get("random_seed", 0)
        a = oracle.make_input_bits(M, K, t, seed, 0, mode)
        b = oracle.make_input_bits(N, K, t, seed, 1, mode)
        af, bf = oracle.from_bits(a, t).reshape(-1), oracle.from_bits(b, t).reshape(-1)
        assert af[:16].tolist() == entry["a_head"] and bf[:16].tolist() == entry["b_head"]
        assert _sha(af) == entry["a_sha256"] and _sha(bf) == entry["b_sha256"]
        c = oracle.round_output(oracle.gemm_ref(a, b, t), case.get("output_type", "f32"))
        layout = case.get("output_layout", "row-major")
        got = oracle.layout_output(c, layout, case.get("BM", 1), case.get("BN", 1), case.get("wave_m_tiles", 1),
                                   case.get("wave_n_tiles", 1))
        want = np.asarray(entry["out"], np.float64)
        assert np.array_equal(got.astype(np.float64), want), case
        # the NumPy restatement agrees too
        assert np.array_equal(oracle.np_gemm_ref(a, b, t), oracle.gemm_ref(a, b, t))


def toy_fa_inputs(oracle, block_m, head_dim, seq_n, seed):
    """python/mlir/dialects/wave_attention.py:225-245: Q is multiplied by
    log2(e)/sqrt(d) in double precision and rounded straight to f16."""
    q = oracle.np_lcg_values(block_m * head_dim, seed, 0, 0.0625)
    k = oracle.np_lcg_values(seq_n * head_dim, seed, 1, 0.0625)
    v = oracle.np_lcg_values(seq_n * head_dim, seed, 2, 0.125)
    scale = np.log2(np.e) / np.sqrt(head_dim)
    f16 = lambda x: np.asarray(x, np.float64).astype(np.float16).view(np.uint16)
    return (f16(q * scale).reshape(1, block_m, head_dim), f16(k).reshape(1, seq_n, head_dim),
            f16(v).reshape(1, seq_n, head_dim))


def test_toy_attention_golden_vectors(oracle):
    data = _load("fa_toy_golden.json")
    assert data["cases"][0]["sizes"] == [256, 512, 512, 256]  # `fa-ref 256 512 512 256`
    for entry in data["cases"]:
        case = entry["case"]
        bm, hd, sn, seed = case["block_m"], case["head_dim"], case["seq_n"], case["random_seed"]
        q, k, v = toy_fa_inputs(oracle, bm, hd, sn, seed)
        for bits, head, sha in ((q, "q_head", "q_sha256"), (k, "k_head", "k_sha256"), (v, "v_head", "v_sha256")):
            vals = oracle.from_bits(bits, oracle.F16).reshape(-1)
            assert vals[:16].tolist() == entry[head]
            assert _sha(vals) == entry[sha]
        got = oracle.fa_ref(q, k, v, oracle.F16, 1.0, exp2_mode=True)[0].reshape(-1)
        want = np.asarray(entry["out"], np.float64)
        assert np.allclose(got, want, rtol=2e-7, atol=1e-9), case


# ------------------------------------------------- the compiled reference
def _ref_or_skip(oracle):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref/libwave_ref.so not built (no reference checkout on this machine)")
    return oracle.ref_lib()


@pytest.mark.parametrize("t", ["F16", "BF16"])
@pytest.mark.parametrize("mode", ["MODE_LCG", "MODE_ALL_ONES", "MODE_RAND_INT", "MODE_HPL"])
def test_generators_match_compiled_reference(oracle, t, mode):
    _ref_or_skip(oracle)
    T, mo = getattr(oracle, t), getattr(oracle, mode)
    for rows, k, seed, stream in ((7, 48, 0, 0), (33, 80, 91, 1), (128, 16, 12345, 0)):
        assert np.array_equal(oracle.make_input_bits(rows, k, T, seed, stream, mo),
                              oracle.ref_make_input_bits(rows, k, T, seed, stream, mo))


@pytest.mark.parametrize("t", ["F16", "BF16"])
def test_gemm_matches_compiled_reference_on_random_data(oracle, t):
    """Non-trivial summation: N(0,1) operands, where order matters.  The oracle
    must reproduce the reference's k-ascending f32 accumulation bit for bit."""
    _ref_or_skip(oracle)
    T = getattr(oracle, t)
    a = oracle.baseline_inputs((37, 1040), "normal", 1, 0, T)
    b = oracle.baseline_inputs((83, 1040), "normal", 1, 1, T, scale=0.03)
    got = oracle.gemm_ref(a, b, T)
    want = oracle.ref_gemm_rows(a, b, T)
    assert np.array_equal(got, want)
    rows = np.array([0, 5, 36], np.int32)
    assert np.array_equal(oracle.gemm_ref(a, b, T, rows=rows), want[rows])
    assert oracle.gemm_element(a, b, T, 5, 7) == want[5, 7]
    assert np.array_equal(oracle.np_gemm_ref(a, b, T), want)
    R = oracle.ref_lib()
    for v in (1.0009765625, -132.5625, 3.14159, 65519.0):
        assert R.wave_ref_round_output(v, 1) == float(oracle.round_output(np.array([v], np.float32), "f16")[0])
        assert R.wave_ref_round_output(v, 2) == float(oracle.round_output(np.array([v], np.float32), "bf16")[0])


def test_attention_matches_compiled_reference(oracle):
    R = _ref_or_skip(oracle)
    batch, heads, S = 1, 3, 640
    n = batch * heads * S * 128
    q = oracle.fa_input_bits(n, oracle.BF16, 4, 0, 0.125).reshape(heads, S, 128)
    k = oracle.fa_input_bits(n, oracle.BF16, 4, 1, 0.125).reshape(heads, S, 128)
    v = oracle.fa_input_bits(n, oracle.BF16, 4, 2, 0.25).reshape(heads, S, 128)
    ref_q = np.empty(n, np.uint16)
    R.wave_ref_fa_input_bits(ref_q, n, 4, 0, 0.125)
    assert np.array_equal(q.reshape(-1), ref_q)
    hs, rs = oracle.fa_sample_heads(batch * heads), oracle.fa_sample_rows(S)
    rh, rr = np.empty(8, np.int32), np.empty(600, np.int32)
    assert rh[:R.wave_ref_fa_sample_heads(batch, heads, rh)].tolist() == hs.tolist()
    assert rr[:R.wave_ref_fa_sample_rows(S, rr)].tolist() == rs.tolist() == [0, 31, 32, 127, 320, 512, 639]
    assert oracle.fa_sample_rows(256).tolist() == list(range(256))
    assert oracle.fa_sample_heads(9).tolist() == [0, 4, 8]
    want = oracle.ref_fa_rows(q, k, v, batch, heads, S, hs, rs)
    got = oracle.fa_ref(q, k, v, oracle.BF16, 1.0 / np.sqrt(128.0), heads=hs, rows=rs)
    assert np.array_equal(got, want)


def test_fragment_output_coordinates_known_answers(oracle):
    """Index -> (m, n) of the runner's tile-packed fragment layouts: the values
    test/Integration/Inputs/wave_matmul_rand_int_test.cpp:112-139 checks."""
    def coord(index, wmma, wave):
        m, n = oracle.tile_packed_fragment_coordinate(index, 16, 16, 1, 1, 1, 1, wmma, wave)
        return int(m), int(n)
    assert [coord(i, False, 64) for i in (0, 3, 4, 64, 255)] == [(0, 0), (3, 0), (0, 1), (4, 0), (15, 15)]
    assert [coord(i, True, 32) for i in (0, 7, 8, 128, 255)] == [(0, 0), (14, 0), (0, 1), (1, 0), (15, 15)]
    assert [coord(i, False, 32) for i in (7, 128)] == [(7, 0), (8, 0)]


@pytest.mark.parametrize("layout", ["tile-packed-mfma64", "tile-packed-wmma32", "tile-packed-mfma32"])
def test_fragment_layouts_are_permutations_and_match_compiled_reference(oracle, layout):
    M, N, BM, BN, wmt, wnt = 96, 128, 2, 2, 3, 2
    wmma, wave = oracle.FRAGMENT_LAYOUTS[layout]
    c = np.arange(M * N, dtype=np.float32).reshape(M, N)
    packed = oracle.layout_output(c, layout, BM, BN, wmt, wnt)
    assert sorted(packed.tolist()) == list(range(M * N))  # every coordinate exactly once (runner.cpp:846-872)
    if oracle.ref_lib() is None:
        pytest.skip("compiled reference not built")
    rng = np.random.default_rng(5)
    for index in rng.integers(0, M * N, 400).tolist() + [0, M * N - 1]:
        m, n = oracle.ref_output_coordinate(M, N, BM, BN, wmt, wnt, wmma, wave, index)
        assert packed[index] == c[m, n]


def test_causal_extension_is_masked_softmax(oracle):
    """The causal extension equals the non-causal reference run on the prefix
    of keys a row may see."""
    q = oracle.baseline_inputs((1, 96, 128), "normal", 2, 0, oracle.BF16)
    k = oracle.baseline_inputs((1, 96, 128), "normal", 2, 1, oracle.BF16)
    v = oracle.baseline_inputs((1, 96, 128), "normal", 2, 2, oracle.BF16)
    causal = oracle.fa_ref(q, k, v, oracle.BF16, 0.088, causal=True)
    for row in (0, 1, 17, 95):
        prefix = oracle.fa_ref(q, k[:, :row + 1], v[:, :row + 1], oracle.BF16, 0.088, rows=np.array([row], np.int32))
        assert np.array_equal(causal[0, row], prefix[0, 0])
