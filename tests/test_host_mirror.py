"""Host-side mirror of the reference's Python interface: generators, config
validation and the Stream-K partition arithmetic, against the oracle and the
golden vectors recorded from the reference
(test/python/dialects/wave_matmul_streamk.py:13-57 is the model for the
exhaustive partition check)."""
import importlib
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def wm():
    return importlib.import_module("7_b200.wave_matmul")


def test_vectorised_lcg_matches_oracle(wm, oracle):
    for seed, stream, n in [(7, 0, 4096), (0, 1, 33), (91, 2, 100001), (5, 0, 1), (2 ** 31 - 1, 3, 777)]:
        assert np.array_equal(wm.deterministic_random_values(n, seed=seed, stream=stream),
                              oracle.lcg_values(n, seed, stream))
        assert np.allclose(wm.deterministic_random_values(min(n, 500), seed=seed, stream=stream),
                           oracle.np_lcg_values(min(n, 500), seed, stream))


@pytest.mark.parametrize("input_type", ["f16", "bf16"])
@pytest.mark.parametrize("random_data", [False, True])
def test_generate_inputs_matches_oracle(wm, oracle, input_type, random_data):
    t = oracle.F16 if input_type == "f16" else oracle.BF16
    mode = oracle.MODE_LCG if random_data else oracle.MODE_HALVES
    a, b = wm.generate_wmma_f16_matmul_inputs(48, 80, 96, input_type=input_type, random_data=random_data,
                                              random_seed=12345)
    assert np.array_equal(a, oracle.make_input_bits(48, 96, t, 12345, 0, mode))
    assert np.array_equal(b, oracle.make_input_bits(80, 96, t, 12345, 1, mode))


def test_config_geometry_and_validation(wm):
    cfg = wm.MatmulConfig(32, 32, 64, BM=2, BN=2, wave_k_tiles=2)  # the reference's --compare-cpu case
    assert (cfg.M_blocks, cfg.N_blocks, cfg.waves_per_workgroup, cfg.total_elements, cfg.trip_count) == (1, 1, 4, 1024, 1)
    with pytest.raises(ValueError, match="BN must be a positive power of two"):
        wm.MatmulConfig(32, 32, 64, BN=3)
    with pytest.raises(ValueError, match="output_type must be one of"):
        wm.MatmulConfig(32, 32, 64, output_type="f64")
    with pytest.raises(ValueError, match="M must be a positive multiple of 16"):
        wm.MatmulConfig(40, 32, 64)


def test_streamk_partition_matches_reference_golden(wm):
    with open(os.path.join(GOLDEN, "streamk_golden.json")) as f:
        data = json.load(f)
    assert data["sizes"]["scratch_elements_3"] == wm.streamk_scratch_elements(3) == 3 * 2 * 65536
    for case in data["cases"]:
        tiles, kit, workers = case["tiles"], case["k_iterations"], case["workers"]
        total = tiles * kit
        for w in range(workers):
            assert list(wm.streamk_worker_interval(total, workers, w)) == case["intervals"][w]
            segs = [[t, kb, ke, -1 if slot is None else slot]
                    for t, kb, ke, slot in wm.streamk_worker_segments(tiles, kit, workers, w)]
            assert segs == case["segments"][w]
        for t in range(tiles):
            assert list(wm.streamk_tile_contributors(t, kit, total, workers)) == case["contributors"][t]


def test_streamk_partition_exhaustive_properties(wm):
    """Tiles 1-9 x k 1-11 x every legal worker count: intervals tile the
    iteration space, owners agree with intervals, every tile's contributors
    are consecutive and each contributes exactly one segment, partial segments
    of a tile cover its k range exactly once, at most two slots per worker."""
    for tiles in range(1, 10):
        for kit in range(1, 12):
            total = tiles * kit
            for workers in range(1, total + 1):
                cover = np.zeros(total, np.int32)
                for w in range(workers):
                    b, e = wm.streamk_worker_interval(total, workers, w)
                    assert e > b
                    cover[b:e] += 1
                    assert wm.streamk_owner_for_iteration(total, workers, b) == w
                    assert wm.streamk_owner_for_iteration(total, workers, e - 1) == w
                    slots = [s for _, _, _, s in wm.streamk_worker_segments(tiles, kit, workers, w) if s is not None]
                    assert slots == list(range(len(slots))) and len(slots) <= 2
                assert (cover == 1).all()
                for t in range(tiles):
                    first, last = wm.streamk_tile_contributors(t, kit, total, workers)
                    kcover = np.zeros(kit, np.int32)
                    for w in range(first, last + 1):
                        mine = [s for s in wm.streamk_worker_segments(tiles, kit, workers, w) if s[0] == t]
                        assert len(mine) == 1
                        kcover[mine[0][1]:mine[0][2]] += 1
                    assert (kcover == 1).all()


def test_attention_runner_inputs_match_oracle(oracle):
    wa = importlib.import_module("7_b200.wave_attention")
    q, k, v = wa.make_runner_inputs(1, 2, 256, seed=9)
    n = 2 * 256 * 128
    assert np.array_equal(q.reshape(-1), oracle.fa_input_bits(n, oracle.BF16, 9, 0, 0.125))
    assert np.array_equal(k.reshape(-1), oracle.fa_input_bits(n, oracle.BF16, 9, 1, 0.125))
    assert np.array_equal(v.reshape(-1), oracle.fa_input_bits(n, oracle.BF16, 9, 2, 0.25))
    assert wa.flops(2, 64, 8192) == 4.0 * 2 * 64 * 8192 * 8192 * 128


def test_perf_sweep_selectors_dry_run():
    """The sweep's selectors and their validation need no GPU
    (tools/wave-matmul-calibrate/wave-matmul-perf-sweep.py:864-1058)."""
    import subprocess
    import sys
    tool = os.path.join(os.path.dirname(os.path.abspath(__file__)), "drivers", "wave_matmul_perf_sweep.py")

    def sweep(*args):
        return subprocess.run([sys.executable, tool, "--dry-run", *args], capture_output=True, text=True, timeout=120)
    p = sweep("--kernels=f16-4wave,fa", "--m=2048", "--n=1024", "--k-values=1024", "--fa-sequence=4096",
              "--fa-modes=bounded", "--fa-causal=no", "--variants=scheduled", "--hpl" if False else "--seed=3")
    assert p.returncode == 0, p.stderr
    assert "--m 2048 --n 1024 --k 1024" in p.stdout and "--sequence 4096" in p.stdout and "--qk-max-abs 1" in p.stdout
    assert p.stdout.count("wave_matmul_calibrate.py") == 1 and p.stdout.count("wave_fa_gfx950.py") == 1
    p = sweep()  # default: K sweep + the two 8192^3 points for f16 and bf16, four attention rows
    assert p.stdout.count("wave_matmul_calibrate.py") == 16 and p.stdout.count("wave_fa_gfx950.py") == 4
    for bad, message in ((["--kernels=mxfp4"], "outside this backend"),
                         (["--kernels=f16", "--streamk-workers=8"], "--streamk-workers requires --kernels=f16-streamk"),
                         (["--kernels=fa", "--rand-int"], "FA sweep supports random floating-point inputs only"),
                         (["--kernels=fa", "--variants=baseline"], "FA sweep supports only --variants=scheduled"),
                         (["--m=0"], "--m must be positive"),
                         (["--kernels=fa", "--fa-qk-max-abs=0"], "--fa-qk-max-abs must be finite and positive")):
        p = sweep(*bad)
        assert p.returncode != 0 and message in p.stderr, (bad, p.stderr)


def test_toy_attention_inputs_match_oracle(oracle):
    """The product-side generator of the toy attention inputs against the oracle's
    restatement of python/mlir/dialects/wave_attention.py:225-245."""
    import importlib
    wa = importlib.import_module("7_b200.wave_attention")
    from test_oracle import toy_fa_inputs
    for bm, hd, sn, seed in ((16, 32, 16, 0), (16, 64, 512, 7), (16, 128, 256, 91)):
        q, k, v = wa.generate_flash_attention_f32_inputs(bm, hd, sn, random_seed=seed)
        wq, wk, wv = toy_fa_inputs(oracle, bm, hd, sn, seed)
        assert np.array_equal(q, wq[0]) and np.array_equal(k, wk[0]) and np.array_equal(v, wv[0])
