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
