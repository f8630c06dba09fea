"""Generates the golden vectors in this directory by running the reference's
own Python CPU references.

Runs only where a reference checkout exists (``--reference PATH``).  The
reference modules import an MLIR Python package that is not installed; the
functions used here (input generators, CPU references, Stream-K partition
math) are dependency-free arithmetic, so the MLIR names are replaced by inert
stand-ins for the duration of the import.  Nothing of the reference is copied:
its functions are executed and their outputs recorded.

Usage:  python tests/golden/make_golden.py [--reference /path/to/reference]
Writes: gemm_golden.json, fa_toy_golden.json, streamk_golden.json
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import os
import struct
import sys
import types
from unittest.mock import MagicMock

HERE = os.path.dirname(os.path.abspath(__file__))


class _Inert(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        value = MagicMock(name=name)
        setattr(self, name, value)
        return value


def _load_reference(reference: str):
    for name in (
        "mlir", "mlir._mlir_libs", "mlir._mlir_libs._waveDialectsNanobind", "mlir.dialects",
        "mlir.dialects.scf", "mlir.dialects.wave", "mlir.dialects.waveamd", "mlir.dialects.wavemeta",
        "mlir.dialects.wave_dsl", "mlir.dialects.wave_target", "mlir.ir", "ixsimpl",
    ):
        mod = _Inert(name)
        mod.__path__ = []
        sys.modules[name] = mod

    def load(name, rel):
        spec = importlib.util.spec_from_file_location(name, os.path.join(reference, rel))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    return (load("_ref_wave_matmul", "python/mlir/dialects/wave_matmul.py"),
            load("_ref_wave_attention", "python/mlir/dialects/wave_attention.py"))


def _digest(values) -> str:
    return hashlib.sha256(struct.pack(f"<{len(values)}f", *values)).hexdigest()


GEMM_CASES = [
    # (M, N, K, kwargs) -- kwargs go to compute_wmma_f16_matmul_reference_buffer
    dict(M=16, N=16, K=16, random_data=True, random_seed=7),
    dict(M=32, N=32, K=64, BM=2, BN=2, wave_k_tiles=2, random_data=True, random_seed=7),
    dict(M=32, N=32, K=64, BM=2, BN=2, wave_k_tiles=2, random_data=True, random_seed=7,
         input_type="bf16", matrix_intrinsic="mfma_gfx950"),
    dict(M=32, N=32, K=32, wave_m_tiles=2, wave_n_tiles=2, wave_k_tiles=2, random_data=True,
         random_seed=7, matrix_intrinsic="mfma"),
    dict(M=32, N=48, K=32, wave_m_tiles=2, wave_n_tiles=3, wave_k_tiles=2, random_data=True,
         random_seed=7, matrix_intrinsic="mfma", output_layout="row-major"),
    dict(M=32, N=48, K=32, wave_m_tiles=2, wave_n_tiles=3, wave_k_tiles=2, random_data=True,
         random_seed=7, matrix_intrinsic="mfma", output_layout="column-major"),
    dict(M=16, N=16, K=32, matrix_intrinsic="mfma_gfx950", input_type="bf16"),
    dict(M=16, N=16, K=512, random_data=True, random_seed=91, output_type="f32"),
    dict(M=16, N=16, K=512, random_data=True, random_seed=91, output_type="f16"),
    dict(M=64, N=32, K=128, BM=2, BN=2, random_data=True, random_seed=3, output_type="f16"),
    dict(M=48, N=80, K=96, random_data=True, random_seed=12345, input_type="bf16",
         matrix_intrinsic="mfma_gfx950"),
    dict(M=64, N=96, K=32, BM=2, BN=2, wave_m_tiles=2, wave_n_tiles=3, random_data=True, random_seed=21,
         output_layout="tile-packed"),
    dict(M=32, N=32, K=64, BM=2, BN=2, wave_k_tiles=2, random_data=True, random_seed=7,
         output_layout="tile-packed", output_type="f16"),
]

FA_CASES = [
    dict(block_m=16, block_n=16, head_dim=16, random_seed=11, seq_n=32),
    dict(block_m=16, block_n=16, head_dim=32, random_seed=0, seq_n=16),
    dict(block_m=16, block_n=16, head_dim=64, random_seed=5, seq_n=64),
    dict(block_m=16, block_n=16, head_dim=128, random_seed=9, seq_n=128),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("WAVE_REFERENCE_ROOT"), required="WAVE_REFERENCE_ROOT" not in os.environ,
                    help="path of the reference checkout (or set WAVE_REFERENCE_ROOT)")
    args = ap.parse_args()
    wm, wa = _load_reference(args.reference)

    gemm = []
    for case in GEMM_CASES:
        kw = dict(case)
        M, N, K = kw.pop("M"), kw.pop("N"), kw.pop("K")
        out = wm.compute_wmma_f16_matmul_reference_buffer(M, N, K, **kw)
        a, b = wm.generate_wmma_f16_matmul_inputs(
            M, N, K, input_type=kw.get("input_type", "f16"),
            random_data=kw.get("random_data", False), random_seed=kw.get("random_seed", 0))
        gemm.append(dict(case=case, a_head=list(a[:16]), b_head=list(b[:16]),
                         a_sha256=_digest(a), b_sha256=_digest(b), out=list(out)))
    with open(os.path.join(HERE, "gemm_golden.json"), "w") as f:
        json.dump(dict(source="python/mlir/dialects/wave_matmul.py "
                              "compute_wmma_f16_matmul_reference_buffer / generate_wmma_f16_matmul_inputs",
                       cases=gemm), f)

    fa = []
    for case in FA_CASES:
        kw = dict(case)
        bm, bn, hd = kw.pop("block_m"), kw.pop("block_n"), kw.pop("head_dim")
        q, k, v = wa.generate_flash_attention_f32_inputs(bm, bn, hd, **kw)
        out = wa.compute_flash_attention_f32_reference(bm, bn, hd, **kw)
        fa.append(dict(case=case, q_head=list(q[:16]), k_head=list(k[:16]), v_head=list(v[:16]),
                       q_sha256=_digest(q), k_sha256=_digest(k), v_sha256=_digest(v),
                       sizes=[len(q), len(k), len(v), len(out)], out=list(out)))
    with open(os.path.join(HERE, "fa_toy_golden.json"), "w") as f:
        json.dump(dict(source="python/mlir/dialects/wave_attention.py "
                              "compute_flash_attention_f32_reference / generate_flash_attention_f32_inputs",
                       cases=fa), f)

    sk = []
    for tiles, kiters, workers in [(1, 1, 1), (3, 4, 5), (4, 8, 3), (9, 11, 7), (224, 128, 148), (6, 32, 5)]:
        total = tiles * kiters
        intervals = [list(wm.streamk_worker_interval(total, workers, w)) for w in range(workers)]
        contributors = [list(wm.streamk_tile_contributors(t, kiters, total, workers)) for t in range(tiles)]
        segments = [[[s.tile, s.k_begin, s.k_end, -1 if s.scratch_slot is None else s.scratch_slot]
                     for s in wm.streamk_worker_segments(tiles, kiters, workers, w)] for w in range(workers)]
        sk.append(dict(tiles=tiles, k_iterations=kiters, workers=workers, intervals=intervals,
                       contributors=contributors, segments=segments))
    sizes = dict(scratch_elements_3=wm.streamk_scratch_elements(3),
                 counter_elements_512_768=wm.streamk_counter_elements(512, 768))
    with open(os.path.join(HERE, "streamk_golden.json"), "w") as f:
        json.dump(dict(source="python/mlir/dialects/wave_matmul.py streamk_* partition math",
                       cases=sk, sizes=sizes), f)
    print("wrote", [n for n in sorted(os.listdir(HERE)) if n.endswith(".json")])


if __name__ == "__main__":
    main()
