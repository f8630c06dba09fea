"""The command-line checkers in tests/drivers, run the way the reference's
integration tests run its tools: a child process whose stdout must contain
`CPU comparison passed` / `output_check: passed`
(test/Integration/wave_mfma_per_wave_tiles.mlir:3-11,
wave_flash_attention_gfx950_runtime.mlir:3-22,
wave_gfx950_streamk_f16_runtime.mlir:3-88)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
DRIVERS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "drivers")


def run(tool, *args, expect=0):
    proc = subprocess.run([sys.executable, os.path.join(DRIVERS, tool), *map(str, args)], capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == expect, proc.stdout + proc.stderr
    return proc.stdout, proc.stderr


def test_example_driver_compare_cpu_reference_case(cuda):
    # README / wave_mfma_per_wave_tiles.mlir: 32x32x64, bm=bn=2, wave-k-tiles=2, seed 7
    out, _ = run("wmma_matmul_tiled.py", "--m=32", "--n=32", "--k=64", "--bm=2", "--bn=2", "--wave-k-tiles=2",
                 "--compare-cpu", "--seed=7", "--matrix-intrinsic=mfma", "--chip=gfx942")
    assert "CPU comparison passed: elements=1024" in out


@pytest.mark.parametrize("extra", [
    ["--input-type=bf16", "--output-type=f16"],
    ["--output-layout=column-major", "--wave-m-tiles=2", "--wave-n-tiles=2"],
    ["--output-layout=tile-packed", "--bm=2", "--bn=2", "--wave-n-tiles=2"],
])
def test_example_driver_variants(cuda, extra):
    out, _ = run("wmma_matmul_tiled.py", "--m=64", "--n=128", "--k=96", "--compare-cpu", "--seed=3", *extra)
    assert "CPU comparison passed" in out


def test_example_driver_prints_data_and_rejects_bad_shape(cuda):
    out, _ = run("wmma_matmul_tiled.py", "--m=16", "--n=16", "--k=16", "--run")
    assert out.startswith("data = ") and out.count(",") == 255
    _, err = run("wmma_matmul_tiled.py", "--m=24", "--n=16", "--k=16", "--run", expect=2)
    assert "M must be a positive multiple of 16; got 24" in err


def test_gemm_calibrate_runner_contract(cuda):
    out, _ = run("wave_matmul_calibrate.py", "--m=256", "--n=512", "--k=1024", "--bm=4", "--bn=4", "--wave-m-tiles=2",
                 "--wave-n-tiles=4", "--rand-int", "--iters=5", "--warmup=2", "--c-type=f16")
    for key in ("kernel: wmma_f16_matmul_tiled", "shape: m=256 n=512 k=1024", "iters: 5", "per_launch_us: ",
                "total_ms: ", "tflops: ", "output_check: passed mode=strict layout=row-major elements=131072"):
        assert key in out, out
    assert "input_mode=rand_int" in out


@pytest.mark.parametrize("flags,layout", [
    (("--wave-size=64",), "tile-packed-mfma64"),
    ((), "tile-packed-wmma32"),
    (("--accumulator-layout=mfma",), "tile-packed-mfma32"),
])
def test_gemm_calibrate_runner_tile_packed_fragments(cuda, flags, layout):
    """Tile-packed output in the accumulator-fragment order the reference's runner
    validates (wave-matmul-calibrate-runner.cpp:765-769, 809-836, 888-988)."""
    out, _ = run("wave_matmul_calibrate.py", "--m=128", "--n=256", "--k=512", "--bm=2", "--bn=2", "--wave-m-tiles=2",
                 "--wave-n-tiles=4", "--output-layout=tile-packed", "--iters=3", "--warmup=1", *flags)
    assert f"output_check: passed mode=strict layout={layout} elements=32768" in out, out


def test_calibrate_tools_sustained_loop(cuda):
    """The >= N s back-to-back loop next to the 200-launch timing (the clock the
    power cap allows shows only after a fraction of a second)."""
    out, _ = run("wave_matmul_calibrate.py", "--m=1024", "--n=1024", "--k=1024", "--bm=4", "--bn=4", "--wave-m-tiles=2",
                 "--wave-n-tiles=4", "--iters=5", "--warmup=1", "--no-check", "--sustained-seconds=0.2")
    assert "sustained_per_launch_us: " in out and "sustained_tflops: " in out, out
    out, _ = run("wave_fa_gfx950.py", "--batch=1", "--heads=4", "--sequence=1024", "--iters=3", "--warmup=1",
                 "--sustained-seconds=0.2")
    assert "sustained_per_launch_us: " in out and "sustained_tflops: " in out, out


def test_gemm_calibrate_runner_streamk(cuda):
    out, _ = run("wave_matmul_calibrate.py", "--m=512", "--n=512", "--k=2048", "--bm=4", "--bn=4", "--wave-m-tiles=2",
                 "--wave-n-tiles=4", "--hpl", "--input-type=bf16", "--kernel-abi=streamk", "--streamk-workers=5",
                 "--iters=50", "--warmup=2")
    assert "output_check: passed" in out and "streamk_counter_check: passed" in out
    assert "kernel: gfx950_f16_streamk_gemm" in out


def test_gemm_calibrate_runner_bad_arguments(cuda):
    _, err = run("wave_matmul_calibrate.py", "--m=64", "--n=64", "--k=64", "--bn=3", expect=2)
    assert "BN must be a positive power of two" in err


def test_attention_calibrate_runner(cuda):
    out, _ = run("wave_fa_gfx950.py", "--batch=1", "--heads=2", "--sequence=512", "--iters=3", "--warmup=1", "--check")
    assert "shape: B=1 H=2 N=512 D=128" in out and "output_check: passed max_abs_diff=" in out
    assert "median_tflops: " in out
    out, _ = run("wave_fa_gfx950.py", "--batch=2", "--heads=3", "--sequence=1024", "--iters=3", "--warmup=1", "--check",
                 "--causal", "--seed=5")
    assert "output_check: passed" in out
    _, err = run("wave_fa_gfx950.py", "--sequence=300", expect=2)
    assert "multiple of 256" in err
    # the fixed softmax reference the reference's published numbers use (wave-fa-gfx950.py:103-107)
    out, _ = run("wave_fa_gfx950.py", "--batch=1", "--heads=2", "--sequence=1024", "--iters=3", "--warmup=1", "--check",
                 "--qk-max-abs=1")
    assert "output_check: passed" in out
    _, err = run("wave_fa_gfx950.py", "--qk-max-abs=1", "--input-scale=2", expect=2)
    assert "--qk-max-abs must cover the generated input range" in err
    out, _ = run("wave_fa_gfx950.py", "--batch=1", "--heads=2", "--sequence=512", "--iters=3", "--warmup=1", "--check",
                 "--head-dim=64", "--causal")
    assert "shape: B=1 H=2 N=512 D=64" in out and "output_check: passed" in out
    _, err = run("wave_fa_gfx950.py", "--head-dim=72", expect=1)
    assert "head_dim must be a multiple of 16 between 16 and 128" in err
    _, err = run("wave_fa_gfx950.py", "--qk-max-abs=2", "--input-scale=2", expect=1)
    assert "qk_max_abs fixed reference exceeds BF16 range" in err


def test_toy_attention_calibrate_tool(cuda):
    """The drop-in for tools/wave-fa-calibrate/wave-fa-calibrate.py: the toy
    kernel `flash_attention_f32` by name, the runner's keys and its 3e-3 check
    (wave-fa-calibrate-runner.cpp:250-292; the configurations of
    test/Integration/wave_flash_attention.mlir)."""
    out, _ = run("wave_fa_calibrate.py", "--iters=5", "--warmup=1")
    for key in ("kernel: flash_attention_f32", "shape: block_m=16 block_n=16 seq_n=16 head_dim=32 seed=0", "iters: 5",
                "total_ms: ", "per_launch_us: ", "per_launch_cycles_wallclock: ", "output_check: passed max_abs_diff="):
        assert key in out, out
    assert out.count("variant: ") == 2  # baseline and scheduled, like the reference's default
    out, _ = run("wave_fa_calibrate.py", "--head-dim=64", "--seq-n=512", "--seed=7", "--iters=3", "--warmup=1", "--repeats=3",
                 "--variants=scheduled", "--target-waves=2")
    assert "seq_n=512 head_dim=64 seed=7" in out and "output_check: passed" in out and "median_per_launch_us: " in out
    out, _ = run("wave_fa_calibrate.py", "--head-dim=128", "--seq-n=256", "--skip-hw")
    assert "grid: 1,1,1" in out and "per_launch_us" not in out
    _, err = run("wave_fa_calibrate.py", "--seq-n=24", expect=2)
    assert "seq-n must be a multiple of block-n" in err


def test_perf_sweep_selected_kernels_and_shapes(cuda, tmp_path):
    """--kernels / --m / --n / --k-values / --fa-* pick what the sweep runs
    (wave-matmul-perf-sweep.py:864-992); the CSV keeps the reference's columns."""
    csv_path = tmp_path / "sweep.csv"
    out, _ = run("wave_matmul_perf_sweep.py", "--kernels=f16,f16-streamk,fa", "--m=512", "--n=768", "--k-values=256,512",
                 "--streamk-workers=24", "--fa-batch=1", "--fa-heads=2", "--fa-sequence=512", "--fa-modes=adaptive",
                 "--fa-causal=no", "--iters=3", "--warmup=1", "--repeats=2", "--check", f"--csv={csv_path}")
    lines = [ln for ln in out.splitlines() if ln.startswith("| f") ]
    assert len(lines) == 5 and all("passed" in ln for ln in lines), out
    assert "| f16-gemm-streamk | 512x768x512 |" in out and "| fa-bf16-adaptive | B=1 H=2 S=512 D=128 |" in out
    header = csv_path.read_text().splitlines()[0].split(",")
    assert header[:5] == ["kernel", "profile", "m", "n", "k"] and header[-1] == "waves" and len(header) == 22
