"""The CUDA C++ calibrate runner (tests/drivers/wave_matmul_calibrate_runner.cpp):
its host logic as a plain g++ program without a GPU (the reference tests its HIP
runner the same way, test/Integration/Inputs/wave_matmul_rand_int_test.cpp), and
on a GPU the runner itself through the reference's stdout contract
(test/Integration/wave_gfx950_streamk_f16_runtime.mlir:3-88)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVERS = os.path.join(ROOT, "tests", "drivers")
LINK = ["-I" + os.path.join(ROOT, "include"), "-L" + os.path.join(ROOT, "7_b200"), "-lwave_cuda",
        "-L" + os.path.join(ROOT, "oracle"), "-lwave_oracle",
        "-Wl,-rpath," + os.path.join(ROOT, "7_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle")]


def test_runner_host_logic_without_gpu(wc, oracle, tmp_path):
    wc.lib()  # builds libwave_cuda.so if needed
    exe = str(tmp_path / "runner_host_test")
    subprocess.run(["g++", "-std=c++17", "-O1", os.path.join(DRIVERS, "runner_host_test.cpp"), "-o", exe, *LINK],
                   check=True, cwd=DRIVERS)
    proc = subprocess.run([exe], capture_output=True, text=True)
    assert proc.returncode == 0 and "runner_host_test: ok" in proc.stdout, proc.stdout + proc.stderr


@pytest.fixture(scope="module")
def runner_exe(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = str(tmp_path_factory.mktemp("runner") / "wave_matmul_calibrate_runner")
    link = [a.replace("-Wl,-rpath,", "-Xlinker=-rpath=") for a in LINK]
    subprocess.run([nvcc, "-std=c++17", "-O2", "-x", "cu", os.path.join(DRIVERS, "wave_matmul_calibrate_runner.cpp"),
                    "-o", exe, *link], check=True, cwd=DRIVERS)
    return exe


def _run(exe, *args, expect=0):
    proc = subprocess.run([exe, *map(str, args)], capture_output=True, text=True, timeout=600)
    assert proc.returncode == expect, proc.stdout + proc.stderr
    return proc.stdout, proc.stderr


@pytest.mark.gpu
def test_runner_plain_abi(cuda, oracle, runner_exe):
    out, _ = _run(runner_exe, "--m=256", "--n=512", "--k=1024", "--bm=4", "--bn=4", "--wave-m-tiles=2",
                  "--wave-n-tiles=4", "--rand-int", "--iters=5", "--warmup=2", "--c-type=f16", "--hsaco", "unused.hsaco")
    for key in ("kernel: wmma_f16_matmul_tiled", "shape: m=256 n=512 k=1024", "loop_trip_count: 63", "iters: 5",
                "per_launch_us: ", "output_check: passed mode=strict layout=row-major elements=131072"):
        assert key in out, out


@pytest.mark.gpu
def test_runner_streamk_abi_and_counter_reset(cuda, oracle, runner_exe):
    out, _ = _run(runner_exe, "--m=512", "--n=512", "--k=2048", "--bm=4", "--bn=4", "--wave-m-tiles=2",
                  "--wave-n-tiles=4", "--hpl", "--input-type=bf16", "--kernel-abi=streamk", "--streamk-workers=5",
                  "--iters=1000", "--warmup=2", "--output-layout=column-major")
    assert "output_check: passed mode=strict layout=column-major" in out and "streamk_counter_check: passed" in out


@pytest.mark.gpu
def test_runner_exit_codes(cuda, oracle, runner_exe):
    _, err = _run(runner_exe, "--m=64", "--n=64", "--k=64", "--bn=3", expect=2)
    assert "BN must be a positive power of two" in err
    _, err = _run(runner_exe, "--rand-int", "--hpl", expect=2)
    assert "mutually exclusive" in err


@pytest.fixture(scope="module")
def fa_runner_exe(tmp_path_factory, wc):
    wc.lib()  # builds libwave_cuda.so if needed
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = str(tmp_path_factory.mktemp("fa_runner") / "wave_fa_runner")
    subprocess.run([nvcc, "-std=c++17", "-O2", "-x", "cu", "-Wno-deprecated-gpu-targets",
                    os.path.join(DRIVERS, "wave_fa_runner.cpp"), "-o", exe, "-I" + os.path.join(ROOT, "include"),
                    "-L" + os.path.join(ROOT, "7_b200"), "-lwave_cuda", "-Xlinker=-rpath=" + os.path.join(ROOT, "7_b200")],
                   check=True, cwd=DRIVERS)
    return exe


def test_fa_runner_rejects_bad_arguments(fa_runner_exe):
    """Exit code 2 and the reference runner's messages
    (tools/wave-fa-calibrate/wave-fa-gfx950-runner.cpp:63-66, 136-150); no GPU needed."""
    _, err = _run(fa_runner_exe, "--sequence", "300", expect=2)
    assert "sequence must be a multiple of 256" in err
    _, err = _run(fa_runner_exe, "--bogus", "1", expect=2)
    assert "unknown flag" in err
    _, err = _run(fa_runner_exe, "--iters", "0", expect=2)
    assert "invalid non-positive argument" in err
    _, err = _run(fa_runner_exe, "--heads", "x", expect=2)
    assert "bad integer argument" in err
    # tools/wave-fa-calibrate/wave-fa-gfx950.py:70-78
    _, err = _run(fa_runner_exe, "--qk-max-abs", "-1", expect=2)
    assert "--qk-max-abs must be finite and positive" in err
    _, err = _run(fa_runner_exe, "--qk-max-abs", "1", "--input-scale", "2", expect=2)
    assert "--qk-max-abs must cover the generated input range" in err


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [(), ("--causal",), ("--zero-qk",), ("--input-scale", "2"), ("--qk-max-abs", "1"),
                                   ("--qk-max-abs=1.5", "--causal")])
def test_fa_runner_contract(cuda, fa_runner_exe, extra):
    """The reference runner's stdout lines and its sampled f64 check
    (wave-fa-gfx950-runner.cpp:204-232, 388-394, 472-481)."""
    out, _ = _run(fa_runner_exe, "--batch", "2", "--heads", "3", "--sequence", "1024", "--iters", "3", "--warmup", "1",
                  "--check", "unused.hsaco", "flash_attention_bf16_gfx950", *extra)
    for key in ("shape: B=2 H=3 N=1024 D=128", "grid: 4,6,1 block: ", "per_launch_us: ", "tflops: ",
                "output_check: passed max_abs_diff="):
        assert key in out, out
