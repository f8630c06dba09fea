"""Builds libwave_cuda.so (the C-ABI CUDA backend) in-tree with nvcc for sm_100a.

Usage: python 7_b200/build.py [--force] [--verbose]
The library is written next to this file so that it travels with the source
tree; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libwave_cuda.so")
SOURCES = ["gemm_sm100.cu", "gemm_pair_sm100.cu", "gemm_noalloc_sm100.cu", "fa_sm100.cu", "fa_stream_sm100.cu",
           "fa_pair_sm100.cu", "fa_decoupled_sm100.cu", "wave_cuda_backend.cu", "mgpu_runtime.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def needs_build(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    built = os.path.getmtime(lib)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [
        os.path.join(HERE, "..", "include", "wave_cuda.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def _compile_and_link(lib: str, build_dir: str, extra_flags: list[str], verbose: bool) -> str:
    objs = []
    procs = []
    os.makedirs(build_dir, exist_ok=True)
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", *extra_flags,
               "-Xptxas", "-v" if verbose else "-warn-spills", "-c", os.path.join(CSRC, src), "-o", obj]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    # link beside the target and rename: a reader never sees a half-written library
    link = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", lib + ".tmp", *objs]
    subprocess.run(link, check=True)
    os.replace(lib + ".tmp", lib)
    return lib


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    return _compile_and_link(LIB, os.path.join(HERE, "build"), [], verbose)


# A second build of the same sources for ONE test (tests/test_wait_unwind_gpu.py):
# device-side waits give up after about a millisecond instead of a second, and
# the one-CTA GEMM's producer can be told to leave out a K step, so that the
# unwind of a wait that runs out (status word, abort flag, TMEM release) can be
# watched without anything hanging.  The product library has neither.
WAIT_TEST_LIB = os.path.join(HERE, "libwave_cuda_waittest.so")
WAIT_TEST_FLAGS = ["-DWAVE_WAIT_TEST", "-DWAVE_WAIT_LIMIT_CYCLES=2000000"]


def build_wait_test(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.exists(WAIT_TEST_LIB) and not needs_build(WAIT_TEST_LIB):
        return WAIT_TEST_LIB
    return _compile_and_link(WAIT_TEST_LIB, os.path.join(HERE, "build_waittest"), WAIT_TEST_FLAGS, verbose)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--wait-test" in sys.argv:
        print(build_wait_test(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
