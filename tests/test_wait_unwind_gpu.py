"""A device-side wait that runs out, and what the kernel does then.

Every wait inside the kernels is bounded: when the limit passes, the waiting
role raises its CTA's abort flag, records {code, block, role, detail} in a
device status word, the other roles give up on their own waits, copies in
flight are given time to land, tensor memory is released and the kernel
returns.  The reference's analogue is the runner's timeout wrapper and counter
check (tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp:1718-1733).

Nothing here faults, traps or hangs the GPU.  The test uses a second build of
the library (7_b200/build.py build_wait_test) whose limit is about a
millisecond instead of a second and whose one-CTA GEMM can be told, through an
environment variable only that build reads, to leave the last K step of a tile
unloaded: the UMMA thread then waits for a shared-memory stage that never
fills, and the epilogue warps for an accumulator that never completes.
"""
import ctypes as C
import importlib
import os

import numpy as np
import pytest

from _util import to_device_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def waitlib(cuda):
    build = importlib.import_module("7_b200.build")
    wc = importlib.import_module("7_b200.wave_cuda")
    path = build.build_wait_test()
    lib = C.CDLL(path)
    vp = C.c_void_p
    lib.wave_cuda_gemm.argtypes = [C.POINTER(wc.GemmDesc), vp, vp, vp, vp, vp]
    lib.wave_cuda_check_device_status.argtypes = [C.POINTER(C.c_int)]
    lib.wave_cuda_last_error.restype = C.c_char_p
    return lib


def _launch(torch, lib, wc, a, b, c, desc):
    return lib.wave_cuda_gemm(C.byref(desc), a.data_ptr(), b.data_ptr(), c.data_ptr(), None,
                              torch.cuda.current_stream().cuda_stream)


def test_wait_runs_out_kernel_unwinds_and_next_launch_is_exact(cuda, wc, oracle, waitlib):
    torch = cuda
    M, N, K = 128, 128, 256  # one tile, four K steps
    a_bits = oracle.make_input_bits(M, K, oracle.F16, 13, 0, oracle.MODE_LCG)
    b_bits = oracle.make_input_bits(N, K, oracle.F16, 13, 1, oracle.MODE_LCG)
    a, b = to_device_bits(torch, a_bits), to_device_bits(torch, b_bits)
    desc = wc.gemm_desc(M, N, K, bm=4, bn=4, wave_m_tiles=2, wave_n_tiles=2)  # 128 x 128 tile, one-CTA kernel
    want = oracle.gemm_ref(a_bits, b_bits, oracle.F16)
    status = (C.c_int * 4)()

    # 1. an ordinary launch through the test build is exact and reports nothing
    c = torch.full((M, N), float("nan"), device="cuda")
    assert _launch(torch, waitlib, wc, a, b, c, desc) == 0
    assert waitlib.wave_cuda_check_device_status(status) == 0
    assert np.array_equal(c.cpu().numpy(), want)

    # 2. the producer leaves out the last K step: the wait for it runs out
    c = torch.full((M, N), float("nan"), device="cuda")
    os.environ["WAVE_CUDA_TEST_SKIP_LAST_K"] = "1"
    try:
        assert _launch(torch, waitlib, wc, a, b, c, desc) == 0  # the launch itself succeeds
        rc = waitlib.wave_cuda_check_device_status(status)      # synchronises: the kernel has returned
    finally:
        del os.environ["WAVE_CUDA_TEST_SKIP_LAST_K"]
    assert rc == wc.E_DEVICE_STATUS, waitlib.wave_cuda_last_error()
    code, block, role, detail = list(status)
    assert code == 1 and block == 0          # a wait timed out, in the only CTA
    # whichever waiter's limit passed first reports: the UMMA thread (role 1, the
    # stage it waited for) or an epilogue warp (role 2, 200 + accumulator buffer)
    assert (role == 1 and detail == 3) or (role == 2 and detail == 200), (role, detail)
    assert np.isnan(c.cpu().numpy()).all()   # no output was written from the incomplete accumulator
    assert b"status 1" in waitlib.wave_cuda_last_error()

    # 3. the record was cleared by reading it, the context is usable, and tensor
    #    memory was released: the next launches allocate it again and are exact
    assert waitlib.wave_cuda_check_device_status(status) == 0
    for _ in range(3):
        c = torch.full((M, N), float("nan"), device="cuda")
        assert _launch(torch, waitlib, wc, a, b, c, desc) == 0
        assert waitlib.wave_cuda_check_device_status(status) == 0
        assert np.array_equal(c.cpu().numpy(), want)
    # and the product library, loaded in the same process, is unaffected
    c = torch.full((M, N), float("nan"), device="cuda")
    wc.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), 0, torch.cuda.current_stream().cuda_stream)
    wc.check_device_status()
    assert np.array_equal(c.cpu().numpy(), want)
