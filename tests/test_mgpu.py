"""The mgpu* wrappers of include/wave_mgpu.h: what a host `main` lowered by
gpu-to-llvm calls when mlir-runner runs it with libwave_cuda.so in place of
libmlir_rocm_runtime.so and libwave_runtime.so (the reference's README.md:99-106
and the RUN lines of test/Integration/*.mlir).  The GPU tests walk the sequence
of calls of the host module the reference emits (python/mlir/dialects/
wave_matmul.py:11244-11272: host buffers, gpu.host_register, the pointer helper,
one launch of `wmma_f16_matmul_tiled` with {A, B, C, trip}, read C on the host)
through ctypes, like the reference's own ctypes runner
(test/Integration/Inputs/wavec_wmma_matmul_ctypes_runner.py).
"""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest


class MemRef1D(C.Structure):
    _fields_ = [("allocated", C.c_void_p), ("aligned", C.c_void_p), ("offset", C.c_int64), ("size", C.c_int64),
                ("stride", C.c_int64)]


def memref_of(array: np.ndarray) -> MemRef1D:
    flat = array.reshape(-1)
    return MemRef1D(flat.ctypes.data, flat.ctypes.data, 0, flat.size, 1)


def params_block(*values):
    """void *params[]: one pointer per kernel argument, each to the argument's value."""
    cells = [v if isinstance(v, C._SimpleCData) else C.c_void_p(v) for v in values]
    block = (C.c_void_p * len(cells))(*[C.cast(C.pointer(c), C.c_void_p) for c in cells])
    return block, cells


def test_blob_round_trip_and_rejections(wc):
    lib = wc.lib()
    n = C.c_size_t(0)
    assert lib.wave_cuda_module_blob_bytes(wc.BLOB_GEMM, C.byref(n)) == wc.OK and n.value == 24 + C.sizeof(wc.GemmDesc)
    assert lib.wave_cuda_module_blob_bytes(wc.BLOB_FA, C.byref(n)) == wc.OK and n.value == 24 + C.sizeof(wc.FaDesc)
    assert lib.wave_cuda_module_blob_bytes(7, C.byref(n)) == wc.E_INVALID
    blob = wc.module_blob(wc.BLOB_GEMM, wc.gemm_desc(32, 32, 64, bm=2, bn=2, wave_k_tiles=2))
    assert blob[:8] == b"WAVECUDA"
    with pytest.raises(wc.WaveCudaError) as err:  # the writer validates like the code generator would
        wc.module_blob(wc.BLOB_GEMM, wc.gemm_desc(33, 32, 64))
    assert "M must be a positive multiple of 16; got 33" in err.value.message

    assert lib.wave_cuda_mgpu_status() == 0
    module = lib.mgpuModuleLoad(blob, len(blob))
    assert module and lib.wave_cuda_mgpu_status() == 0
    fn = lib.mgpuModuleGetFunction(module, b"wmma_f16_matmul_tiled")
    assert fn and lib.wave_cuda_mgpu_status() == 0
    assert not lib.mgpuModuleGetFunction(module, b"flash_attention_bf16_gfx950")
    assert lib.wave_cuda_mgpu_status() == wc.E_NOT_FOUND
    assert not lib.mgpuModuleGetFunction(module, b"some_other_kernel")
    assert lib.wave_cuda_mgpu_status() == wc.E_NOT_FOUND
    lib.mgpuModuleUnload(module)

    # a device code object (what the AMD flow embeds) is not a descriptor
    elf = b"\x7fELF" + bytes(60)
    assert not lib.mgpuModuleLoad(elf, len(elf))
    assert lib.wave_cuda_mgpu_status() == wc.E_INVALID
    assert not lib.mgpuModuleLoad(blob[:20], 20)
    assert lib.wave_cuda_mgpu_status() == wc.E_INVALID
    bad_version = blob[:8] + (99).to_bytes(4, "little") + blob[12:]
    assert not lib.mgpuModuleLoad(bad_version, len(bad_version))
    assert lib.wave_cuda_mgpu_status() == wc.E_INVALID
    # gpu-to-llvm passes the size, but older lowerings pass 0: the header then decides
    module = lib.mgpuModuleLoad(blob, 0)
    assert module
    lib.mgpuModuleUnload(module)

    fa_blob = wc.module_blob(wc.BLOB_FA, wc.fa_desc(1, 2, 256, 256, 128, qk_max_abs=1.0))
    module = lib.mgpuModuleLoad(fa_blob, len(fa_blob))
    assert module and lib.mgpuModuleGetFunction(module, b"flash_attention_bf16_gfx950")
    assert not lib.mgpuModuleGetFunction(module, b"wmma_f16_matmul_tiled")
    assert lib.wave_cuda_mgpu_status() == wc.E_NOT_FOUND
    lib.mgpuModuleUnload(module)


@pytest.mark.gpu
@pytest.mark.parametrize("out_name", ["f32", "f16"])
def test_host_module_sequence_gemm(cuda, wc, oracle, out_name):
    """The reference's --compare-cpu case (32x32x64, bm=bn=2, wave-k-tiles=2,
    seed 7) through the calls of its emitted host main, buffers in registered
    host memory."""
    lib = wc.lib()
    M, N, K = 32, 32, 64
    desc = wc.gemm_desc(M, N, K, bm=2, bn=2, wave_k_tiles=2, out_type=wc.TYPE_BY_NAME[out_name])
    a = oracle.make_input_bits(M, K, oracle.F16, 7, 0, oracle.MODE_LCG)
    b = oracle.make_input_bits(N, K, oracle.F16, 7, 1, oracle.MODE_LCG)
    c = np.full(M * N, 0x7FC0 if out_name == "f16" else np.nan, dtype=np.uint16 if out_name == "f16" else np.float32)
    refs = [memref_of(x) for x in (a, b, c)]
    for r, x in zip(refs, (a, b, c)):
        lib.mgpuMemHostRegisterMemRef(1, C.byref(r), x.itemsize)
    assert lib.wave_cuda_mgpu_status() == 0
    a_ptr = lib._mlir_ciface_wave_memref_to_ptr_global_f16(C.byref(refs[0]))
    b_ptr = lib._mlir_ciface_wave_memref_to_ptr_global_f16(C.byref(refs[1]))
    c_ptr = getattr(lib, f"_mlir_ciface_wave_memref_to_ptr_global_{out_name}")(C.byref(refs[2]))
    assert (a_ptr, b_ptr, c_ptr) == (a.ctypes.data, b.ctypes.data, c.ctypes.data)

    blob = wc.module_blob(wc.BLOB_GEMM, desc)
    module = lib.mgpuModuleLoad(blob, len(blob))
    fn = lib.mgpuModuleGetFunction(module, b"wmma_f16_matmul_tiled")
    stream = lib.mgpuStreamCreate()
    assert module and fn and stream
    trip = C.c_int32(K // (16 * 2) - 1)
    block, keep = params_block(a_ptr, b_ptr, c_ptr, trip)
    # grid = M_blocks x N_blocks, block = 64 * bm * bn threads (wave_matmul.py:426-444)
    lib.mgpuLaunchKernel(fn, 1, 1, 1, 256, 1, 1, 0, stream, block, None, 4)
    lib.mgpuStreamSynchronize(stream)
    assert lib.wave_cuda_mgpu_status() == 0
    wc.check_device_status()
    want = oracle.round_output(oracle.gemm_ref(a, b, oracle.F16), out_name).reshape(-1)
    got = c if out_name == "f32" else oracle.from_bits(c, oracle.F16)
    assert np.array_equal(got, want)

    # a grid that does not describe this problem is refused, C untouched
    c[:] = 0
    lib.mgpuLaunchKernel(fn, 2, 1, 1, 256, 1, 1, 0, stream, block, None, 4)
    assert lib.wave_cuda_mgpu_status() == wc.E_INVALID and not c.any()
    bad_trip = C.c_int32(5)
    block2, keep2 = params_block(a_ptr, b_ptr, c_ptr, bad_trip)
    lib.mgpuLaunchKernel(fn, 1, 1, 1, 256, 1, 1, 0, stream, block2, None, 4)
    assert lib.wave_cuda_mgpu_status() == wc.E_INVALID and not c.any()

    lib.mgpuStreamDestroy(stream)
    lib.mgpuModuleUnload(module)
    for r, x in zip(refs, (a, b, c)):
        lib.mgpuMemHostUnregisterMemRef(1, C.byref(r), x.itemsize)
    assert lib.wave_cuda_mgpu_status() == 0


@pytest.mark.gpu
def test_device_buffers_events_and_memset(cuda, wc, oracle):
    """gpu.alloc / gpu.memcpy / gpu.memset / gpu.wait lowerings: device buffers,
    a 512x256x384 bf16 problem, an event between two streams."""
    lib = wc.lib()
    M, N, K = 512, 256, 384
    desc = wc.gemm_desc(M, N, K, bm=2, bn=2, wave_m_tiles=2, wave_n_tiles=2, in_type=wc.BF16, out_type=wc.BF16)
    a = oracle.make_input_bits(M, K, oracle.BF16, 3, 0, oracle.MODE_LCG)
    b = oracle.make_input_bits(N, K, oracle.BF16, 3, 1, oracle.MODE_LCG)
    c = np.zeros(M * N, np.uint16)
    copy_stream, stream = lib.mgpuStreamCreate(), lib.mgpuStreamCreate()
    event = lib.mgpuEventCreate()
    d_a, d_b, d_c = (lib.mgpuMemAlloc(x.nbytes, copy_stream, 0) for x in (a, b, c))
    assert d_a and d_b and d_c and event
    lib.mgpuMemcpy(d_a, a.ctypes.data, a.nbytes, copy_stream)
    lib.mgpuMemcpy(d_b, b.ctypes.data, b.nbytes, copy_stream)
    lib.mgpuMemset16(d_c, 0x7FC0, c.size, copy_stream)  # bf16 NaN: unwritten elements would show
    lib.mgpuEventRecord(event, copy_stream)
    lib.mgpuStreamWaitEvent(stream, event)
    blob = wc.module_blob(wc.BLOB_GEMM, desc)
    module = lib.mgpuModuleLoad(blob, len(blob))
    fn = lib.mgpuModuleGetFunction(module, b"wmma_f16_matmul_tiled")
    block, keep = params_block(d_a, d_b, d_c, C.c_int32(K // 16 - 1))
    lib.mgpuLaunchKernel(fn, M // 64, N // 64, 1, 256, 1, 1, 0, stream, block, None, 4)
    lib.mgpuMemcpy(c.ctypes.data, d_c, c.nbytes, stream)
    lib.mgpuStreamSynchronize(stream)
    assert lib.wave_cuda_mgpu_status() == 0
    wc.check_device_status()
    want = oracle.round_output(oracle.gemm_ref(a, b, oracle.BF16), "bf16").reshape(-1)
    assert np.array_equal(oracle.from_bits(c, oracle.BF16), want)

    probe = np.zeros(1000, np.uint32)
    d_p = lib.mgpuMemAlloc(probe.nbytes, stream, 0)
    lib.mgpuMemset32(d_p, 0xDEADBEEF, probe.size, stream)
    lib.mgpuMemcpy(probe.ctypes.data, d_p, probe.nbytes, stream)
    lib.mgpuEventRecord(event, stream)
    lib.mgpuEventSynchronize(event)
    assert (probe == 0xDEADBEEF).all()
    for ptr in (d_a, d_b, d_c, d_p):
        lib.mgpuMemFree(ptr, stream)
    lib.mgpuEventDestroy(event)
    lib.mgpuStreamDestroy(stream)
    lib.mgpuStreamDestroy(copy_stream)
    lib.mgpuModuleUnload(module)
    assert lib.wave_cuda_mgpu_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("bound", [0.0, 1.0])
def test_host_module_sequence_attention(cuda, wc, oracle, bound):
    """{Q, K, V, O} of `flash_attention_bf16_gfx950` on registered host buffers,
    grid sequence/256 x batch*heads (wave_flash_attention.py:91-93)."""
    lib = wc.lib()
    B, H, S, D, t = 1, 3, 512, 128, oracle.BF16
    q = oracle.fa_input_bits(B * H * S * D, t, 5, 0, 0.125)
    k = oracle.fa_input_bits(B * H * S * D, t, 5, 1, 0.125)
    v = oracle.fa_input_bits(B * H * S * D, t, 5, 2, 0.25)
    o = np.zeros_like(q)
    for x in (q, k, v, o):
        lib.mgpuMemHostRegister(x.ctypes.data, x.nbytes)
    blob = wc.module_blob(wc.BLOB_FA, wc.fa_desc(B, H, S, S, D, qk_max_abs=bound))
    module = lib.mgpuModuleLoad(blob, len(blob))
    fn = lib.mgpuModuleGetFunction(module, b"flash_attention_bf16_gfx950")
    stream = lib.mgpuStreamCreate()
    block, keep = params_block(q.ctypes.data, k.ctypes.data, v.ctypes.data, o.ctypes.data)
    lib.mgpuLaunchKernel(fn, S // 256, B * H, 1, 512, 1, 1, 197888, stream, block, None, 4)
    lib.mgpuStreamSynchronize(stream)
    assert lib.wave_cuda_mgpu_status() == 0
    wc.check_device_status()
    shape = (B * H, S, D)
    want = oracle.fa_ref(q.reshape(shape), k.reshape(shape), v.reshape(shape), t, 1.0 / np.sqrt(128.0))
    got = oracle.from_bits(o, t).reshape(shape)
    assert np.abs(got - want).max() <= 3.0e-2  # wave-fa-gfx950-runner.cpp:388
    lib.mgpuStreamDestroy(stream)
    lib.mgpuModuleUnload(module)
    for x in (q, k, v, o):
        lib.mgpuMemHostUnregister(x.ctypes.data)
    assert lib.wave_cuda_mgpu_status() == 0


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def host_main_exe(tmp_path_factory, wc):
    """tests/drivers/wave_mlir_host_main.c built with gcc alone: no CUDA header
    and only libwave_cuda.so on the link line."""
    wc.lib()  # builds libwave_cuda.so if needed
    exe = str(tmp_path_factory.mktemp("host_main") / "wave_mlir_host_main")
    lib_dir = os.path.join(ROOT, "7_b200")
    subprocess.run(["gcc", "-std=c11", "-O2", "-Wall", "-Werror",
                    os.path.join(ROOT, "tests", "drivers", "wave_mlir_host_main.c"), "-o", exe,
                    "-I" + os.path.join(ROOT, "include"), "-L" + lib_dir, "-lwave_cuda", "-Wl,-rpath," + lib_dir],
                   check=True)
    return exe


def test_host_main_links_against_the_library_alone(host_main_exe):
    """An invalid tiling is refused by the blob writer with the reference's
    message before anything touches a GPU."""
    proc = subprocess.run([host_main_exe, "32", "32", "64", "2", "3"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 2
    assert "BN must be a positive power of two" in proc.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("args", [(), ("512", "768", "1024", "4", "4", "2", "4", "1", "11")])
def test_host_main_runs(cuda, host_main_exe, args):
    proc = subprocess.run([host_main_exe, *args], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    elements = 32 * 32 if not args else 512 * 768
    assert f"CPU comparison passed: elements={elements}" in proc.stdout
