"""ctypes binding of libwave_cuda.so (the C ABI declared in include/wave_cuda.h).

This is the only way Python reaches the CUDA kernels.  There is no CPU or
PyTorch fallback: if the library is missing it is built, and if that fails or
no CUDA device is present the compute calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwave_cuda.so")

F16, BF16, F32 = 0, 1, 2
ROW_MAJOR, COL_MAJOR, TILE_PACKED = 0, 1, 2
TILE_PACKED_MFMA64, TILE_PACKED_WMMA32, TILE_PACKED_MFMA32 = 3, 4, 5  # AMD fragment order inside a tile
OK, E_INVALID, E_UNSUPPORTED, E_CUDA, E_DEVICE_STATUS, E_NOT_FOUND = 0, -1, -2, -3, -4, -5

TYPE_BY_NAME = {"f16": F16, "bf16": BF16, "f32": F32}
LAYOUT_BY_NAME = {"row-major": ROW_MAJOR, "column-major": COL_MAJOR, "tile-packed": TILE_PACKED,
                  "tile-packed-mfma64": TILE_PACKED_MFMA64, "tile-packed-wmma32": TILE_PACKED_WMMA32,
                  "tile-packed-mfma32": TILE_PACKED_MFMA32}


class WaveCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"wave_cuda error {code}: {message}")
        self.code = code
        self.message = message


class GemmDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in (
        "M", "N", "K", "bm", "bn", "wave_m_tiles", "wave_n_tiles", "wave_k_tiles", "in_type", "out_type",
        "out_layout", "cta_group_m", "streamk_workers", "ldc")]


class FaDesc(C.Structure):
    _fields_ = [("batch", C.c_int), ("heads", C.c_int), ("seq_q", C.c_int), ("seq_k", C.c_int),
                ("head_dim", C.c_int), ("scale", C.c_float), ("causal", C.c_int), ("io_type", C.c_int),
                ("out_f32", C.c_int), ("qk_max_abs", C.c_float)]


EXPORTS = [
    "wave_cuda_last_error", "wave_cuda_version", "wave_cuda_reload_env",
    "_mlir_ciface_wave_memref_to_ptr_global_i32", "_mlir_ciface_wave_memref_to_ptr_global_i8",
    "_mlir_ciface_wave_memref_to_ptr_global_f32", "_mlir_ciface_wave_memref_to_ptr_global_f16",
    "_mlir_ciface_wave_memref_to_ptr_global_bf16", "_mlir_ciface_wave_memref_to_ptr_global_i64",
    "_mlir_ciface_wave_memref_to_ptr_global_f64",
    "wave_cuda_gemm_desc_init", "wave_cuda_gemm_validate", "wave_cuda_gemm_workspace_bytes", "wave_cuda_gemm",
    "wave_cuda_gemm_host", "wave_cuda_gemm_host_a_resident", "wave_cuda_gemm_multi_output", "wave_cuda_gemm_multicast_output",
    "wave_cuda_gemm_plan", "wave_cuda_gemm_plan_for_sms", "wave_cuda_gemm_streamk_static", "wave_cuda_fa_validate", "wave_cuda_flash_attention_fwd",
    "wave_cuda_flash_attention_fwd_multi_output", "wave_cuda_flash_attention_fwd_multicast_output",
    "wave_cuda_flash_attention_fwd_host", "wave_cuda_module_get_function", "wave_cuda_launch",
    "wave_cuda_function_release", "wave_cuda_check_device_status",
    # include/wave_mgpu.h: the wrappers a host module lowered by gpu-to-llvm calls
    "wave_cuda_module_blob_bytes", "wave_cuda_module_blob_write", "wave_cuda_mgpu_status", "wave_cuda_memref_region",
    "mgpuModuleLoad", "mgpuModuleUnload", "mgpuModuleGetFunction", "mgpuLaunchKernel", "mgpuStreamCreate",
    "mgpuStreamDestroy", "mgpuStreamSynchronize", "mgpuStreamWaitEvent", "mgpuEventCreate", "mgpuEventDestroy",
    "mgpuEventSynchronize", "mgpuEventRecord", "mgpuMemAlloc", "mgpuMemFree", "mgpuMemcpy", "mgpuMemset32",
    "mgpuMemset16", "mgpuMemHostRegister", "mgpuMemHostUnregister", "mgpuMemHostRegisterMemRef",
    "mgpuMemHostUnregisterMemRef", "mgpuSetDefaultDevice",
]
BLOB_GEMM, BLOB_FA = 0, 1

_lib = None


def lib() -> C.CDLL:
    """Loads (building first if needed) the backend library."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    L = C.CDLL(LIB_PATH)
    vp, ip = C.c_void_p, C.POINTER(C.c_int)
    L.wave_cuda_last_error.restype = C.c_char_p
    L.wave_cuda_version.restype = C.c_char_p
    L.wave_cuda_reload_env.restype = None
    L.wave_cuda_reload_env.argtypes = []
    for name in EXPORTS[3:10]:
        getattr(L, name).restype = vp
        getattr(L, name).argtypes = [vp]
    L.wave_cuda_gemm_desc_init.argtypes = [C.POINTER(GemmDesc), C.c_int, C.c_int, C.c_int]
    L.wave_cuda_gemm_desc_init.restype = None
    L.wave_cuda_gemm_validate.argtypes = [C.POINTER(GemmDesc)]
    L.wave_cuda_gemm_workspace_bytes.argtypes = [C.POINTER(GemmDesc), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
    L.wave_cuda_gemm.argtypes = [C.POINTER(GemmDesc), vp, vp, vp, vp, vp]
    L.wave_cuda_gemm_host.argtypes = [C.POINTER(GemmDesc), vp, vp, vp, vp]
    L.wave_cuda_gemm_host_a_resident.argtypes = [C.POINTER(GemmDesc), vp, vp, vp, vp]
    L.wave_cuda_gemm_multi_output.argtypes = [C.POINTER(GemmDesc), vp, vp, C.POINTER(vp), C.c_int, vp]
    L.wave_cuda_gemm_multicast_output.argtypes = [C.POINTER(GemmDesc), vp, vp, vp, vp, vp]
    L.wave_cuda_gemm_streamk_static.argtypes = [C.POINTER(GemmDesc), vp, vp, vp, vp]
    L.wave_cuda_gemm_plan.argtypes = [C.POINTER(GemmDesc), ip, ip, ip, ip, ip]
    L.wave_cuda_gemm_plan_for_sms.argtypes = [C.POINTER(GemmDesc), C.c_int, C.c_int, ip, ip, ip, ip, ip,
                                              C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]
    L.wave_cuda_fa_validate.argtypes = [C.POINTER(FaDesc)]
    L.wave_cuda_flash_attention_fwd.argtypes = [C.POINTER(FaDesc), vp, vp, vp, vp, vp, vp]
    L.wave_cuda_flash_attention_fwd_host.argtypes = [C.POINTER(FaDesc), vp, vp, vp, vp, vp]
    L.wave_cuda_flash_attention_fwd_multi_output.argtypes = [C.POINTER(FaDesc), vp, vp, vp, C.POINTER(vp), C.c_int, vp, vp]
    L.wave_cuda_flash_attention_fwd_multicast_output.argtypes = [C.POINTER(FaDesc), vp, vp, vp, vp, vp, vp, vp]
    L.wave_cuda_module_get_function.argtypes = [C.c_char_p, vp, C.POINTER(vp)]
    L.wave_cuda_launch.argtypes = [vp, C.POINTER(vp), vp]
    L.wave_cuda_function_release.argtypes = [vp]
    L.wave_cuda_function_release.restype = None
    L.wave_cuda_check_device_status.argtypes = [ip]
    ll, sz = C.c_int64, C.c_size_t
    L.wave_cuda_module_blob_bytes.argtypes = [C.c_uint32, C.POINTER(sz)]
    L.wave_cuda_module_blob_write.argtypes = [C.c_uint32, vp, vp, sz]
    L.wave_cuda_mgpu_status.argtypes = []
    L.wave_cuda_memref_region.argtypes = [ll, vp, ll, C.POINTER(vp), C.POINTER(sz)]
    for name, res, args in [
            ("mgpuModuleLoad", vp, [vp, sz]), ("mgpuModuleUnload", None, [vp]),
            ("mgpuModuleGetFunction", vp, [vp, C.c_char_p]),
            ("mgpuLaunchKernel", None, [vp, ll, ll, ll, ll, ll, ll, C.c_int32, vp, C.POINTER(vp), C.POINTER(vp), sz]),
            ("mgpuStreamCreate", vp, []), ("mgpuStreamDestroy", None, [vp]), ("mgpuStreamSynchronize", None, [vp]),
            ("mgpuStreamWaitEvent", None, [vp, vp]), ("mgpuEventCreate", vp, []), ("mgpuEventDestroy", None, [vp]),
            ("mgpuEventSynchronize", None, [vp]), ("mgpuEventRecord", None, [vp, vp]),
            ("mgpuMemAlloc", vp, [C.c_uint64, vp, C.c_uint8]), ("mgpuMemFree", None, [vp, vp]),
            ("mgpuMemcpy", None, [vp, vp, sz, vp]), ("mgpuMemset32", None, [vp, C.c_uint, sz, vp]),
            ("mgpuMemset16", None, [vp, C.c_ushort, sz, vp]), ("mgpuMemHostRegister", None, [vp, C.c_uint64]),
            ("mgpuMemHostUnregister", None, [vp]), ("mgpuMemHostRegisterMemRef", None, [ll, vp, ll]),
            ("mgpuMemHostUnregisterMemRef", None, [ll, vp, ll]), ("mgpuSetDefaultDevice", None, [C.c_int32])]:
        getattr(L, name).restype = res
        getattr(L, name).argtypes = args
    _lib = L
    return L


def module_blob(kind: int, desc) -> bytes:
    """The bytes a host module carries in place of a device code object: a
    header and the kernel's descriptor (include/wave_mgpu.h)."""
    n = C.c_size_t(0)
    if lib().wave_cuda_module_blob_bytes(kind, C.byref(n)) != OK:
        raise ValueError(f"unknown blob kind {kind}")
    buf = C.create_string_buffer(n.value)
    check(lib().wave_cuda_module_blob_write(kind, C.byref(desc), buf, n.value))
    return buf.raw


def reload_env() -> None:
    """Has the library read its WAVE_CUDA_* environment knobs again (it reads
    them once by itself); call after changing os.environ."""
    lib().wave_cuda_reload_env()


def check(rc: int) -> None:
    if rc != OK:
        raise WaveCudaError(rc, lib().wave_cuda_last_error().decode())


def gemm_desc(M: int, N: int, K: int, *, bm: int = 1, bn: int = 2, wave_m_tiles: int = 1, wave_n_tiles: int = 1,
              wave_k_tiles: int = 1, in_type: int = F16, out_type: int = F32, out_layout: int = ROW_MAJOR,
              cta_group_m: int = 1, streamk_workers: int = 1, ldc: int = 0) -> GemmDesc:
    return GemmDesc(M, N, K, bm, bn, wave_m_tiles, wave_n_tiles, wave_k_tiles, in_type, out_type, out_layout,
                    cta_group_m, streamk_workers, ldc)


def gemm_validate(desc: GemmDesc) -> None:
    check(lib().wave_cuda_gemm_validate(C.byref(desc)))


def gemm_workspace_bytes(desc: GemmDesc) -> tuple[int, int]:
    s, c = C.c_size_t(0), C.c_size_t(0)
    check(lib().wave_cuda_gemm_workspace_bytes(C.byref(desc), C.byref(s), C.byref(c)))
    return s.value, c.value


def gemm_plan(desc: GemmDesc) -> dict:
    v = [C.c_int(0) for _ in range(5)]
    check(lib().wave_cuda_gemm_plan(C.byref(desc), *[C.byref(x) for x in v]))
    return dict(tile_m=v[0].value, tile_n=v[1].value, grid=v[2].value, streamk_workers=v[3].value,
                swapped=bool(v[4].value))


def gemm_plan_for_sms(desc: GemmDesc, sm_count: int, have_workspace: bool = True) -> dict:
    """The launch the backend would choose on a GPU of `sm_count` SMs (no device needed)."""
    v = [C.c_int(0) for _ in range(5)]
    s, c = C.c_size_t(0), C.c_size_t(0)
    check(lib().wave_cuda_gemm_plan_for_sms(C.byref(desc), sm_count, int(have_workspace), *[C.byref(x) for x in v],
                                            C.byref(s), C.byref(c)))
    return dict(tile_m=v[0].value, tile_n=v[1].value, grid=v[2].value, streamk_workers=v[3].value,
                swapped=bool(v[4].value), scratch_bytes=s.value, counter_bytes=c.value)


def gemm(desc: GemmDesc, a_ptr: int, b_ptr: int, c_ptr: int, workspace_ptr: int = 0, stream: int = 0) -> None:
    check(lib().wave_cuda_gemm(C.byref(desc), a_ptr, b_ptr, c_ptr, workspace_ptr or None, stream or None))


STATIC_WORKSPACE_BYTES = 8 * 1024 * 1024


def gemm_streamk_static(desc: GemmDesc, a_ptr: int, b_ptr: int, c_ptr: int, stream: int = 0) -> None:
    """Stream-K GEMM on the library's built-in workspace, for callers that
    cannot pass or allocate one; see include/wave_cuda.h for its limits."""
    check(lib().wave_cuda_gemm_streamk_static(C.byref(desc), a_ptr, b_ptr, c_ptr, stream or None))


def gemm_host(desc: GemmDesc, a_ptr: int, b_ptr: int, c_ptr: int, stream: int = 0) -> None:
    check(lib().wave_cuda_gemm_host(C.byref(desc), a_ptr, b_ptr, c_ptr, stream or None))


def gemm_multi_output(desc: GemmDesc, a_ptr: int, b_ptr: int, c_ptrs, stream: int = 0) -> None:
    """The GEMM with C written to every buffer of `c_ptrs` (the first as usual,
    the others tile by tile out of the epilogue): the fused all-gather of a
    column-sharded GEMM when the others are peer GPUs' copies of C."""
    arr = (C.c_void_p * len(c_ptrs))(*c_ptrs)
    check(lib().wave_cuda_gemm_multi_output(C.byref(desc), a_ptr, b_ptr, arr, len(c_ptrs), stream or None))


def gemm_multicast_output(desc: GemmDesc, a_ptr: int, b_ptr: int, c_local_ptr: int, c_multicast_ptr: int,
                          stream: int = 0) -> None:
    """The GEMM with C also written through an NVLink multicast address (NVLS): every GPU bound to
    the multicast object receives each finished tile."""
    check(lib().wave_cuda_gemm_multicast_output(C.byref(desc), a_ptr, b_ptr, c_local_ptr, c_multicast_ptr,
                                                stream or None))


def gemm_host_a_resident(desc: GemmDesc, a_dev_ptr: int, b_ptr: int, c_ptr: int, stream: int = 0) -> None:
    """Host-buffer GEMM of one rank's column block with the replicated A already on the device."""
    check(lib().wave_cuda_gemm_host_a_resident(C.byref(desc), a_dev_ptr, b_ptr, c_ptr, stream or None))


def fa_desc(batch: int, heads: int, seq_q: int, seq_k: int, head_dim: int = 128, *, scale: float = 0.0,
            causal: bool = False, io_type: int = BF16, out_f32: bool = False, qk_max_abs: float = 0.0) -> FaDesc:
    """`qk_max_abs` > 0 selects the fixed-reference softmax (a bound on |q| and |k| entries)."""
    return FaDesc(batch, heads, seq_q, seq_k, head_dim, scale, int(causal), io_type, int(out_f32), qk_max_abs)


def fa_validate(desc: FaDesc) -> None:
    check(lib().wave_cuda_fa_validate(C.byref(desc)))


def flash_attention_fwd(desc: FaDesc, q_ptr: int, k_ptr: int, v_ptr: int, o_ptr: int, lse_ptr: int = 0,
                        stream: int = 0) -> None:
    check(lib().wave_cuda_flash_attention_fwd(C.byref(desc), q_ptr, k_ptr, v_ptr, o_ptr, lse_ptr or None,
                                              stream or None))


def flash_attention_fwd_multi_output(desc: FaDesc, q_ptr: int, k_ptr: int, v_ptr: int, o_ptrs, lse_ptr: int = 0,
                                     stream: int = 0) -> None:
    """The forward with O written to every buffer of `o_ptrs` (the first as usual, the others 16 bytes
    at a time out of the epilogue): the gather of (batch, head)-sharded attention inside the kernel
    when the others are peer GPUs' copies of O."""
    arr = (C.c_void_p * len(o_ptrs))(*o_ptrs)
    check(lib().wave_cuda_flash_attention_fwd_multi_output(C.byref(desc), q_ptr, k_ptr, v_ptr, arr, len(o_ptrs),
                                                           lse_ptr or None, stream or None))


def flash_attention_fwd_multicast_output(desc: FaDesc, q_ptr: int, k_ptr: int, v_ptr: int, o_local_ptr: int,
                                         o_multicast_ptr: int, lse_ptr: int = 0, stream: int = 0) -> None:
    """The same through one NVLink multicast address (multimem.st)."""
    check(lib().wave_cuda_flash_attention_fwd_multicast_output(C.byref(desc), q_ptr, k_ptr, v_ptr, o_local_ptr,
                                                               o_multicast_ptr, lse_ptr or None, stream or None))


def flash_attention_fwd_host(desc: FaDesc, q_ptr: int, k_ptr: int, v_ptr: int, o_ptr: int, stream: int = 0) -> None:
    check(lib().wave_cuda_flash_attention_fwd_host(C.byref(desc), q_ptr, k_ptr, v_ptr, o_ptr, stream or None))


def check_device_status() -> None:
    out = (C.c_int * 4)()
    check(lib().wave_cuda_check_device_status(out))
