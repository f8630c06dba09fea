"""B200 (sm_100a) backend for the Wave compiler's two dense kernels: the tiled
f16/bf16 GEMM and the flash-attention forward.

Layout of the package:
  csrc/            hand-written CUDA kernels and the C-ABI host code
  build.py         in-tree nvcc build of libwave_cuda.so
  wave_cuda.py     ctypes binding of the C ABI
  wave_matmul.py   host-side mirror of the reference's GEMM builder/driver API
  wave_attention.py host-side mirror of the reference's attention API

The directory name starts with a digit, so import it with
``importlib.import_module("7_b200")``.
"""
from . import wave_cuda  # noqa: F401
