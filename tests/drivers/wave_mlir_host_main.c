/* A host `main` of the shape the reference emits for mlir-runner
 * (python/mlir/dialects/wave_matmul.py:11244-11272), written out as plain C: the
 * calls are the ones gpu-to-llvm lowers that module to.  It is built with gcc
 * alone and linked against libwave_cuda.so only -- no CUDA header, no CUDA
 * library on the link line -- which is what a module JIT-compiled by
 * mlir-runner with --shared-libs=libwave_cuda.so sees.
 *
 *   host buffers -> fill (the reference's LCG, wave_matmul.py:828-836) -> zero C
 *   -> gpu.host_register -> wave_memref_to_ptr_global_* -> gpu.launch_func
 *   wmma_f16_matmul_tiled {A, B, C, trip} on grid M_blocks x N_blocks -> compare
 *   with the f32 dot products, k ascending (the --compare-cpu check of
 *   examples/wave/wmma_matmul_tiled.py) -> print like the example driver.
 *
 * Usage: wave_mlir_host_main [M N K bm bn wave_m_tiles wave_n_tiles wave_k_tiles seed]
 * Exit code 0 on a match, 1 on a mismatch or a runtime failure.
 */
#include "wave_cuda.h"
#include "wave_mgpu.h"

#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  void *allocated, *aligned;
  int64_t offset, size, stride;
} memref1d;

static void fill_lcg(_Float16 *out, size_t count, int seed, int stream) {
  uint32_t state = (uint32_t)seed ^ ((uint32_t)(stream + 1) * 0x9E3779B9u);
  for (size_t i = 0; i < count; ++i) {
    state = 1664525u * state + 1013904223u;
    out[i] = (_Float16)((float)((int)((state >> 24) % 17u) - 8) * 0.25f);
  }
}

int main(int argc, char **argv) {
  int v[9] = {32, 32, 64, 2, 2, 1, 1, 2, 7};
  for (int i = 1; i < argc && i <= 9; ++i)
    v[i - 1] = atoi(argv[i]);
  const int M = v[0], N = v[1], K = v[2];

  wave_gemm_desc desc;
  wave_cuda_gemm_desc_init(&desc, M, N, K);
  desc.bm = v[3];
  desc.bn = v[4];
  desc.wave_m_tiles = v[5];
  desc.wave_n_tiles = v[6];
  desc.wave_k_tiles = v[7];
  size_t blob_bytes = 0;
  wave_cuda_module_blob_bytes(WAVE_BLOB_GEMM, &blob_bytes);
  void *blob = malloc(blob_bytes);
  if (wave_cuda_module_blob_write(WAVE_BLOB_GEMM, &desc, blob, blob_bytes) != WAVE_OK) {
    fprintf(stderr, "%s\n", wave_cuda_last_error());
    return 2;
  }

  _Float16 *a = aligned_alloc(64, (size_t)M * K * 2), *b = aligned_alloc(64, (size_t)N * K * 2);
  float *c = aligned_alloc(64, (size_t)M * N * 4);
  fill_lcg(a, (size_t)M * K, v[8], 0);
  fill_lcg(b, (size_t)N * K, v[8], 1);
  memset(c, 0, (size_t)M * N * 4);
  memref1d ma = {a, a, 0, (int64_t)M * K, 1}, mb = {b, b, 0, (int64_t)N * K, 1}, mc = {c, c, 0, (int64_t)M * N, 1};
  mgpuMemHostRegisterMemRef(1, &ma, 2);
  mgpuMemHostRegisterMemRef(1, &mb, 2);
  mgpuMemHostRegisterMemRef(1, &mc, 4);
  void *pa = _mlir_ciface_wave_memref_to_ptr_global_f16(&ma), *pb = _mlir_ciface_wave_memref_to_ptr_global_f16(&mb),
       *pc = _mlir_ciface_wave_memref_to_ptr_global_f32(&mc);

  void *module = mgpuModuleLoad(blob, blob_bytes);
  void *function = module ? mgpuModuleGetFunction(module, "wmma_f16_matmul_tiled") : NULL;
  void *stream = mgpuStreamCreate();
  if (!function || !stream)
    return 1;
  int32_t trip = K / (16 * desc.wave_k_tiles) - 1;
  void *params[4] = {&pa, &pb, &pc, &trip};
  mgpuLaunchKernel(function, M / (16 * desc.bm * desc.wave_m_tiles), N / (16 * desc.bn * desc.wave_n_tiles), 1,
                   64 * desc.bm * desc.bn, 1, 1, 0, stream, params, NULL, 4);
  mgpuStreamSynchronize(stream);
  mgpuStreamDestroy(stream);
  mgpuModuleUnload(module);
  if (wave_cuda_mgpu_status() != 0 || wave_cuda_check_device_status(NULL) != WAVE_OK)
    return 1;

  size_t bad = 0;
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = 0.0f;
      for (int k = 0; k < K; ++k)
        acc += (float)a[(size_t)m * K + k] * (float)b[(size_t)n * K + k];
      if (c[(size_t)m * N + n] != acc && bad++ < 5)
        fprintf(stderr, "mismatch at (%d, %d): got %g, expected %g\n", m, n, c[(size_t)m * N + n], acc);
    }
  mgpuMemHostUnregisterMemRef(1, &ma, 2);
  mgpuMemHostUnregisterMemRef(1, &mb, 2);
  mgpuMemHostUnregisterMemRef(1, &mc, 4);
  if (bad) {
    fprintf(stderr, "CPU comparison failed: mismatches=%zu\n", bad);
    return 1;
  }
  printf("CPU comparison passed: elements=%zu\n", (size_t)M * N);
  return 0;
}
