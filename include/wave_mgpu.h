/* GPU runtime wrappers for host modules run by mlir-runner.
 *
 * The reference runs the host `main` it emits (python/mlir/dialects/
 * wave_matmul.py:11244-11272: allocate, fill, gpu.host_register, one
 * gpu.launch_func, print) with three shared libraries: MLIR's
 * libmlir_rocm_runtime.so (the mgpu* wrappers that gpu-to-llvm calls),
 * libmlir_runner_utils.so (printMemrefF32/F16, host only) and its own
 * libwave_runtime.so (the reference's README.md:99-106 and the RUN lines of
 * the .mlir files under its test/Integration).
 * libwave_cuda.so stands in for the first and the third: it exports the
 * seven pointer helpers of runtime/wave_runtime.cpp:46-74 (wave_cuda.h) and
 * the mgpu* entry points below with MLIR's names and argument lists, so a
 * lowered host module links against it unchanged.  libmlir_runner_utils.so is
 * host code and stays as it is.
 *
 * What differs from a code-object runtime: there is no device binary per
 * kernel.  The blob that gpu.binary carries and mgpuModuleLoad receives is a
 * wave_cuda_module_blob: a header and the wave_gemm_desc or wave_fa_desc of the
 * kernel (written by wave_cuda_module_blob_write).  mgpuModuleGetFunction takes
 * the reference's kernel names, and mgpuLaunchKernel checks the grid the host
 * computed against the descriptor (wave_matmul.py:426-444: M_blocks x N_blocks;
 * wave_flash_attention.py:91-93: sequence/256 x batch*heads) and runs the
 * kernel with the reference's argument block ({&A,&B,&C,&trip} or {&Q,&K,&V,&O}).
 * Pointers into host memory (the reference registers its host buffers instead
 * of copying them, wave_matmul.py:6926-6937) are served by the host-buffer
 * entry points, which stage them through device memory.
 *
 * The wrappers return nothing, like MLIR's.  A failure is written to stderr as
 * "'<call>' failed with '<message>'" and recorded; wave_cuda_mgpu_status()
 * returns the first recorded code since its last call (0 if none) and clears it.
 */
#ifndef WAVE_MGPU_H
#define WAVE_MGPU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WAVE_BLOB_GEMM 0u
#define WAVE_BLOB_FA 1u
#define WAVE_BLOB_VERSION 1u

typedef struct wave_cuda_module_blob {
  char magic[8];       /* "WAVECUDA" */
  uint32_t version;    /* WAVE_BLOB_VERSION */
  uint32_t kind;       /* WAVE_BLOB_GEMM or WAVE_BLOB_FA */
  uint32_t desc_bytes; /* sizeof(wave_gemm_desc) or sizeof(wave_fa_desc) */
  uint32_t reserved;   /* 0 */
  /* desc_bytes bytes of descriptor follow */
} wave_cuda_module_blob;

/* Size of a blob of this kind, and a writer for it (validates the descriptor). */
int wave_cuda_module_blob_bytes(uint32_t kind, size_t *bytes);
int wave_cuda_module_blob_write(uint32_t kind, const void *desc, void *out, size_t out_bytes);
int wave_cuda_mgpu_status(void);
/* The host range mgpuMemHostRegisterMemRef / ...UnregisterMemRef act on for a
 * ranked memref descriptor {allocated, aligned, offset, sizes[rank],
 * strides[rank]} of `elem_bytes`-byte elements: from the lowest to the highest
 * addressed element (strides may be negative), `bytes` = 0 for an empty
 * memref.  Needs no GPU.  (MLIR's own wrapper, mgpuMemHostRegisterMemRef in
 * mlir/lib/ExecutionEngine/CudaRuntimeWrappers.cpp, assumes dense row-major.) */
int wave_cuda_memref_region(int64_t rank, void *descriptor, int64_t elem_bytes, void **first, size_t *bytes);

/* ---- MLIR's wrapper API (names and argument lists as gpu-to-llvm emits them) */
void *mgpuModuleLoad(void *data, size_t gpuBlobSize);
void mgpuModuleUnload(void *module);
void *mgpuModuleGetFunction(void *module, const char *name);
void mgpuLaunchKernel(void *function, intptr_t gridX, intptr_t gridY, intptr_t gridZ, intptr_t blockX,
                      intptr_t blockY, intptr_t blockZ, int32_t smem, void *stream, void **params, void **extra,
                      size_t paramsCount);
void *mgpuStreamCreate(void);
void mgpuStreamDestroy(void *stream);
void mgpuStreamSynchronize(void *stream);
void mgpuStreamWaitEvent(void *stream, void *event);
void *mgpuEventCreate(void);
void mgpuEventDestroy(void *event);
void mgpuEventSynchronize(void *event);
void mgpuEventRecord(void *event, void *stream);
void *mgpuMemAlloc(uint64_t sizeBytes, void *stream, uint8_t isHostShared);
void mgpuMemFree(void *ptr, void *stream);
void mgpuMemcpy(void *dst, void *src, size_t sizeBytes, void *stream);
void mgpuMemset32(void *dst, unsigned int value, size_t count, void *stream);
void mgpuMemset16(void *dst, unsigned short value, size_t count, void *stream);
void mgpuMemHostRegister(void *ptr, uint64_t sizeBytes);
void mgpuMemHostUnregister(void *ptr);
/* `descriptor` is a StridedMemRefType<char, rank>: {allocated, aligned, offset, sizes[rank], strides[rank]}. */
void mgpuMemHostRegisterMemRef(int64_t rank, void *descriptor, int64_t elementSizeBytes);
void mgpuMemHostUnregisterMemRef(int64_t rank, void *descriptor, int64_t elementSizeBytes);
void mgpuSetDefaultDevice(int32_t device);

#ifdef __cplusplus
}
#endif
#endif /* WAVE_MGPU_H */
