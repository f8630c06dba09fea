/*
 * Host-only stand-in for <hip/hip_runtime.h>, used solely to compile the
 * reference's calibrate-runner sources on a machine without ROCm so that their
 * HOST arithmetic (input generators, CPU references) can be called as a
 * checker.  Every device entry point reports failure; nothing here launches
 * or emulates a kernel.  Test infrastructure only.
 */
#ifndef WAVE_REF_SHIM_HIP_RUNTIME_H
#define WAVE_REF_SHIM_HIP_RUNTIME_H
#include <cstddef>
#include <cstdint>

#ifndef __host__
#define __host__
#endif
#ifndef __device__
#define __device__
#endif
typedef int hipError_t;
enum { hipSuccess = 0, hipErrorNoDevice = 100 };
typedef void *hipModule_t;
typedef void *hipFunction_t;
typedef void *hipEvent_t;
typedef void *hipStream_t;
enum hipMemcpyKind { hipMemcpyHostToDevice = 1, hipMemcpyDeviceToHost = 2 };
enum hipFuncAttribute { hipFuncAttributeMaxDynamicSharedMemorySize = 8 };
struct hipDeviceProp_t {
  char name[256];
  char gcnArchName[256];
  int clockRate;
};

static inline const char *hipGetErrorString(hipError_t) {
  return "HIP is not available (host-only reference shim)";
}
#define WAVE_REF_SHIM_FAIL(name, ...)                                          \
  static inline hipError_t name(__VA_ARGS__) { return hipErrorNoDevice; }
WAVE_REF_SHIM_FAIL(hipDeviceSynchronize, void)
WAVE_REF_SHIM_FAIL(hipEventCreate, hipEvent_t *)
WAVE_REF_SHIM_FAIL(hipEventDestroy, hipEvent_t)
WAVE_REF_SHIM_FAIL(hipEventElapsedTime, float *, hipEvent_t, hipEvent_t)
WAVE_REF_SHIM_FAIL(hipEventRecord, hipEvent_t, hipStream_t)
WAVE_REF_SHIM_FAIL(hipEventSynchronize, hipEvent_t)
WAVE_REF_SHIM_FAIL(hipFree, void *)
WAVE_REF_SHIM_FAIL(hipGetDeviceProperties, hipDeviceProp_t *, int)
WAVE_REF_SHIM_FAIL(hipMalloc, void **, size_t)
WAVE_REF_SHIM_FAIL(hipMemcpy, void *, const void *, size_t, hipMemcpyKind)
WAVE_REF_SHIM_FAIL(hipMemset, void *, int, size_t)
WAVE_REF_SHIM_FAIL(hipModuleGetFunction, hipFunction_t *, hipModule_t,
                   const char *)
WAVE_REF_SHIM_FAIL(hipModuleLoad, hipModule_t *, const char *)
WAVE_REF_SHIM_FAIL(hipModuleUnload, hipModule_t)
WAVE_REF_SHIM_FAIL(hipFuncSetAttribute, const void *, hipFuncAttribute, int)
WAVE_REF_SHIM_FAIL(hipModuleLaunchKernel, hipFunction_t, unsigned, unsigned,
                   unsigned, unsigned, unsigned, unsigned, unsigned,
                   hipStream_t, void **, void **)
#undef WAVE_REF_SHIM_FAIL
template <class T> static inline hipError_t hipMalloc(T **p, size_t n) {
  return hipMalloc(reinterpret_cast<void **>(p), n);
}
static inline hipError_t hipEventRecord(hipEvent_t e) {
  return hipEventRecord(e, nullptr);
}
#endif
