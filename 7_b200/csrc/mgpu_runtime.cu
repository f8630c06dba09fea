// mgpu* wrappers for host modules run by mlir-runner (see include/wave_mgpu.h).
// Everything here sits on the public C ABI of wave_cuda.h and the CUDA
// runtime; the only kernel in this file is the pattern fill behind mgpuMemset.
#include "../../include/wave_cuda.h"
#include "../../include/wave_mgpu.h"

#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

template <typename T> __global__ void fill_kernel(T *dst, T value, size_t count) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    dst[i] = value;
}

std::atomic<int> g_first_failure{0};

void record(const char *call, int code, const char *message) {
  std::fprintf(stderr, "'%s' failed with '%s'\n", call, message ? message : "unknown error");
  int expected = 0;
  g_first_failure.compare_exchange_strong(expected, code);
}

// Reports a failed CUDA runtime call; returns true when it failed.
bool cuda_failed(const char *call, cudaError_t err) {
  if (err == cudaSuccess)
    return false;
  record(call, WAVE_E_CUDA, cudaGetErrorString(err));
  return true;
}

bool wave_failed(const char *call, int rc) {
  if (rc == WAVE_OK)
    return false;
  record(call, rc, wave_cuda_last_error());
  return true;
}

struct Function;

struct Module {
  uint32_t kind;
  wave_gemm_desc gemm;
  wave_fa_desc fa;
  std::mutex lock;
  std::vector<Function *> functions; // owned; released by mgpuModuleUnload
};

struct Function {
  const Module *module;
  void *fn; // handle of the name-based facade
};

size_t desc_bytes_of(uint32_t kind) {
  return kind == WAVE_BLOB_GEMM ? sizeof(wave_gemm_desc) : kind == WAVE_BLOB_FA ? sizeof(wave_fa_desc) : 0;
}

// True when the pointer is plain or registered host memory (what
// gpu.host_register leaves the kernel arguments pointing at).
bool is_host_pointer(const void *ptr) {
  cudaPointerAttributes attr{};
  if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
    cudaGetLastError(); // older runtimes fail on unregistered host memory: clear, treat as host
    return true;
  }
  return attr.type == cudaMemoryTypeHost || attr.type == cudaMemoryTypeUnregistered;
}

// The range of bytes a strided memref descriptor addresses:
// {allocated, aligned, offset, sizes[rank], strides[rank]}.  Element (i_0, ...)
// lies at aligned + (offset + sum i_d * stride_d) * elem, so a dimension with a
// negative stride reaches BELOW the element at index zero: the lowest and the
// highest addressed element are found separately and the region between them
// is what gets registered.
void memref_region(int64_t rank, void *descriptor, int64_t elem, char **first, size_t *bytes) {
  char **ptrs = static_cast<char **>(descriptor);
  const int64_t *ints = reinterpret_cast<const int64_t *>(ptrs + 2);
  const int64_t offset = ints[0];
  const int64_t *sizes = ints + 1, *strides = ints + 1 + rank;
  int64_t lowest = 0, highest = 0; // element offsets relative to the element at index zero
  bool empty = false;
  for (int64_t i = 0; i < rank; ++i) {
    if (sizes[i] <= 0) {
      empty = true;
      continue;
    }
    const int64_t reach = (sizes[i] - 1) * strides[i];
    if (reach < 0)
      lowest += reach;
    else
      highest += reach;
  }
  *first = ptrs[1] + (offset + (empty ? 0 : lowest)) * elem;
  *bytes = empty ? 0 : static_cast<size_t>(highest - lowest + 1) * static_cast<size_t>(elem);
}

} // namespace

extern "C" {

int wave_cuda_mgpu_status(void) { return g_first_failure.exchange(0); }

int wave_cuda_memref_region(int64_t rank, void *descriptor, int64_t elem_bytes, void **first, size_t *bytes) {
  if (rank < 0 || !descriptor || elem_bytes <= 0 || !first || !bytes)
    return WAVE_E_INVALID;
  char *lo = nullptr;
  memref_region(rank, descriptor, elem_bytes, &lo, bytes);
  *first = lo;
  return WAVE_OK;
}

int wave_cuda_module_blob_bytes(uint32_t kind, size_t *bytes) {
  const size_t d = desc_bytes_of(kind);
  if (!bytes || d == 0)
    return WAVE_E_INVALID;
  *bytes = sizeof(wave_cuda_module_blob) + d;
  return WAVE_OK;
}

int wave_cuda_module_blob_write(uint32_t kind, const void *desc, void *out, size_t out_bytes) {
  size_t need = 0;
  if (!desc || !out || wave_cuda_module_blob_bytes(kind, &need) != WAVE_OK || out_bytes < need)
    return WAVE_E_INVALID;
  const int rc = kind == WAVE_BLOB_GEMM ? wave_cuda_gemm_validate(static_cast<const wave_gemm_desc *>(desc))
                                        : wave_cuda_fa_validate(static_cast<const wave_fa_desc *>(desc));
  if (rc != WAVE_OK)
    return rc;
  wave_cuda_module_blob head{};
  std::memcpy(head.magic, "WAVECUDA", 8);
  head.version = WAVE_BLOB_VERSION;
  head.kind = kind;
  head.desc_bytes = static_cast<uint32_t>(desc_bytes_of(kind));
  std::memcpy(out, &head, sizeof(head));
  std::memcpy(static_cast<char *>(out) + sizeof(head), desc, head.desc_bytes);
  return WAVE_OK;
}

void *mgpuModuleLoad(void *data, size_t gpuBlobSize) {
  wave_cuda_module_blob head{};
  if (!data || (gpuBlobSize != 0 && gpuBlobSize < sizeof(head))) {
    record("mgpuModuleLoad", WAVE_E_INVALID, "blob is null or shorter than its header");
    return nullptr;
  }
  std::memcpy(&head, data, sizeof(head));
  if (std::memcmp(head.magic, "WAVECUDA", 8) != 0) {
    record("mgpuModuleLoad", WAVE_E_INVALID,
           "blob does not start with WAVECUDA: this runtime takes kernel descriptors, not device code objects");
    return nullptr;
  }
  if (head.version != WAVE_BLOB_VERSION || desc_bytes_of(head.kind) == 0 ||
      head.desc_bytes != desc_bytes_of(head.kind) ||
      (gpuBlobSize != 0 && gpuBlobSize < sizeof(head) + head.desc_bytes)) {
    record("mgpuModuleLoad", WAVE_E_INVALID, "blob version, kind or descriptor size not understood");
    return nullptr;
  }
  Module *m = new Module{};
  m->kind = head.kind;
  const char *body = static_cast<const char *>(data) + sizeof(head);
  if (head.kind == WAVE_BLOB_GEMM)
    std::memcpy(&m->gemm, body, sizeof(m->gemm));
  else
    std::memcpy(&m->fa, body, sizeof(m->fa));
  return m;
}

void mgpuModuleUnload(void *module) {
  Module *m = static_cast<Module *>(module);
  if (!m)
    return;
  for (Function *f : m->functions) {
    wave_cuda_function_release(f->fn);
    delete f;
  }
  delete m;
}

void *mgpuModuleGetFunction(void *module, const char *name) {
  if (!module || !name) {
    record("mgpuModuleGetFunction", WAVE_E_INVALID, "module and name must be non-null");
    return nullptr;
  }
  Module *m = static_cast<Module *>(module);
  const bool fa_name = std::strncmp(name, "flash_attention", 15) == 0;
  if (fa_name != (m->kind == WAVE_BLOB_FA)) {
    record("mgpuModuleGetFunction", WAVE_E_NOT_FOUND, "the module's descriptor is of the other kernel family");
    return nullptr;
  }
  void *fn = nullptr;
  const void *desc = m->kind == WAVE_BLOB_GEMM ? static_cast<const void *>(&m->gemm) : &m->fa;
  if (wave_failed("mgpuModuleGetFunction", wave_cuda_module_get_function(name, desc, &fn)))
    return nullptr;
  Function *f = new Function{m, fn};
  std::lock_guard<std::mutex> guard(m->lock);
  m->functions.push_back(f);
  return f;
}

void mgpuLaunchKernel(void *function, intptr_t gridX, intptr_t gridY, intptr_t gridZ, intptr_t, intptr_t, intptr_t,
                      int32_t, void *stream, void **params, void **, size_t paramsCount) {
  if (!function || !params) {
    record("mgpuLaunchKernel", WAVE_E_INVALID, "function and params must be non-null");
    return;
  }
  Function *f = static_cast<Function *>(function);
  const Module &m = *f->module;
  // The block shape and the dynamic shared memory are the AMD kernel's; the
  // grid is the host's statement of the problem size and must agree with the
  // descriptor the module was built from.
  intptr_t want_x, want_y;
  if (m.kind == WAVE_BLOB_GEMM) {
    want_x = m.gemm.M / (16 * m.gemm.bm * m.gemm.wave_m_tiles);
    want_y = m.gemm.N / (16 * m.gemm.bn * m.gemm.wave_n_tiles);
  } else {
    want_x = (m.fa.seq_q + 255) / 256;
    want_y = static_cast<intptr_t>(m.fa.batch) * m.fa.heads;
  }
  if (gridX != want_x || gridY != want_y || gridZ != 1) {
    char text[160];
    std::snprintf(text, sizeof(text), "grid %ld,%ld,%ld does not match the module's descriptor (%ld,%ld,1)",
                  static_cast<long>(gridX), static_cast<long>(gridY), static_cast<long>(gridZ),
                  static_cast<long>(want_x), static_cast<long>(want_y));
    record("mgpuLaunchKernel", WAVE_E_INVALID, text);
    return;
  }
  if (paramsCount != 4) {
    record("mgpuLaunchKernel", WAVE_E_INVALID, "expected 4 kernel parameters ({A,B,C,trip} or {Q,K,V,O})");
    return;
  }
  void *p0 = *static_cast<void **>(params[0]), *p1 = *static_cast<void **>(params[1]),
       *p2 = *static_cast<void **>(params[2]);
  const bool host0 = is_host_pointer(p0), host1 = is_host_pointer(p1), host2 = is_host_pointer(p2);
  if (m.kind == WAVE_BLOB_GEMM) {
    if (host0 != host1 || host0 != host2) {
      record("mgpuLaunchKernel", WAVE_E_INVALID, "A, B and C must all be host or all be device memory");
      return;
    }
    if (!host0) {
      wave_failed("mgpuLaunchKernel", wave_cuda_launch(f->fn, params, stream));
      return;
    }
    const int trip = *static_cast<int *>(params[3]);
    if (trip != m.gemm.K / (16 * m.gemm.wave_k_tiles) - 1) { // wave_matmul.py:6964
      record("mgpuLaunchKernel", WAVE_E_INVALID, "trip count does not match K/(16*wave_k_tiles)-1");
      return;
    }
    wave_gemm_desc d = m.gemm;
    d.streamk_workers = 1; // this argument list has no workspace
    wave_failed("mgpuLaunchKernel", wave_cuda_gemm_host(&d, p0, p1, p2, stream));
    return;
  }
  void *p3 = *static_cast<void **>(params[3]);
  const bool host3 = is_host_pointer(p3);
  if (host0 != host1 || host0 != host2 || host0 != host3) {
    record("mgpuLaunchKernel", WAVE_E_INVALID, "Q, K, V and O must all be host or all be device memory");
    return;
  }
  if (!host0)
    wave_failed("mgpuLaunchKernel", wave_cuda_launch(f->fn, params, stream));
  else
    wave_failed("mgpuLaunchKernel", wave_cuda_flash_attention_fwd_host(&m.fa, p0, p1, p2, p3, stream));
}

void *mgpuStreamCreate(void) {
  cudaStream_t s = nullptr;
  if (cuda_failed("mgpuStreamCreate", cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking)))
    return nullptr;
  return s;
}

void mgpuStreamDestroy(void *stream) {
  cuda_failed("mgpuStreamDestroy", cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
}

void mgpuStreamSynchronize(void *stream) {
  cuda_failed("mgpuStreamSynchronize", cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
}

void mgpuStreamWaitEvent(void *stream, void *event) {
  cuda_failed("mgpuStreamWaitEvent",
              cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
}

void *mgpuEventCreate(void) {
  cudaEvent_t e = nullptr;
  if (cuda_failed("mgpuEventCreate", cudaEventCreateWithFlags(&e, cudaEventDisableTiming)))
    return nullptr;
  return e;
}

void mgpuEventDestroy(void *event) { cuda_failed("mgpuEventDestroy", cudaEventDestroy(static_cast<cudaEvent_t>(event))); }

void mgpuEventSynchronize(void *event) {
  cuda_failed("mgpuEventSynchronize", cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
}

void mgpuEventRecord(void *event, void *stream) {
  cuda_failed("mgpuEventRecord", cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
}

void *mgpuMemAlloc(uint64_t sizeBytes, void *stream, uint8_t isHostShared) {
  void *ptr = nullptr;
  if (sizeBytes == 0)
    return nullptr;
  if (isHostShared) {
    if (cuda_failed("mgpuMemAlloc", cudaMallocManaged(&ptr, sizeBytes, cudaMemAttachGlobal)))
      return nullptr;
    return ptr;
  }
  (void)stream; // a plain allocation: what it returns is usable on every stream
  if (cuda_failed("mgpuMemAlloc", cudaMalloc(&ptr, sizeBytes)))
    return nullptr;
  return ptr;
}

void mgpuMemFree(void *ptr, void *stream) {
  if (!ptr)
    return;
  // Work queued on the stream may still use the buffer.
  if (stream && cuda_failed("mgpuMemFree", cudaStreamSynchronize(static_cast<cudaStream_t>(stream))))
    return;
  cuda_failed("mgpuMemFree", cudaFree(ptr));
}

void mgpuMemcpy(void *dst, void *src, size_t sizeBytes, void *stream) {
  cuda_failed("mgpuMemcpy", cudaMemcpyAsync(dst, src, sizeBytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)));
}

void mgpuMemset32(void *dst, unsigned int value, size_t count, void *stream) {
  if (count == 0)
    return;
  const unsigned blocks = static_cast<unsigned>(count / 256 + 1 < 1184 ? count / 256 + 1 : 1184);
  fill_kernel<unsigned int><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<unsigned int *>(dst),
                                                                                    value, count);
  cuda_failed("mgpuMemset32", cudaGetLastError());
}

void mgpuMemset16(void *dst, unsigned short value, size_t count, void *stream) {
  if (count == 0)
    return;
  const unsigned blocks = static_cast<unsigned>(count / 256 + 1 < 1184 ? count / 256 + 1 : 1184);
  fill_kernel<unsigned short><<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned short *>(dst), value, count);
  cuda_failed("mgpuMemset16", cudaGetLastError());
}

void mgpuMemHostRegister(void *ptr, uint64_t sizeBytes) {
  if (!ptr || sizeBytes == 0)
    return;
  cuda_failed("mgpuMemHostRegister", cudaHostRegister(ptr, sizeBytes, cudaHostRegisterDefault));
}

void mgpuMemHostUnregister(void *ptr) {
  if (ptr)
    cuda_failed("mgpuMemHostUnregister", cudaHostUnregister(ptr));
}

void mgpuMemHostRegisterMemRef(int64_t rank, void *descriptor, int64_t elementSizeBytes) {
  if (!descriptor || rank < 0 || elementSizeBytes <= 0) {
    record("mgpuMemHostRegisterMemRef", WAVE_E_INVALID, "descriptor, rank or element size not valid");
    return;
  }
  char *first = nullptr;
  size_t bytes = 0;
  memref_region(rank, descriptor, elementSizeBytes, &first, &bytes);
  mgpuMemHostRegister(first, bytes);
}

void mgpuMemHostUnregisterMemRef(int64_t rank, void *descriptor, int64_t elementSizeBytes) {
  if (!descriptor || rank < 0 || elementSizeBytes <= 0) {
    record("mgpuMemHostUnregisterMemRef", WAVE_E_INVALID, "descriptor, rank or element size not valid");
    return;
  }
  char *first = nullptr;
  size_t bytes = 0;
  memref_region(rank, descriptor, elementSizeBytes, &first, &bytes);
  if (bytes)
    mgpuMemHostUnregister(first);
}

void mgpuSetDefaultDevice(int32_t device) { cuda_failed("mgpuSetDefaultDevice", cudaSetDevice(device)); }

} // extern "C"
