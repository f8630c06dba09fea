// Stream-K GEMM for callers that cannot hand the library a workspace.
//
// The Stream-K form of the GEMM needs global memory beyond A, B and C: f32
// partial tiles and one arrival counter per output tile.  wave_cuda_gemm takes
// that memory from the caller.  Some callers have none to give and no way to
// get any:
//   * a host program written against the reference's plain kernel argument
//     list {A, B, C, trip} -- what an mlir-runner host module or the calibrate
//     runner's "matmul" ABI passes -- has no slot for a workspace pointer;
//   * a process whose device memory is entirely owned by another allocator (a
//     serving runtime that reserved the whole GPU at start-up) gets
//     out-of-memory from cudaMalloc even though the GPU is otherwise idle;
//   * code on a path where a device allocation is not allowed to happen
//     (allocation may synchronise the device or fail, neither of which such a
//     path can tolerate).
// For them this file keeps ONE fixed area in the library's own device image: a
// file-scope `static __device__` array that every GPU loading the library
// holds until the process exits.  The entry point below lays the partial tiles
// and the counters out inside that area, clears the counters on the caller's
// stream, and runs the ordinary Stream-K kernel with the area as its
// workspace.  It calls no cudaMalloc, cudaFree or other allocating routine.
//
// Limits and rules:
//   * capacity WAVE_CUDA_STATIC_WORKSPACE_BYTES (8 MiB); a descriptor with an
//     explicit worker count whose partial tiles and counters need more is
//     refused with WAVE_E_INVALID.  With streamk_workers = 0 the caller left
//     the choice to the library: if the automatic Stream-K plan does not fit,
//     the launch runs as whole tiles instead (no workspace, still no
//     allocation), with the same results;
//   * the first call on each device looks the area's device address up
//     (cudaGetSymbolAddress) with that device current; make that first call
//     before any stream capture begins;
//   * all calls share the one area, which keeps whatever the previous call left
//     in it: the counters are cleared on every call, the partial tiles are
//     always written before they are read; two calls whose kernels overlap on
//     the GPU (different streams, or different host threads) race on it --
//     serialise them.
#include "../../include/wave_cuda.h"
#include "gemm_sm100.h"

#include <cstdio>
#include <mutex>

namespace wave {
void set_last_error(const char *message); // wave_cuda_backend.cu
}

namespace {

static __device__ __align__(256) unsigned char g_static_workspace[WAVE_CUDA_STATIC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
void *g_workspace_addr[kMaxDevices]; // device address of g_static_workspace, per device ordinal

int fail_msg(int code, const char *fmt, size_t a, size_t b, int c) {
  char buf[400];
  snprintf(buf, sizeof buf, fmt, a, b, c);
  wave::set_last_error(buf);
  return code;
}

// In host code `g_static_workspace` is only a handle for the runtime, not a
// device address; the address the kernel must be given comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int workspace_for_current_device(void **out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    wave::set_last_error(err != cudaSuccess ? cudaGetErrorString(err) : "device ordinal out of range");
    return WAVE_E_CUDA;
  }
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (!g_workspace_addr[dev]) {
    void *ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_workspace);
    if (err != cudaSuccess || !ptr) {
      wave::set_last_error(err != cudaSuccess ? cudaGetErrorString(err)
                                              : "cudaGetSymbolAddress returned a null address");
      return WAVE_E_CUDA;
    }
    g_workspace_addr[dev] = ptr;
  }
  *out = g_workspace_addr[dev];
  return WAVE_OK;
}

} // namespace

extern "C" int wave_cuda_gemm_streamk_static(const wave_gemm_desc *desc, const void *A, const void *B, void *C,
                                             void *stream) {
  size_t scratch = 0, counters = 0;
  int rc = wave_cuda_gemm_workspace_bytes(desc, &scratch, &counters); // validates the descriptor too
  if (rc != WAVE_OK)
    return rc;
  if (scratch + counters > static_cast<size_t>(WAVE_CUDA_STATIC_WORKSPACE_BYTES) && desc->streamk_workers == 0)
    return wave_cuda_gemm(desc, A, B, C, nullptr, stream); // automatic plan too large: whole tiles, no workspace
  if (scratch + counters > static_cast<size_t>(WAVE_CUDA_STATIC_WORKSPACE_BYTES))
    return fail_msg(WAVE_E_INVALID,
                    "this Stream-K launch needs %zu bytes of partial tiles and counters but the built-in "
                    "workspace holds %zu (streamk_workers=%d): use fewer workers or narrower tiles, or call "
                    "wave_cuda_gemm with a workspace of your own",
                    scratch + counters, static_cast<size_t>(WAVE_CUDA_STATIC_WORKSPACE_BYTES),
                    desc->streamk_workers);
  void *area = nullptr;
  if ((rc = workspace_for_current_device(&area)) != WAVE_OK)
    return rc;
  if (counters > 0) {
    // The previous call (perhaps one that was cut short) may have left counts
    // behind; the partial tiles need no clearing, each is written before it is read.
    cudaError_t err = cudaMemsetAsync(static_cast<char *>(area) + scratch, 0, counters,
                                      static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) {
      wave::set_last_error(cudaGetErrorString(err));
      return WAVE_E_CUDA;
    }
  }
  return wave_cuda_gemm(desc, A, B, C, (scratch + counters) ? area : nullptr, stream);
}
