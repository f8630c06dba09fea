#include "fa_sm100.h"
namespace wave {
__device__ int g_fa_status[4];
int launch_flash_attention(const FaParams &, const void *, const void *, const void *, int, cudaStream_t) {
  return -2;
}
cudaError_t fa_read_status(int out[4], bool clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fa_status, sizeof(int) * 4);
  if (err == cudaSuccess && clear) {
    int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(g_fa_status, zero, sizeof(zero));
  }
  return err;
}
} // namespace wave
