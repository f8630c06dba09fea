// Device helpers shared by the flash-attention forward kernels.
#pragma once
#include "fa_sm100.h"
#include "sm100_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace wave {
namespace fa_detail {

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// 2^x for a pair of values on the FMA pipe instead of the special-function
// unit: round-to-nearest split x = n + f with |f| <= 0.5 (adding 1.5*2^23 leaves
// n in the low mantissa bits), a degree-3 minimax polynomial for 2^f (maximum
// relative error 7.6e-5, far below the 2^-9 of the 16-bit rounding that
// follows), then n is added to the exponent field.  Arguments below -125 are
// clamped (the result is then ~2^-125, which rounds away in every use here).
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  x.x = fmaxf(x.x, -125.0f);
  x.y = fmaxf(x.y, -125.0f);
  const float2 t = __fadd2_rn(x, make_float2(12582912.0f, 12582912.0f));
  const float2 n = __fadd2_rn(t, make_float2(-12582912.0f, -12582912.0f));
  const float2 f = __ffma2_rn(n, make_float2(-1.0f, -1.0f), x);
  float2 q = __ffma2_rn(f, make_float2(0.05520550534129143f, 0.05520550534129143f),
                        make_float2(0.24261397123336792f, 0.24261397123336792f));
  q = __ffma2_rn(q, f, make_float2(0.6932547688484192f, 0.6932547688484192f));
  q = __ffma2_rn(q, f, make_float2(0.9999276995658875f, 0.9999276995658875f));
  float2 r;
  r.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
  return r;
}

// Which of the 64 column pairs of a row take the polynomial path: kPoly of
// every 8, spread evenly so that FMA-pipe and special-function work interleave.
template <int kPoly> __device__ __forceinline__ constexpr bool pair_uses_poly(int i) {
  return ((i + 1) * kPoly) / 8 > (i * kPoly) / 8;
}

// The epilogue's 16-byte store of a piece of O repeated into the further output
// buffers of a launch (peer GPUs' copies of O, or one multicast address).
// `ex` must be a __grid_constant__ kernel parameter (its array is indexed in place).
__device__ __forceinline__ void store_extra_16B(const FaExtra &ex, size_t byte_offset, const uint4 &v) {
  if (ex.multimem) {
    multimem_st_16B(static_cast<uint8_t *>(ex.o[0]) + byte_offset, v);
    return;
  }
#pragma unroll 1
  for (int x = 0; x < ex.n; ++x)
    *reinterpret_cast<uint4 *>(static_cast<uint8_t *>(ex.o[x]) + byte_offset) = v;
}

// Bytes of shared memory the kernel variants with further output buffers add:
// a 2 KB slot per softmax warp (eight of them) for store_extra_chunk_16bit.
constexpr int kExtraStageBytes = 8 * 2048;

// One 32-column chunk of 16-bit O (64 bytes per row) of a warp's 32 consecutive
// rows to the further output buffers, coalesced: every lane parks its row's 64
// bytes in the warp's shared-memory slot and the warp reads them back so that
// four lanes cover one row -- a store instruction then writes eight whole
// 64-byte pieces instead of thirty-two scattered 16-byte ones, which is what
// NVLink (and the multicast path through the switch) needs to run at speed.
// `first_row_offset`: byte offset of (the warp's first row, the chunk's first
// column) inside O; rows >= rows_live and bytes >= bytes_live do not exist.
__device__ __forceinline__ void store_extra_chunk_16bit(const FaExtra &ex, uint8_t *slot, int lane,
                                                        const uint32_t (&w)[16], size_t first_row_offset,
                                                        size_t row_bytes, int rows_live, int bytes_live) {
  uint4 *mine = reinterpret_cast<uint4 *>(slot) + lane * 4;
#pragma unroll
  for (int v = 0; v < 4; ++v)
    mine[v] = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
  __syncwarp();
  const int piece = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = (lane >> 2) + 8 * i;
    if (r < rows_live && piece * 16 < bytes_live)
      store_extra_16B(ex, first_row_offset + static_cast<size_t>(r) * row_bytes + piece * 16,
                      reinterpret_cast<const uint4 *>(slot)[r * 4 + piece]);
  }
  __syncwarp();
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool bf16) {
  if (bf16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

} // namespace fa_detail
} // namespace wave
