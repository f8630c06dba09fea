// Pieces shared by the one-CTA and the CTA-pair GEMM kernels: tile
// rasterisation and the register -> global-memory epilogue stores.
#pragma once
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace wave {
namespace gemm_detail {

// Linear tile id -> (m block, n block) with grouped-M rasterisation, the
// portable half of the reference's CTA remap (wave_matmul.py:1248-1276):
// consecutive ids walk down `group_m` row blocks before moving one column
// block over, so CTAs running at the same time share A and B panels in L2.
__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int group_m, int &mb, int &nb) {
  const int per_group = group_m * num_n;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int rows = min(num_m - first_m, group_m);
  const int in_group = tile - group * per_group;
  mb = first_m + in_group % rows;
  nb = in_group / rows;
}

// Balanced contiguous split of `total` iterations over `workers`
// (wave_matmul.py:88-100, streamk_worker_interval).
__device__ __forceinline__ void streamk_interval(long long total, int workers, int worker, long long &begin,
                                                 long long &end) {
  const long long q = total / workers, r = total % workers;
  begin = worker * q + min(static_cast<long long>(worker), r);
  end = begin + q + (worker < r ? 1 : 0);
}
// Owner of one iteration (wave_matmul.py:103-116, streamk_owner_for_iteration).
__device__ __forceinline__ int streamk_owner(long long total, int workers, long long it) {
  const long long q = total / workers, r = total % workers;
  const long long large_end = r * (q + 1);
  if (it < large_end)
    return static_cast<int>(it / (q + 1));
  return static_cast<int>(r + (it - large_end) / q);
}
// Scratch slot (0 or 1) that `owner` uses for its partial of `tile`
// (wave_matmul.py:135-159, streamk_worker_segments): partial tiles are
// numbered in tile order and a contiguous interval has at most two.
__device__ __forceinline__ int streamk_slot(long long total, int workers, int k_iters, int owner, int tile) {
  long long b, e;
  streamk_interval(total, workers, owner, b, e);
  const long long first_tile = b / k_iters;
  if (tile == first_tile)
    return 0;
  const bool first_partial = (b % k_iters != 0) || (e < (first_tile + 1) * static_cast<long long>(k_iters));
  return first_partial ? 1 : 0;
}

template <int OUT> struct OutT;
template <> struct OutT<WAVE_GEMM_OUT_F32> { using type = float; };
template <> struct OutT<WAVE_GEMM_OUT_F16> { using type = __half; };
template <> struct OutT<WAVE_GEMM_OUT_BF16> { using type = __nv_bfloat16; };

__device__ __forceinline__ void store_elem(float *p, float v) { *p = v; }
__device__ __forceinline__ void store_elem(__half *p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void store_elem(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// Stores `W` consecutive-n values of row m.  When n is the contiguous
// direction the values go out as 16-byte vectors; otherwise (m contiguous)
// each value is a scalar store that coalesces across the warp's 32 rows.
template <typename T, int W>
__device__ __forceinline__ void store_row_chunk(const GemmParams &p, int m, int n0, const float (&v)[W]) {
  if (m >= p.M)
    return;
  if (p.tile_packed) {
    // Tile-packed output: 16 x 16 tiles stored one after another, row-major
    // inside a tile, in the reference's workgroup -> wave -> per-wave-tile
    // order (python/mlir/dialects/wave_matmul.py:1025-1041, 1106-1139).
    constexpr int per_vec = 16 / sizeof(T);
    const int m_tile = m >> 4;
    const int tm = p.tp_bm * p.tp_wmt, tn = p.tp_bn * p.tp_wnt;
    const int wg_m = m_tile / tm, rm = m_tile % tm;
    const int m_wave = rm / p.tp_wmt, ti = rm % p.tp_wmt;
#pragma unroll
    for (int g = 0; g < W; g += 16) {
      const int n = n0 + g;
      if (n >= p.N)
        break;
      const int n_tile = n >> 4;
      const int wg_n = n_tile / tn, rn = n_tile % tn;
      const int n_wave = rn / p.tp_wnt, tj = rn % p.tp_wnt;
      const long long tile =
          (((static_cast<long long>(wg_m) * p.tp_n_blocks + wg_n) * (p.tp_bm * p.tp_bn) + (m_wave * p.tp_bn + n_wave)) *
               p.tp_wmt +
           ti) *
              p.tp_wnt +
          tj;
      if (p.tp_fragment) {
        // AMD accumulator-fragment order inside the tile (the reference runner's
        // getOutputCoordinate, wave-matmul-calibrate-runner.cpp:809-836): the
        // 16 values of a row go to 16 lanes' slots, values_per_lane apart.
        const int r = m & 15;
        const int vpl = p.tp_fragment == 1 ? 4 : 8;
        const int lane_row = p.tp_fragment == 2 ? (r & 1) : r / vpl; // lane / 16
        const int v_idx = p.tp_fragment == 2 ? (r >> 1) : r % vpl;
        T *frag = reinterpret_cast<T *>(p.C) + tile * 256 + lane_row * 16 * vpl + v_idx;
#pragma unroll
        for (int j = 0; j < 16; ++j)
          store_elem(frag + j * vpl, v[g + j]);
        continue;
      }
      T *dst = reinterpret_cast<T *>(p.C) + tile * 256 + (m & 15) * 16;
#pragma unroll
      for (int j = 0; j < 16; j += per_vec) {
        if constexpr (sizeof(T) == 4) {
          *reinterpret_cast<float4 *>(dst + j) = make_float4(v[g + j], v[g + j + 1], v[g + j + 2], v[g + j + 3]);
        } else {
          T tmp[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            store_elem(&tmp[e], v[g + j + e]);
          *reinterpret_cast<uint4 *>(dst + j) = *reinterpret_cast<uint4 *>(tmp);
        }
      }
    }
    return;
  }
  T *base = reinterpret_cast<T *>(p.C) + static_cast<long long>(m) * p.stride_m +
            static_cast<long long>(n0) * p.stride_n;
  if (p.stride_n == 1) {
    constexpr int per_vec = 16 / sizeof(T);
#pragma unroll
    for (int j = 0; j < W; j += per_vec) {
      if (n0 + j < p.N) { // N is a multiple of 16, so a started vector is whole
        if constexpr (sizeof(T) == 4) {
          float4 q = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
          *reinterpret_cast<float4 *>(base + j) = q;
        } else {
          T tmp[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            store_elem(&tmp[e], v[j + e]);
          *reinterpret_cast<uint4 *>(base + j) = *reinterpret_cast<uint4 *>(tmp);
        }
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j)
      if (n0 + j < p.N)
        store_elem(base + static_cast<long long>(j) * p.stride_n, v[j]);
  }
}

} // namespace gemm_detail
} // namespace wave
