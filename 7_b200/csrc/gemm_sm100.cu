// Tiled f16/bf16 GEMM for sm_100a: D[M x N] = A[M x K] * B[N x K]^T with f32
// accumulation in tensor memory.  This is the B200 stand-in for the kernel the
// reference generates as `wmma_f16_matmul_tiled`
// (python/mlir/dialects/wave_matmul.py:11163-11241) and, in its Stream-K mode,
// for `gfx950_f16_streamk_gemm` (wave_matmul.py:9987-10150, 11521-11578).
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: A and B tiles -> 128B-swizzled shared memory
//   warp 1      UMMA issuer (one thread): tcgen05.mma 128 x BN x 16, K-major
//               operands straight from shared memory, accumulator in TMEM
//   warps 2..5  epilogue: tcgen05.ld -> round to the C type -> global stores
// Shared-memory stages are handed over with full/empty mbarriers; the TMEM
// accumulator is double buffered so the epilogue of tile i overlaps the main
// loop of tile i+1.  No load uses cluster multicast.
//
// Numerics (they decide parity with the reference's CPU check,
// tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp:1586-1595):
// operands are used as given (already f16/bf16), products are exact, the
// accumulator is f32, and there is a single round-to-nearest-even to the C
// element type at the end.  No alpha/beta: C is overwritten.
#include "gemm_common.cuh"
#include "launch_cache.h"

namespace wave {

__device__ int g_gemm_status[4]; // [0] code, [1] block, [2] role, [3] detail

namespace {

using namespace gemm_detail;

constexpr int kBM = 128;      // UMMA M (rows of the accumulator = TMEM lanes)
constexpr int kBK = 64;       // 64 16-bit elements = one 128-byte swizzle row
constexpr int kUmmaK = 16;    // K per tcgen05.mma for 16-bit operands
constexpr int kThreads = 192; // 6 warps
constexpr int kEpiThreads = 128;
constexpr int kStoreCols = 64;                         // 16-bit output columns per TMA store: one 128-byte swizzle row
constexpr int kStoreTileBytes = kBM * kStoreCols * 2; // 16 KB

template <int BN> struct TileCfg {
  static constexpr int kStages = BN >= 256 ? 4 : BN >= 128 ? 6 : BN >= 64 ? 8 : 10;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kAccCols = BN < 32 ? 32 : BN; // TMEM columns per accumulator buffer
  static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
  // Two 128-row x 128-byte staging tiles of the TMA-store epilogue (tiles of at least 64 columns).
  static constexpr int kStoreBytes = BN >= 64 ? 2 * kStoreTileBytes : 0;
  // slack for 1024-byte alignment + stage ring + 1 KB of barriers and bookkeeping + staging tiles
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + 1024 + kStoreBytes;
};

struct Shared {
  uint64_t full[10];
  uint64_t empty[10];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int last_arriver; // Stream-K: broadcast of the arrival-counter result
};

__device__ __forceinline__ void report(int code, int role, int detail) {
  if (atomicCAS(&g_gemm_status[0], 0, code) == 0) {
    g_gemm_status[1] = static_cast<int>(blockIdx.x);
    g_gemm_status[2] = role;
    g_gemm_status[3] = detail;
  }
}

struct Segment {
  int tile, k_begin, k_end; // k in units of kBK iterations
};

// Work iterator shared by the three roles so that they agree on the sequence
// of (tile, k range) segments without talking to each other.
struct WorkIter {
  const GemmParams &p;
  long long dp_cur;   // next whole tile of the data-parallel part (strided by the grid)
  long long cur, end; // Stream-K part: this worker's interval of (tile, k) iterations
  __device__ WorkIter(const GemmParams &params) : p(params) {
    // Tiles [0, dp_tiles) are whole tiles dealt round-robin; tiles
    // [dp_tiles, num_tiles) are split Stream-K style over all workers.  Pure
    // data-parallel launches have dp_tiles == num_tiles, pure Stream-K 0.
    dp_cur = blockIdx.x;
    cur = end = 0;
    if (p.streamk_workers > 0)
      streamk_interval(static_cast<long long>(p.num_tiles - p.dp_tiles) * p.k_iters, p.streamk_workers, blockIdx.x,
                       cur, end);
  }
  __device__ bool next(Segment &s) {
    if (dp_cur < p.dp_tiles) {
      s.tile = static_cast<int>(dp_cur);
      s.k_begin = 0;
      s.k_end = p.k_iters;
      dp_cur += gridDim.x;
      return true;
    }
    if (cur >= end)
      return false;
    const long long tile = cur / p.k_iters; // index within the Stream-K part
    const long long tile_begin = tile * p.k_iters;
    const long long seg_end = min(end, tile_begin + p.k_iters);
    s.tile = static_cast<int>(tile) + p.dp_tiles;
    s.k_begin = static_cast<int>(cur - tile_begin);
    s.k_end = static_cast<int>(seg_end - tile_begin);
    cur = seg_end;
    return true;
  }
};

template <int BN, int OUT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
  using Cfg = TileCfg<BN>;
  using T = typename OutT<OUT>::type;
  constexpr int kStages = Cfg::kStages;
  constexpr int CW = BN >= 32 ? 32 : 16; // columns per TMEM load

  extern __shared__ uint8_t smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Shared *sh = reinterpret_cast<Shared *>(tiles + kStages * Cfg::kStageBytes);
  volatile int *abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tfull[a], 1);
      mbar_init(&sh->tempty[a], 4);
    }
    sh->abort_flag = 0;
    sh->last_arriver = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
  // Programmatic dependent launch: the set-up above touched only this CTA's own
  // state and may run while the kernel before this one on the stream is still
  // finishing; global memory (operands, C, Stream-K scratch and counters) waits
  // for that kernel to be complete.  No-ops for a launch without the attribute.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      WorkIter work(p);
      Segment seg;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && work.next(seg)) {
        int mb, nb;
        tile_coords(seg.tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
#ifdef WAVE_WAIT_TEST
        const int k_stop = seg.k_end - (p.test_skip_last_k ? 1 : 0);
#else
        const int k_stop = seg.k_end;
#endif
        for (int kb = seg.k_begin; kb < k_stop; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) {
            report(kStatusWaitTimeout, 0, stage);
            ok = false;
            break;
          }
          uint8_t *a_dst = tiles + stage * Cfg::kStageBytes;
          uint8_t *b_dst = a_dst + Cfg::kABytes;
          mbar_arrive_expect_tx(&sh->full[stage], Cfg::kStageBytes);
          tma_load_2d(a_dst, &tmap_a, &sh->full[stage], kb * kBK, mb * kBM);
          tma_load_2d(b_dst, &tmap_b, &sh->full[stage], kb * kBK, nb * BN);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok)
        bounded_delay(1 << 21); // let copies in flight land before teardown
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- UMMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_f16 = umma_idesc_f16(kBM, BN, 0);
      constexpr uint32_t idesc_bf16 = umma_idesc_f16(kBM, BN, 1);
      const uint32_t idesc = p.in_type == WAVE_GEMM_IN_BF16 ? idesc_bf16 : idesc_f16;
      WorkIter work(p);
      Segment seg;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      while (ok && work.next(seg)) {
        if (!mbar_wait(&sh->tempty[acc], acc_phase ^ 1, abort_flag)) {
          report(kStatusWaitTimeout, 1, 100 + acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * Cfg::kAccCols);
        for (int kb = seg.k_begin; kb < seg.k_end; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            report(kStatusWaitTimeout, 1, stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + stage * Cfg::kStageBytes);
          const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
          const uint64_t b_desc = umma_desc_kmajor_sw128(a_addr + Cfg::kABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // +32 bytes per K step inside the 128-byte swizzle row (>>4 = 2)
            umma_ss(tmem_d, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 2), idesc,
                    (kb > seg.k_begin || k > 0) ? 1u : 0u);
          }
          umma_commit(&sh->empty[stage]); // frees the stage once the MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok)
          break;
        umma_commit(&sh->tfull[acc]); // accumulator complete
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int row_in_tile = quarter * 32 + lane;
    const int epi_tid = row_in_tile;       // 0..127, unique per epilogue thread
    WorkIter work(p);
    Segment seg;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t store_n = 0; // TMA stores issued so far (staging tile = parity)
    uint8_t *store_tiles = tiles + kStages * Cfg::kStageBytes + 1024;
    const long long total_iters = static_cast<long long>(p.num_tiles - p.dp_tiles) * p.k_iters; // Stream-K part
    while (work.next(seg)) {
      int mb, nb;
      tile_coords(seg.tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
      bool failed = !mbar_wait(&sh->tfull[acc], acc_phase, abort_flag);
      {
        // The four warps meet at named barriers below: they must leave together.
        uint32_t any;
        __syncwarp();
        asm volatile("{\n\t.reg .pred pin, pout;\n\tsetp.ne.b32 pin, %1, 0;\n\t"
                     "bar.red.or.pred pout, 1, %2, pin;\n\tselp.b32 %0, 1, 0, pout;\n\t}"
                     : "=r"(any)
                     : "r"(failed ? 1u : 0u), "n"(kEpiThreads)
                     : "memory");
        failed = any != 0;
      }
      if (failed) {
        if (lane == 0)
          report(kStatusWaitTimeout, 2, 200 + acc);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(acc * Cfg::kAccCols);
      const int m = mb * kBM + row_in_tile;
      const bool whole = seg.k_begin == 0 && seg.k_end == p.k_iters;
      if constexpr (sizeof(T) == 2 && BN >= 64) {
        if (whole && p.c_tma) {
          // Row-major 16-bit output: 64 columns of the tile's 128 rows at a time go
          // through a swizzled shared-memory tile and out with one TMA store
          // (whole 128-byte rows instead of 16 bytes per thread; clipped at the
          // matrix edge).  Two tiles: a store reads one while the other is filled.
#pragma unroll 1
          for (int c = 0; c < BN; c += kStoreCols, ++store_n) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(taddr + c, r0);
            tmem_ld_32x32b_x32(taddr + c + 32, r1);
            tmem_ld_wait();
            if (c + kStoreCols >= BN) { // the accumulator has been read: the next tile may use it
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0)
                mbar_arrive(&sh->tempty[acc]);
            }
            uint8_t *buf = store_tiles + (store_n & 1u) * kStoreTileBytes;
            if (epi_tid == 0)
              tma_store_wait_read<1>(); // the store that last used this tile has read it
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
            uint8_t *row_ptr = buf + row_in_tile * (kStoreCols * 2);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t *src = k < 4 ? &r0[8 * k] : &r1[8 * (k - 4)];
              T tmp[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                store_elem(&tmp[e], __uint_as_float(src[e]));
              // 128-byte swizzle: 16-byte chunk k of row r sits at chunk k ^ (r & 7)
              *reinterpret_cast<uint4 *>(row_ptr + ((k ^ (row_in_tile & 7)) << 4)) = *reinterpret_cast<uint4 *>(tmp);
            }
            fence_proxy_async_smem();
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
            if (epi_tid == 0) {
              tma_store_2d_evict_first(&tmap_c, buf, nb * BN + c, mb * kBM);
              tma_store_commit();
            }
          }
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1;
          }
          continue;
        }
      }
      if (whole) {
#pragma unroll 1
        for (int c = 0; c < BN; c += CW) {
          uint32_t r[CW];
          if constexpr (CW == 32)
            tmem_ld_32x32b_x32(taddr + c, r);
          else
            tmem_ld_32x32b_x16(taddr + c, r);
          tmem_ld_wait();
          float v[CW];
#pragma unroll
          for (int j = 0; j < CW; ++j)
            v[j] = __uint_as_float(r[j]);
          store_row_chunk<T, CW>(p, m, nb * BN + c, v);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&sh->tempty[acc]);
      } else {
        // Stream-K partial: raw f32 accumulator -> this worker's scratch slot,
        // element (row, col) at col*128 + row so a warp writes 128 contiguous
        // bytes.  Then count the arrival; the last arriver reduces.
        const int sk_tile = seg.tile - p.dp_tiles; // index within the Stream-K part
        const int slot = streamk_slot(total_iters, p.streamk_workers, p.k_iters, blockIdx.x, sk_tile);
        float *mine = p.scratch + (static_cast<size_t>(blockIdx.x) * 2 + slot) * (kBM * BN);
#pragma unroll 1
        for (int c = 0; c < BN; c += CW) {
          uint32_t r[CW];
          if constexpr (CW == 32)
            tmem_ld_32x32b_x32(taddr + c, r);
          else
            tmem_ld_32x32b_x16(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CW; ++j)
            mine[(c + j) * kBM + row_in_tile] = __uint_as_float(r[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&sh->tempty[acc]); // TMEM buffer is free; the rest is global memory only
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        const long long tile_begin = static_cast<long long>(sk_tile) * p.k_iters;
        const int first_owner = streamk_owner(total_iters, p.streamk_workers, tile_begin);
        const int last_owner = streamk_owner(total_iters, p.streamk_workers, tile_begin + p.k_iters - 1);
        const int parts = last_owner - first_owner + 1;
        if (epi_tid == 0) {
          const int old = atomicAdd(&p.counters[sk_tile], 1);
          sh->last_arriver = (old + 1 == parts) ? 1 : 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        const bool last = sh->last_arriver != 0;
        if (last) {
          __threadfence();
          // Fixed order: ascending owner id, starting from zero
          // (wave_matmul.py:9756-9784), so the result is run-to-run identical.
#pragma unroll 1
          for (int c = 0; c < BN; c += CW) {
            float v[CW];
#pragma unroll
            for (int j = 0; j < CW; ++j)
              v[j] = 0.0f;
            for (int owner = first_owner; owner <= last_owner; ++owner) {
              const int oslot = streamk_slot(total_iters, p.streamk_workers, p.k_iters, owner, sk_tile);
              const float *src = p.scratch + (static_cast<size_t>(owner) * 2 + oslot) * (kBM * BN);
#pragma unroll
              for (int j = 0; j < CW; ++j)
                v[j] += __ldcg(&src[(c + j) * kBM + row_in_tile]);
            }
            store_row_chunk<T, CW>(p, m, nb * BN + c, v);
          }
          if (epi_tid == 0)
            atomicAdd(&p.counters[sk_tile], -parts); // back to zero for the next launch
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory"); // sh->last_arriver may be rewritten
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (epi_tid == 0)
      tma_store_wait_read<0>(); // the staging tiles must outlive the stores that read them
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

template <int BN, int OUT>
cudaError_t launch_one(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const GemmParams &p,
                       int grid, cudaStream_t stream) {
  using Cfg = TileCfg<BN>;
  // The shared-memory opt-in belongs to the current device's context: once per (kernel, device).
  cudaError_t err = prepare_kernel(gemm_kernel<BN, OUT>, Cfg::kSmemBytes, nullptr);
  if (err != cudaSuccess)
    return err;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = p.pdl ? 1 : 0; // the stream may begin this launch, up to its griddepcontrol.wait, early
  return cudaLaunchKernelEx(&cfg, gemm_kernel<BN, OUT>, ta, tb, tc, p);
}

template <int BN>
cudaError_t launch_bn(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tc, const GemmParams &p,
                      int grid, cudaStream_t stream) {
  switch (p.out_type) {
  case WAVE_GEMM_OUT_F32:
    return launch_one<BN, WAVE_GEMM_OUT_F32>(ta, tb, tc, p, grid, stream);
  case WAVE_GEMM_OUT_F16:
    return launch_one<BN, WAVE_GEMM_OUT_F16>(ta, tb, tc, p, grid, stream);
  case WAVE_GEMM_OUT_BF16:
    return launch_one<BN, WAVE_GEMM_OUT_BF16>(ta, tb, tc, p, grid, stream);
  }
  return cudaErrorInvalidValue;
}

} // namespace

int gemm_tile_m() { return kBM; }
int gemm_tile_k() { return kBK; }

// `tmap_c` is read only when p.c_tma is set (tile_n >= 64): a box of 64 columns
// x 128 rows over the row-major 16-bit output.
cudaError_t launch_gemm(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, const CUtensorMap &tmap_c,
                        const GemmParams &p, int tile_n, int grid, cudaStream_t stream) {
  switch (tile_n) {
  case 16:
    return launch_bn<16>(tmap_a, tmap_b, tmap_c, p, grid, stream);
  case 32:
    return launch_bn<32>(tmap_a, tmap_b, tmap_c, p, grid, stream);
  case 64:
    return launch_bn<64>(tmap_a, tmap_b, tmap_c, p, grid, stream);
  case 128:
    return launch_bn<128>(tmap_a, tmap_b, tmap_c, p, grid, stream);
  case 256:
    return launch_bn<256>(tmap_a, tmap_b, tmap_c, p, grid, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t gemm_read_status(int out[4], bool clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_gemm_status, sizeof(int) * 4);
  if (err == cudaSuccess && clear) {
    int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(g_gemm_status, zero, sizeof(zero));
  }
  return err;
}

} // namespace wave
