// CTA-pair variant of the tiled f16/bf16 GEMM for large problems: two CTAs of a
// 2-CTA cluster compute one 256 x 256 output tile with tcgen05.mma
// cta_group::2 (UMMA 256 x 256 x 16).  Each CTA loads its own 128 rows of A and
// its own 128 of the tile's 256 B rows (no multicast: every load targets the
// loading CTA's shared memory) and receives its 128 accumulator rows in its
// own TMEM; the even CTA issues the MMAs, which read both CTAs' shared memory.
// Per CTA a K step moves 32 KB instead of the one-CTA kernel's 48 KB for the
// same 128 x 256 outputs, which both deepens the ring (6 stages) and cuts
// shared-memory and L2 traffic per flop.
//
// Same numerics and operator surface as gemm_sm100.cu (the reference's
// `wmma_f16_matmul_tiled`, python/mlir/dialects/wave_matmul.py:11163-11241).
//
// Synchronisation across the pair:
//   full[s]    lives in the leader; the leader's producer arms it with the
//              bytes of BOTH CTAs' loads, the peer's TMA completes on it too
//   empty[s]   one per CTA; the leader's tcgen05.commit arrives on both
//   tfull[a]   one per CTA; the leader's commit arrives on both
//   tempty[a]  lives in the leader; the epilogue warps of both CTAs arrive
#include "gemm_common.cuh"

namespace wave {

__device__ int g_gemm_pair_status[4];

namespace {

using namespace gemm_detail;

constexpr int kRows = 128;     // rows of A / of the accumulator per CTA
constexpr int kPairM = 256;    // UMMA M across the pair
constexpr int kPairN = 256;    // UMMA N
constexpr int kBRows = 128;    // B rows held by one CTA
constexpr int kBK = 64;
#ifndef WAVE_PAIR_STAGES
#define WAVE_PAIR_STAGES 6
#endif
constexpr int kStages = WAVE_PAIR_STAGES;
constexpr int kABytes = kRows * kBK * 2;
constexpr int kBBytes = kBRows * kBK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 192;
constexpr int kTmemCols = 512; // two 256-column accumulators
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;

struct PairShared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void pair_report(int code, int role, int detail) {
  if (atomicCAS(&g_gemm_pair_status[0], 0, code) == 0) {
    g_gemm_pair_status[1] = static_cast<int>(blockIdx.x);
    g_gemm_pair_status[2] = role;
    g_gemm_pair_status[3] = detail;
  }
}

template <int OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  using T = typename OutT<OUT>::type;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  PairShared *sh = reinterpret_cast<PairShared *>(tiles + kStages * kStageBytes);
  volatile int *abort_flag = &sh->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&sh->tfull[a], 1);
      mbar_init(&sh->tempty[a], 8); // four epilogue warps in each CTA of the pair
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&sh->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive(); // the peer's barriers must be initialised before anything signals them
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs) {
        int mb, nb;
        tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
        const int m0 = mb * kPairM + static_cast<int>(rank) * kRows;
        const int n0 = nb * kPairN + static_cast<int>(rank) * kBRows;
        for (int kb = 0; kb < p.k_iters; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) {
            pair_report(kStatusWaitTimeout, 0, stage);
            ok = false;
            break;
          }
          uint8_t *a_dst = tiles + stage * kStageBytes;
          uint8_t *b_dst = a_dst + kABytes;
          if (leader)
            mbar_arrive_expect_tx(&sh->full[stage], 2 * kStageBytes);
          tma_load_2d_pair(a_dst, &tmap_a, &sh->full[stage], kb * kBK, m0);
          tma_load_2d_pair(b_dst, &tmap_b, &sh->full[stage], kb * kBK, n0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok)
        bounded_delay(1 << 21);
    }
  } else if (warp == 1) {
    // ------------------------------------------- UMMA issuer (leader only)
    if (lane == 0 && leader) {
      const uint32_t idesc = umma_idesc_f16(kPairM, kPairN, p.in_type == WAVE_GEMM_IN_BF16 ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < p.num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(&sh->tempty[acc], acc_phase ^ 1, abort_flag)) {
          pair_report(kStatusWaitTimeout, 1, 100 + acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kPairN);
        for (int kb = 0; kb < p.k_iters; ++kb) {
          if (!mbar_wait(&sh->full[stage], phase, abort_flag)) {
            pair_report(kStatusWaitTimeout, 1, stage);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(tiles + stage * kStageBytes);
          const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
          const uint64_t b_desc = umma_desc_kmajor_sw128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_ss_pair(tmem_d, a_desc + static_cast<uint64_t>(k * 2), b_desc + static_cast<uint64_t>(k * 2), idesc,
                         (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&sh->empty[stage], 3); // frees the stage in both CTAs
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok)
          break;
        umma_commit_pair(&sh->tfull[acc], 3);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t tempty_leader[2] = {map_to_cta(&sh->tempty[0], 0), map_to_cta(&sh->tempty[1], 0)};
    for (int tile = pair_id; tile < p.num_tiles; tile += num_pairs) {
      int mb, nb;
      tile_coords(tile, p.num_m_blocks, p.num_n_blocks, p.group_m, mb, nb);
      if (!mbar_wait(&sh->tfull[acc], acc_phase, abort_flag)) {
        if (lane == 0)
          pair_report(kStatusWaitTimeout, 2, 200 + acc);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * kPairN);
      const int m = mb * kPairM + static_cast<int>(rank) * kRows + row_in_tile;
#pragma unroll 1
      for (int c = 0; c < kPairN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          v[j] = __uint_as_float(r[j]);
        store_row_chunk<T, 32>(p, m, nb * kPairN + c, v);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive_cluster(tempty_leader[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // Neither CTA may leave (or free TMEM) while its partner can still read its
  // shared memory, signal its barriers or write its TMEM.
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int OUT>
cudaError_t launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const GemmParams &p, int grid,
                        cudaStream_t stream) {
  cudaError_t err =
      cudaFuncSetAttribute(gemm_pair_kernel<OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (err != cudaSuccess)
    return err;
  gemm_pair_kernel<OUT><<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

} // namespace

int gemm_pair_tile_m() { return kPairM; }
int gemm_pair_tile_n() { return kPairN; }
int gemm_pair_box_rows() { return kRows; }

// `grid` must be even: consecutive CTAs form the pairs.
cudaError_t launch_gemm_pair(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, const GemmParams &p, int grid,
                             cudaStream_t stream) {
  switch (p.out_type) {
  case WAVE_GEMM_OUT_F32:
    return launch_pair<WAVE_GEMM_OUT_F32>(tmap_a, tmap_b, p, grid, stream);
  case WAVE_GEMM_OUT_F16:
    return launch_pair<WAVE_GEMM_OUT_F16>(tmap_a, tmap_b, p, grid, stream);
  case WAVE_GEMM_OUT_BF16:
    return launch_pair<WAVE_GEMM_OUT_BF16>(tmap_a, tmap_b, p, grid, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t gemm_pair_read_status(int out[4], bool clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_gemm_pair_status, sizeof(int) * 4);
  if (err == cudaSuccess && clear) {
    int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(g_gemm_pair_status, zero, sizeof(zero));
  }
  return err;
}

} // namespace wave
