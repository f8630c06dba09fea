// CTA-pair variant of the tiled f16/bf16 GEMM for large problems: two CTAs of a
// 2-CTA cluster compute one 256 x PN output tile (PN = 256 or 128) with
// tcgen05.mma cta_group::2 (UMMA 256 x PN x 16).  Each CTA loads its own 128
// rows of A and its own half of the tile's PN B rows (no multicast: every load
// targets the loading CTA's shared memory) and receives its 128 accumulator
// rows in its own TMEM; the even CTA issues the MMAs, which read both CTAs'
// shared memory.  With PN = 256 a K step moves 32 KB per CTA instead of the
// one-CTA kernel's 48 KB for the same 128 x 256 outputs, which both deepens the
// ring (6 stages) and cuts shared-memory and L2 traffic per flop.  PN = 128
// (24 KB per step, 8 stages) halves the tile; its 256 x 128 x 16 MMAs reach
// only 0.69 of the wide tile's rate (1035 against 1507 TFLOP/s at 8192^3), so
// the host never picks it by itself.
//
// Stream-K tail (p.streamk_workers = number of CTA pairs): tiles [0, dp_tiles)
// are whole tiles dealt round-robin over the pairs; the K iterations of tiles
// [dp_tiles, num_tiles) -- a last round that would leave pairs idle -- are split
// evenly over all pairs with the reference's partition
// (wave_matmul.py:88-159).  Each CTA of a pair treats its 128 rows on its own:
// f32 partial -> its half of the pair's scratch slot, one arrival counter per
// (tile, CTA rank), the last arriver sums the owners in ascending order and
// stores C, counters return to zero (wave_matmul.py:9756-9784, 9987-10150).
// Nothing waits for another CTA pair.
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
#include "launch_cache.h"

namespace wave {

__device__ int g_gemm_pair_status[4];

namespace {

using namespace gemm_detail;

constexpr int kRows = 128;     // rows of A / of the accumulator per CTA
constexpr int kPairM = 256;    // UMMA M across the pair
constexpr int kBK = 64;
constexpr int kABytes = kRows * kBK * 2;
constexpr int kThreads = 192;
constexpr int kMaxStages = 8;
constexpr int kStoreCols = 64;                      // 16-bit output columns per TMA store: 128 bytes, one swizzle row
constexpr int kStoreTileBytes = kRows * kStoreCols * 2; // 16 KB

// Per tile width PN: B rows held by one CTA, ring depth (192 KB of stages) and
// TMEM columns (two PN-column accumulators).
template <int PN> struct PairCfg {
  static constexpr int kBRows = PN / 2;
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = PN == 256 ? 6 : 8;
  static constexpr int kTmemCols = 2 * PN;
  // stage ring | 1 KB of barriers | two 128-row x 128-byte staging tiles of the TMA-store epilogue
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 1024 + 2 * kStoreTileBytes;
};

struct PairShared {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint32_t tmem_base;
  int abort_flag;
  int last_arriver; // Stream-K: broadcast of the arrival-counter result among the epilogue warps
};

// One unit of work of a CTA pair: a whole tile, half a tile (columns
// [n_off, n_off + width) of it) or a K range of a Stream-K tile.
struct PairItem {
  int tile, mb, nb, n_off, width, k_begin, k_end;
};

// Work iterator shared by the three roles of both CTAs, so that they agree on
// the sequence of items without talking to each other.  Data-parallel part:
// items [0, dp_items) strided by the number of pairs (tiles below split_from
// whole, later ones as two half-width items); Stream-K part: this pair's
// interval of (tile, k) iterations of the tiles from dp_tiles on.
template <int PN> struct PairWork {
  const GemmParams &p;
  int split_from, dp_items, num_pairs;
  int tile_w; // columns of a whole tile: PN, or with PN = 256 any multiple of 32 the host chose (p.pair_tile_n)
  long long dp_cur, cur, end;
  __device__ PairWork(const GemmParams &params, int pair_id, int pairs) : p(params), num_pairs(pairs) {
    const bool sk = p.streamk_workers > 0;
    tile_w = PN == 256 ? p.pair_tile_n : PN;
    split_from = (PN == 256 && !sk && tile_w == 256) ? p.split_from : p.num_tiles;
    dp_items = sk ? p.dp_tiles : split_from + 2 * (p.num_tiles - split_from);
    dp_cur = pair_id;
    cur = end = 0;
    if (sk)
      streamk_interval(static_cast<long long>(p.num_tiles - p.dp_tiles) * p.k_iters, p.streamk_workers, pair_id, cur,
                       end);
  }
  __device__ bool next(PairItem &it) {
    if (dp_cur < dp_items) {
      const int item = static_cast<int>(dp_cur);
      dp_cur += num_pairs;
      it.tile = item;
      it.n_off = 0;
      it.width = tile_w;
      if (item >= split_from) {
        const int r = item - split_from;
        it.tile = split_from + (r >> 1);
        it.n_off = (r & 1) * (tile_w / 2);
        it.width = tile_w / 2;
      }
      it.k_begin = 0;
      it.k_end = p.k_iters;
    } else {
      if (cur >= end)
        return false;
      const long long tile = cur / p.k_iters; // index within the Stream-K part
      const long long tile_begin = tile * p.k_iters;
      const long long seg_end = min(end, tile_begin + p.k_iters);
      it.tile = static_cast<int>(tile) + p.dp_tiles;
      it.n_off = 0;
      it.width = tile_w;
      it.k_begin = static_cast<int>(cur - tile_begin);
      it.k_end = static_cast<int>(seg_end - tile_begin);
      cur = seg_end;
    }
    tile_coords(it.tile, p.num_m_blocks, p.num_n_blocks, p.group_m, it.mb, it.nb);
    return true;
  }
};

__device__ __forceinline__ void pair_report(int code, int role, int detail) {
  if (atomicCAS(&g_gemm_pair_status[0], 0, code) == 0) {
    g_gemm_pair_status[1] = static_cast<int>(blockIdx.x);
    g_gemm_pair_status[2] = role;
    g_gemm_pair_status[3] = detail;
  }
}

// Tensor maps over the further copies of C of a launch (same shape, strides
// and box as the map of C itself): a kernel parameter of the variant that
// sends every finished piece to them with TMA stores, and of that variant only.
struct PairExtraMaps {
  CUtensorMap m[7];
};

// The kernel's body.  kTmaExtra: the further copies of C (p.n_extra of them,
// plain addresses) get each 128 x 64 piece by a TMA store from the same staging
// tile as C itself (`em`); otherwise they are written with stores from the
// epilogue warps (the only way to a multicast address).
template <int OUT, int PN, bool kTmaExtra>
__device__ __forceinline__ void gemm_pair_body(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b,
                                               const CUtensorMap &tmap_b_half, const CUtensorMap &tmap_c,
                                               const GemmParams &p, const PairExtraMaps *em) {
  using T = typename OutT<OUT>::type;
  using Cfg = PairCfg<PN>;
  constexpr int kPairN = PN;
  constexpr int kStageBytes = Cfg::kStageBytes;
  constexpr int kStages = Cfg::kStages;
  constexpr int kTmemCols = Cfg::kTmemCols;
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
    sh->last_arriver = 0;
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
  // Programmatic dependent launch: everything above touched only this CTA's own
  // state, so it may run while the kernel before this one on the stream is still
  // finishing; from here on global memory is read and written, which has to wait
  // for that kernel to be complete.  The next kernel on the stream may be set up
  // as soon as SMs come free.  (Both are no-ops for a launch without the attribute.)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      // A panels are shared by every tile of a row group and read again by its
      // later rounds: "evict last".  B panels keep the default policy: marking
      // them "evict first" (hint 1) lets a panel leave L2 before the slower CTAs
      // of the round have read it (8192^3 bf16, one launch: DRAM reads 2046 MB
      // against 1083 MB without hints and 1040 MB with the hint on A alone).
      const uint64_t pol_a = p.l2_hints ? l2_policy_evict_last() : l2_policy_evict_normal();
      const uint64_t pol_b = p.l2_hints == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      PairWork<PN> work(p, pair_id, num_pairs);
      PairItem it;
      while (ok && work.next(it)) {
        const bool half = it.width != work.tile_w;
        const int m0 = it.mb * kPairM + static_cast<int>(rank) * kRows;
        const int n0 = it.nb * work.tile_w + it.n_off + static_cast<int>(rank) * (it.width / 2);
        const uint32_t stage_tx = 2 * (kABytes + (it.width / 2) * kBK * 2);
        for (int kb = it.k_begin; kb < it.k_end; ++kb) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_flag)) {
            pair_report(kStatusWaitTimeout, 0, stage);
            ok = false;
            break;
          }
          uint8_t *a_dst = tiles + stage * kStageBytes;
          uint8_t *b_dst = a_dst + kABytes;
          if (leader)
            mbar_arrive_expect_tx(&sh->full[stage], stage_tx);
          tma_load_2d_pair_hint(a_dst, &tmap_a, &sh->full[stage], kb * kBK, m0, pol_a);
          tma_load_2d_pair_hint(b_dst, half ? &tmap_b_half : &tmap_b, &sh->full[stage], kb * kBK, n0, pol_b);
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
      const int tile_w = PN == 256 ? p.pair_tile_n : PN;
      const uint32_t idesc_whole = umma_idesc_f16(kPairM, tile_w, p.in_type == WAVE_GEMM_IN_BF16 ? 1 : 0);
      const uint32_t idesc_half = umma_idesc_f16(kPairM, tile_w / 2, p.in_type == WAVE_GEMM_IN_BF16 ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      PairWork<PN> work(p, pair_id, num_pairs);
      PairItem it;
      while (ok && work.next(it)) {
        const uint32_t idesc = it.width != tile_w ? idesc_half : idesc_whole;
        if (!mbar_wait(&sh->tempty[acc], acc_phase ^ 1, abort_flag)) {
          pair_report(kStatusWaitTimeout, 1, 100 + acc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * kPairN);
        for (int kb = it.k_begin; kb < it.k_end; ++kb) {
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
                         (kb > it.k_begin || k > 0) ? 1u : 0u);
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
    uint32_t store_n = 0; // TMA stores issued so far (staging tile = parity)
    uint8_t *store_tiles = tiles + kStages * kStageBytes + 1024;
    const uint32_t tempty_leader[2] = {map_to_cta(&sh->tempty[0], 0), map_to_cta(&sh->tempty[1], 0)};
    // Barrier among the four epilogue warps (named barrier 1).
    auto epilogue_barrier = [] { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    const long long total_iters = static_cast<long long>(p.num_tiles - p.dp_tiles) * p.k_iters; // Stream-K part
    PairWork<PN> work(p, pair_id, num_pairs);
    PairItem it;
    while (work.next(it)) {
      const int mb = it.mb, n_off = it.n_off, width = it.width;
      const int n_tile0 = it.nb * work.tile_w; // first column of the tile
      const bool whole = it.k_begin == 0 && it.k_end == p.k_iters;
      bool failed = !mbar_wait(&sh->tfull[acc], acc_phase, abort_flag);
      if (p.c_tma || p.streamk_workers > 0) {
        // The four warps share named barriers below: they must leave together.
        uint32_t any;
        __syncwarp();
        asm volatile("{\n\t.reg .pred pin, pout;\n\tsetp.ne.b32 pin, %1, 0;\n\t"
                     "bar.red.or.pred pout, 1, 128, pin;\n\tselp.b32 %0, 1, 0, pout;\n\t}"
                     : "=r"(any)
                     : "r"(failed ? 1u : 0u)
                     : "memory");
        failed = any != 0;
      }
      if (failed) {
        if (lane == 0)
          pair_report(kStatusWaitTimeout, 2, 200 + acc);
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(acc * kPairN);
      const int m = mb * kPairM + static_cast<int>(rank) * kRows + row_in_tile;
      if (!whole) {
        // Stream-K partial: this CTA's 128 rows of the raw f32 accumulator go to its
        // half of the pair's scratch slot.  Then the arrival is counted; the last
        // arriver of this (tile, CTA rank) reduces.
        const int sk_tile = it.tile - p.dp_tiles;
        const int slot = streamk_slot(total_iters, p.streamk_workers, p.k_iters, pair_id, sk_tile);
        float *mine = p.scratch + ((static_cast<size_t>(pair_id) * 2 + slot) * 2 + rank) * (kRows * PN);
#pragma unroll 1
        for (int c = 0; c < width; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          // groups of four columns: element (row, col) at ((col / 4) * 128 + row) * 4 + col % 4,
          // so a warp's 16-byte stores (and the reducer's loads) cover 512 contiguous bytes
#pragma unroll
          for (int k = 0; k < 8; ++k)
            reinterpret_cast<float4 *>(mine)[((c >> 2) + k) * kRows + row_in_tile] =
                make_float4(__uint_as_float(r[4 * k]), __uint_as_float(r[4 * k + 1]), __uint_as_float(r[4 * k + 2]),
                            __uint_as_float(r[4 * k + 3]));
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive_cluster(tempty_leader[acc]); // TMEM buffer is free; the rest is global memory only
        __threadfence();
        epilogue_barrier();
        const long long tile_begin = static_cast<long long>(sk_tile) * p.k_iters;
        const int first_owner = streamk_owner(total_iters, p.streamk_workers, tile_begin);
        const int last_owner = streamk_owner(total_iters, p.streamk_workers, tile_begin + p.k_iters - 1);
        const int parts = last_owner - first_owner + 1;
        int *counter = &p.counters[sk_tile * 2 + static_cast<int>(rank)];
        if (row_in_tile == 0) {
          const int old = atomicAdd(counter, 1);
          sh->last_arriver = (old + 1 == parts) ? 1 : 0;
        }
        epilogue_barrier();
        if (sh->last_arriver != 0) {
          __threadfence();
          // Fixed order: ascending owner id, starting from zero
          // (wave_matmul.py:9756-9784), so the result is run-to-run identical.
#pragma unroll 1
          for (int c = 0; c < width; c += 32) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = 0.0f;
            // two owners' partials in flight at a time, added in ascending owner order
            for (int owner = first_owner; owner <= last_owner; owner += 2) {
              const bool two = owner + 1 <= last_owner;
              const int slot0 = streamk_slot(total_iters, p.streamk_workers, p.k_iters, owner, sk_tile);
              const int slot1 = two ? streamk_slot(total_iters, p.streamk_workers, p.k_iters, owner + 1, sk_tile) : 0;
              const float4 *src0 = reinterpret_cast<const float4 *>(
                  p.scratch + ((static_cast<size_t>(owner) * 2 + slot0) * 2 + rank) * (kRows * PN));
              const float4 *src1 = reinterpret_cast<const float4 *>(
                  p.scratch + ((static_cast<size_t>(two ? owner + 1 : owner) * 2 + slot1) * 2 + rank) * (kRows * PN));
              float4 x0[8], x1[8];
#pragma unroll
              for (int k = 0; k < 8; ++k)
                x0[k] = __ldcg(src0 + ((c >> 2) + k) * kRows + row_in_tile);
              if (two) {
#pragma unroll
                for (int k = 0; k < 8; ++k)
                  x1[k] = __ldcg(src1 + ((c >> 2) + k) * kRows + row_in_tile);
              }
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                v[4 * k] += x0[k].x;
                v[4 * k + 1] += x0[k].y;
                v[4 * k + 2] += x0[k].z;
                v[4 * k + 3] += x0[k].w;
              }
              if (two) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                  v[4 * k] += x1[k].x;
                  v[4 * k + 1] += x1[k].y;
                  v[4 * k + 2] += x1[k].z;
                  v[4 * k + 3] += x1[k].w;
                }
              }
            }
            store_row_chunk<T, 32>(p, m, n_tile0 + c, v);
          }
          if (row_in_tile == 0)
            atomicAdd(counter, -parts); // back to zero for the next launch
        }
        epilogue_barrier(); // sh->last_arriver may be rewritten
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
        continue;
      }
      if constexpr (sizeof(T) == 2) {
        if (p.c_tma) {
          // Row-major 16-bit output: 64 columns of the CTA's 128 rows at a time go
          // through a swizzled shared-memory tile and out with one TMA store (whole
          // 128-byte rows instead of 16 bytes per thread; the store clips at the
          // matrix edge).  Two tiles, so that a store reads one while the four
          // epilogue warps fill the other.
          int c = 0;
#pragma unroll 1
          for (; c + kStoreCols <= width; c += kStoreCols, ++store_n) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(taddr + c, r0);
            tmem_ld_32x32b_x32(taddr + c + 32, r1);
            tmem_ld_wait();
            if (c + kStoreCols >= width) { // the accumulator has been read: the next tile may use it
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0)
                mbar_arrive_cluster(tempty_leader[acc]);
            }
            uint8_t *buf = store_tiles + (store_n & 1u) * kStoreTileBytes;
            if (warp == 2 && lane == 0)
              tma_store_wait_read<1>(); // the store that last used this tile has read it
            epilogue_barrier();
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
            epilogue_barrier();
            if (warp == 2 && lane == 0) {
              tma_store_2d_evict_first(&tmap_c, buf, n_tile0 + n_off + c,
                                       mb * kPairM + static_cast<int>(rank) * kRows);
              if constexpr (kTmaExtra) {
                // The same piece to every further copy of C (peer GPUs' memory when
                // the column blocks are being gathered): one more TMA store each,
                // in the same bulk group; no thread touches the data again.
#pragma unroll 1
                for (int x = 0; x < p.n_extra; ++x)
                  tma_store_2d(&em->m[x], buf, n_tile0 + n_off + c, mb * kPairM + static_cast<int>(rank) * kRows);
              }
              tma_store_commit();
            }
            if (!kTmaExtra && p.n_extra > 0) {
              // The same 128 x 64 piece to every further copy of C (peer GPUs'
              // memory when the column blocks are being gathered): the four warps
              // read the staging tile back, un-swizzled, and write whole 128-byte
              // rows -- a warp covers four rows per store instruction.  Plain
              // stores; they drain over NVLink while the next tile is computed.
              const int et = row_in_tile;            // 0..127
              const int chunk = et & 7;              // 16-byte chunk of the 128-byte row
              const int col = n_tile0 + n_off + c + chunk * 8;
              if (col < p.N) {
#pragma unroll 1
                for (int i = 0; i < 8; ++i) {
                  const int r = (et >> 3) + 16 * i;  // row of the staging tile
                  const int gm = mb * kPairM + static_cast<int>(rank) * kRows + r;
                  if (gm >= p.M)
                    break;
                  const uint4 v = *reinterpret_cast<const uint4 *>(buf + r * (kStoreCols * 2) + ((chunk ^ (r & 7)) << 4));
                  const long long off = static_cast<long long>(gm) * p.stride_m + col;
                  if (p.extra_multimem)
                    multimem_st_16B(reinterpret_cast<T *>(p.extra_c[0]) + off, v);
                  else
                    for (int x = 0; x < p.n_extra; ++x)
                      *reinterpret_cast<uint4 *>(reinterpret_cast<T *>(p.extra_c[x]) + off) = v;
                }
              }
            }
          }
          if (c < width) {
            // Tile widths that are not a multiple of 64 leave 32 columns: per-thread stores.
            uint32_t r[32];
            tmem_ld_32x32b_x32(taddr + c, r);
            tmem_ld_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0)
              mbar_arrive_cluster(tempty_leader[acc]);
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = __uint_as_float(r[j]);
            store_row_chunk<T, 32>(p, m, n_tile0 + n_off + c, v);
            if (p.n_extra > 0 && m < p.M) {
              T tmp[32];
#pragma unroll
              for (int j = 0; j < 32; ++j)
                store_elem(&tmp[j], v[j]);
              const int col = n_tile0 + n_off + c;
              const long long off = static_cast<long long>(m) * p.stride_m + col;
              for (int x = 0; x < p.n_extra; ++x)
#pragma unroll
                for (int q = 0; q < 4; ++q)
                  if (col + 8 * q < p.N) {
                    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<T *>(p.extra_c[x]) + off) + q;
                    if (p.extra_multimem)
                      multimem_st_16B(dst, reinterpret_cast<const uint4 *>(tmp)[q]);
                    else
                      *dst = reinterpret_cast<const uint4 *>(tmp)[q];
                  }
            }
          }
          if (++acc == 2) {
            acc = 0;
            acc_phase ^= 1;
          }
          continue;
        }
      }
#pragma unroll 1
      for (int c = 0; c < width; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          v[j] = __uint_as_float(r[j]);
        store_row_chunk<T, 32>(p, m, n_tile0 + n_off + c, v);
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
    if (warp == 2 && lane == 0)
      tma_store_wait_read<0>(); // the staging tiles must outlive the stores that read them
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

template <int OUT, int PN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_b_half, const __grid_constant__ CUtensorMap tmap_c,
                 const GemmParams p) {
  gemm_pair_body<OUT, PN, false>(tmap_a, tmap_b, tmap_b_half, tmap_c, p, nullptr);
}

template <int OUT, int PN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_extra_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_b_half, const __grid_constant__ CUtensorMap tmap_c,
                       const GemmParams p, const __grid_constant__ PairExtraMaps em) {
  gemm_pair_body<OUT, PN, true>(tmap_a, tmap_b, tmap_b_half, tmap_c, p, &em);
}

// One launch; with `pdl` the stream may begin it (up to its griddepcontrol.wait)
// while the kernel before it is still finishing.
template <typename Kernel, typename... Args>
cudaError_t launch_config(int grid, int smem, cudaStream_t stream, int pdl, Kernel kernel, const Args &...args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(smem);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int OUT, int PN>
cudaError_t launch_pair(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tbh, const CUtensorMap &tc,
                        const GemmParams &p, const CUtensorMap *extra_maps, int grid, cudaStream_t stream) {
  constexpr int smem = PairCfg<PN>::kSmemBytes;
  if constexpr (OUT != WAVE_GEMM_OUT_F32) {
    if (extra_maps) {
      PairExtraMaps em;
      for (int i = 0; i < 7; ++i)
        em.m[i] = extra_maps[i < p.n_extra ? i : 0];
      cudaError_t err = prepare_kernel(gemm_pair_extra_kernel<OUT, PN>, smem, nullptr);
      if (err != cudaSuccess)
        return err;
      return launch_config(grid, smem, stream, p.pdl, gemm_pair_extra_kernel<OUT, PN>, ta, tb, tbh, tc, p, em);
    }
  }
  cudaError_t err = prepare_kernel(gemm_pair_kernel<OUT, PN>, smem, nullptr);
  if (err != cudaSuccess)
    return err;
  return launch_config(grid, smem, stream, p.pdl, gemm_pair_kernel<OUT, PN>, ta, tb, tbh, tc, p);
}

template <int PN>
cudaError_t launch_pair_out(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tbh, const CUtensorMap &tc,
                            const GemmParams &p, const CUtensorMap *extra_maps, int grid, cudaStream_t stream) {
  switch (p.out_type) {
  case WAVE_GEMM_OUT_F32:
    return launch_pair<WAVE_GEMM_OUT_F32, PN>(ta, tb, tbh, tc, p, extra_maps, grid, stream);
  case WAVE_GEMM_OUT_F16:
    return launch_pair<WAVE_GEMM_OUT_F16, PN>(ta, tb, tbh, tc, p, extra_maps, grid, stream);
  case WAVE_GEMM_OUT_BF16:
    return launch_pair<WAVE_GEMM_OUT_BF16, PN>(ta, tb, tbh, tc, p, extra_maps, grid, stream);
  }
  return cudaErrorInvalidValue;
}

} // namespace

int gemm_pair_tile_m() { return kPairM; }
int gemm_pair_tile_n() { return 256; }
int gemm_pair_box_rows() { return kRows; }

// `grid` must be even: consecutive CTAs form the pairs.  `tile_n` is 128 (the
// narrow instantiation) or a multiple of 32 in (128, 256] (the wide one, whose
// tiles are then p.pair_tile_n = tile_n columns wide); the tensor map of B must
// have a box of tile_n / 2 rows, `tmap_b_half`
// (read only when tile_n is 256 and p.split_from < p.num_tiles) one of 64 rows,
// `tmap_c` (read only when p.c_tma is set) a box of 64 columns x 128 rows over
// the row-major 16-bit output.  Rows of C a store may touch beyond M, and
// columns beyond N, are clipped by the tensor map.  `extra_maps` (or null):
// p.n_extra maps like `tmap_c` over the further copies of C, which then get
// every piece by TMA store (16-bit output with p.c_tma only).
cudaError_t launch_gemm_pair(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, const CUtensorMap &tmap_b_half,
                             const CUtensorMap &tmap_c, const GemmParams &p, const CUtensorMap *extra_maps, int tile_n,
                             int grid, cudaStream_t stream) {
  if (tile_n == 128)
    return launch_pair_out<128>(tmap_a, tmap_b, tmap_b_half, tmap_c, p, extra_maps, grid, stream);
  if (tile_n > 128 && tile_n <= 256 && tile_n % 32 == 0) {
    GemmParams q = p;
    q.pair_tile_n = tile_n;
    return launch_pair_out<256>(tmap_a, tmap_b, tmap_b_half, tmap_c, q, extra_maps, grid, stream);
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
