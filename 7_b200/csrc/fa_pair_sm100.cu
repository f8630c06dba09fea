// Flash-attention forward for sm_100a, CTA-pair variant: two CTAs of a 2-CTA
// cluster work on 512 query rows of one head with tcgen05.mma cta_group::2
// (UMMA 256 x 128 x 16).  Same operator and numerics as fa_sm100.cu, the
// stand-in for the reference's `flash_attention_bf16_gfx950`
// (python/mlir/dialects/wave_flash_attention.py:452-728, 1034-1095): exp2 with
// scale*log2(e) folded into the exponent (:596-600), f32 row sums of the
// unrounded probabilities with 16-bit probabilities feeding P*V (:706-722),
// lazy accumulator rescale with threshold 8 in log2 units (:557-583).
//
// What the pair buys.  One thread (in the even CTA, the "leader") issues every
// MMA for both SMs, and each CTA supplies only half of every B operand from
// its own shared memory: 64 of a block's 128 keys for S = Q K^T, 64 of the 128
// head-dimension columns of V for O += P V.  Per CTA that halves the K/V bytes
// loaded per block (32 KB instead of 64 KB, which pays for four-stage rings
// instead of two) and takes a third off the shared-memory bytes the Q K^T MMAs
// read per cycle.  No load uses cluster multicast: every TMA load targets the
// loading CTA's own shared memory and only its completion is counted on the
// leader's barrier.
//
// Work item: 512 query rows of one (batch, head), drawn by the leader's loader
// from the ticket counter and published to both CTAs.  Pair tile t (t = 0, 1)
// is rows [512 q + 256 t, +256): CTA r owns its rows [.. + 128 r, +128), so a
// CTA runs two 128-row tiles that ping-pong exactly as in fa_sm100.cu.  With
// the causal mask a pair tile visits the K/V blocks its LOWER half needs; the
// upper half's last block is then fully masked (3 % more MMA work at S = 4096).
//
// Roles per CTA (384 threads): warp 0 loader, warp 1 UMMA issuer (leader only;
// it also allocates tensor memory in both CTAs), warps 4..7 / 8..11 softmax of
// tile 0 / 1, one thread per query row.  TMEM per CTA: S_0 | S_1 | O_0 | O_1,
// 128 f32 columns each; P_t overwrites the first 64 columns of S_t.
//
// Barriers.  "leader": lives in the even CTA, the odd CTA signals it remotely.
//   item_full[2]   per CTA   leader's loader publishes the item index to both
//   item_empty[2]  leader    UMMA thread, peer's loader, 16 softmax warps
//   q_full         leader    TMA bytes of both CTAs;   q_empty   per CTA (commit)
//   k_full/v_full  leader    TMA bytes of both CTAs;   k_empty/v_empty per CTA (commit)
//   s_full[t], o_full[t]  per CTA (commit to both)
//   p_full[t], o_free[t]  leader   one arrival per softmax warp of both CTAs
#include "../../include/wave_cuda.h"
#include "fa_common.cuh"
#include "fa_sm100.h"
#include "launch_cache.h"
#include "sm100_ptx.cuh"

#include <type_traits>

namespace wave {

void set_last_error(const char *message); // wave_cuda_backend.cu

__device__ int g_fa_pair_status[4]; // [0] code, [1] block, [2] role (30..), [3] detail

namespace {

using namespace fa_detail;

constexpr int kBlockM = 128;           // rows per Q tile of one CTA = TMEM lanes
constexpr int kPairM = 256;            // UMMA M across the pair
constexpr int kItemRows = 2 * kPairM;  // query rows per work item
constexpr int kBlockN = 128;           // keys per K/V block
constexpr int kD = 128;
constexpr int kThreads = 384;
constexpr int kSubTile = 128 * 64 * 2; // [128 rows][64 elements], 128-byte swizzled rows
constexpr int kQTile = 2 * kSubTile;   // a CTA's 128 x 128 Q tile
constexpr int kKHalf = 64 * 64 * 2;    // [64 keys][64 elements]: one head-dimension chunk of a CTA's half of a K block
constexpr int kKStage = 2 * kKHalf;    // a CTA's 64 keys x 128 elements
constexpr int kVStage = kSubTile;      // a CTA's 128 keys x 64 head-dimension columns
constexpr int kStages = 4;
constexpr int kSmemTiles = 2 * kQTile + kStages * kKStage + kStages * kVStage;
constexpr int kSmemBytes = kSmemTiles + 1024 + 512;
constexpr int kTmemCols = 512;
constexpr int kDefaultPoly = 0;
constexpr float kRescaleThreshold = 8.0f; // log2 units (wave_flash_attention.py:563-569)
// setmaxnreg budget, as in fa_sm100.cu.
constexpr int kLaunchRegs = 168;
constexpr int kIssueRegs = 72;
constexpr int kSoftmaxRegs = 216;
static_assert((kLaunchRegs - kIssueRegs) * 128 >= (kSoftmaxRegs - kLaunchRegs) * 256,
              "setmaxnreg.inc would wait forever: warpgroup 0 does not release enough registers");

struct PairShared {
  uint64_t item_full[2], item_empty[2];
  uint64_t q_full, q_empty;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], o_full[2], o_free[2];
  uint32_t tmem_base;
  int abort_flag;
  int item_idx[2];
};
static_assert(sizeof(PairShared) <= 512, "shared state does not fit its slot");

struct PairItem {
  int q_blk, bh;
  int n_blocks[2]; // K/V blocks each pair tile visits (0: the tile is past the end of Q)
  int n_max;
};
__device__ __forceinline__ PairItem decode_item(int idx, const FaParams &p) {
  PairItem w;
  const int nq = (p.seq_q + kItemRows - 1) / kItemRows;
  w.bh = idx / nq;
  w.q_blk = nq - 1 - idx % nq; // heaviest causal items of a head first
  const int n_kv_blocks = (p.seq_k + kBlockN - 1) / kBlockN;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0 = w.q_blk * kItemRows + t * kPairM;
    int n = 0;
    if (q0 < p.seq_q) {
      n = n_kv_blocks;
      if (p.causal)
        n = min(n, q0 / kBlockN + 2); // the last row of the pair tile is q0 + 255
    }
    w.n_blocks[t] = n;
  }
  w.n_max = max(w.n_blocks[0], w.n_blocks[1]);
  return w;
}

__device__ __noinline__ void pair_report(int code, int role, int detail) {
  if (atomicCAS(&g_fa_pair_status[0], 0, code) == 0) {
    g_fa_pair_status[1] = static_cast<int>(blockIdx.x);
    g_fa_pair_status[2] = role;
    g_fa_pair_status[3] = detail;
  }
}

// ---- PTX pieces only this kernel uses -----------------------------------
// Bounded wait with acquire semantics at cluster scope: for barriers that the
// other CTA of the pair arrives on after writing this CTA's shared or tensor
// memory.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(smem_u32(bar)), "r"(parity)
               : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  const long long start = clock64();
  for (uint32_t tries = 1;; ++tries) {
    if (mbar_try_wait_cluster(bar, parity))
      return true;
    if ((tries & 15u) == 0) {
      if (*abort_flag)
        return false;
      if (clock64() - start > kWaitLimitCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// TMA load of this CTA's own operand half into its own shared memory; the
// bytes are counted on the barrier at `bar`'s offset in the LEADER CTA.
__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const CUtensorMap *tmap, uint64_t *bar, int x, int y,
                                                 int z) {
  asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
               " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar) & kPeerBitMask), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// cta_group::2 forms of umma_ss_halves / umma_ts_halves (sm100_ptx.cuh).
template <int kAccumulate>
__device__ __forceinline__ void umma_ss_halves_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                    uint32_t idesc, uint32_t accumulate = 1) {
  if constexpr (kAccumulate < 0) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                 "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
                 "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
                 : "memory");
  } else {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                 "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
                 "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(kAccumulate)
                 : "memory");
  }
}
template <int kAccumulate>
__device__ __forceinline__ void umma_ts_halves_pair(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t desc_hi,
                                                    uint32_t idesc, uint32_t accumulate = 1) {
  if constexpr (kAccumulate < 0) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                 "mov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(tmem_d),
                 "r"(tmem_a), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
                 : "memory");
  } else {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\t"
                 "mov.b64 db, {%2, %3};\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(tmem_d),
                 "r"(tmem_a), "r"(b_lo), "r"(desc_hi), "r"(idesc), "n"(kAccumulate)
                 : "memory");
  }
}

// kExtra: the epilogue also writes O to the launch's further output buffers
// (FaExtra); compiled out of the ordinary kernels.
template <int kPoly, bool kBf16, bool kExtra>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
fa_pair_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const FaParams p, const __grid_constant__ FaExtra ex) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = tiles;                                   // 2 tiles
  uint8_t *k_smem = tiles + 2 * kQTile;                      // kStages stages
  uint8_t *v_smem = k_smem + kStages * kKStage;              // kStages stages
  PairShared *sh = reinterpret_cast<PairShared *>(tiles + kSmemTiles);
  volatile int *abort_flag = &sh->abort_flag;
  // the variants with further output buffers: 2 KB per softmax warp behind everything else
  uint8_t *extra_stage = tiles + (kSmemBytes - 1024);
  (void)extra_stage;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int total_items = p.batch_heads * ((p.seq_q + kItemRows - 1) / kItemRows);

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->q_empty, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_empty[s], 1);
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->item_full[s], 1);
      mbar_init(&sh->item_empty[s], 18); // UMMA thread, the peer's loader, 8 softmax warps in each CTA
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->p_full[s], 8);      // one lane of each softmax warp of the tile, in both CTAs
      mbar_init(&sh->o_full[s], 1);
      mbar_init(&sh->o_free[s], 8);
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

  if (warp < 4)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIssueRegs));
  if (warp == 0) {
    // ---------------------------------------------------------------- loads
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const uint32_t peer_item_idx[2] = {map_to_cta(&sh->item_idx[0], 1), map_to_cta(&sh->item_idx[1], 1)};
      const uint32_t peer_item_full[2] = {map_to_cta(&sh->item_full[0], 1), map_to_cta(&sh->item_full[1], 1)};
      const uint32_t leader_item_empty[2] = {map_to_cta(&sh->item_empty[0], 0), map_to_cta(&sh->item_empty[1], 0)};
      bool ok = true;
      uint32_t kv_n = 0; // K/V blocks loaded so far: ring stage and phase carry over from item to item
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        int idx;
        if (leader) {
          if (!mbar_wait_cluster(&sh->item_empty[slot], ((n >> 1) & 1) ^ 1, abort_flag)) {
            pair_report(kStatusWaitTimeout, 30, 1);
            break;
          }
          idx = static_cast<int>(atomicAdd(p.ticket, 1u));
          sh->item_idx[slot] = idx;
          st_shared_cluster_u32(peer_item_idx[slot], static_cast<uint32_t>(idx));
          mbar_arrive(&sh->item_full[slot]);
          mbar_arrive_cluster(peer_item_full[slot]); // release at cluster scope: the index is visible to the peer
        } else {
          if (!mbar_wait_cluster(&sh->item_full[slot], (n >> 1) & 1, abort_flag)) {
            pair_report(kStatusWaitTimeout, 30, 2);
            break;
          }
          idx = sh->item_idx[slot];
          mbar_arrive_cluster(leader_item_empty[slot]);
        }
        if (idx >= total_items)
          break;
        const PairItem w = decode_item(idx, p);
        // Q of the previous item may be overwritten once its last Q*K^T has run.
        if (n > 0 && !mbar_wait(&sh->q_empty, (n - 1) & 1, abort_flag)) {
          pair_report(kStatusWaitTimeout, 30, 3);
          break;
        }
        const int q_tiles = (w.n_blocks[0] > 0) + (w.n_blocks[1] > 0);
        if (leader)
          mbar_arrive_expect_tx(&sh->q_full, static_cast<uint32_t>(q_tiles * 2 * kQTile));
        for (int t = 0; t < 2; ++t)
          if (w.n_blocks[t] > 0)
            for (int c = 0; c < 2; ++c)
              tma_load_3d_pair(q_smem + t * kQTile + c * kSubTile, &tm_q, &sh->q_full, c * 64,
                               w.q_blk * kItemRows + t * kPairM + static_cast<int>(rank) * kBlockM, w.bh);
        for (int j = 0; j < w.n_max && ok; ++j, ++kv_n) {
          const int s = kv_n % kStages;
          const uint32_t ph = (kv_n / kStages) & 1;
          if (!mbar_wait(&sh->k_empty[s], ph ^ 1, abort_flag)) {
            pair_report(kStatusWaitTimeout, 30, 10 + s);
            ok = false;
            break;
          }
          if (leader)
            mbar_arrive_expect_tx(&sh->k_full[s], 2 * kKStage);
          for (int c = 0; c < 2; ++c) // this CTA's 64 keys of the block, two head-dimension chunks
            tma_load_3d_pair(k_smem + s * kKStage + c * kKHalf, &tm_k, &sh->k_full[s], c * 64,
                             j * kBlockN + static_cast<int>(rank) * 64, w.bh);
          if (!mbar_wait(&sh->v_empty[s], ph ^ 1, abort_flag)) {
            pair_report(kStatusWaitTimeout, 30, 20 + s);
            ok = false;
            break;
          }
          if (leader)
            mbar_arrive_expect_tx(&sh->v_full[s], 2 * kVStage);
          // this CTA's 64 head-dimension columns of the block's 128 keys
          tma_load_3d_pair(v_smem + s * kVStage, &tm_v, &sh->v_full[s], static_cast<int>(rank) * 64, j * kBlockN, w.bh);
        }
      }
      if (!ok)
        bounded_delay(1 << 21);
    }
  } else if (warp == 1) {
    // ------------------------------------------------ UMMA issue (leader only)
    if (lane == 0 && leader) {
      const uint32_t idesc_s = umma_idesc_f16(kPairM, kBlockN, p.is_bf16, 0, 0);
      const uint32_t idesc_o = umma_idesc_f16(kPairM, kD, p.is_bf16, 0, 1); // V is MN-major
      // Descriptor halves (umma_desc_kmajor_sw128 / umma_desc_mnmajor_sw128): the
      // high half is the same for Q, K (K-major) and V (MN-major): stride 1024
      // bytes between 8-row groups, version 1, 128-byte swizzle.
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kQTile16 = kQTile >> 4, kSub16 = kSubTile >> 4, kKStage16 = kKStage >> 4,
                         kKHalf16 = kKHalf >> 4, kVStage16 = kVStage >> 4;
      const uint32_t q_lo = ((smem_u32(q_smem) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t k_lo = ((smem_u32(k_smem) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t v_lo = ((smem_u32(v_smem) & 0x3FFFFu) >> 4) | (1u << 16); // one 64-column chunk: no chunk stride
      bool ok = true;

      // S_t = Q_t K_j^T over the pair: K = head dim, two 64-element swizzle chunks x four UMMA K steps
      auto issue_s = [&](int t, int stage) {
        const uint32_t d = tmem_base + static_cast<uint32_t>(t * kBlockN);
        const uint32_t a = q_lo + static_cast<uint32_t>(t) * kQTile16;
        const uint32_t b = k_lo + static_cast<uint32_t>(stage) * kKStage16;
        umma_ss_halves_pair<0>(d, a, b, kDescHi, idesc_s);
#pragma unroll
        for (int i = 1; i < 8; ++i) {
          const uint32_t off_a = static_cast<uint32_t>((i >> 2) * kSub16 + (i & 3) * 2);
          const uint32_t off_b = static_cast<uint32_t>((i >> 2) * kKHalf16 + (i & 3) * 2);
          umma_ss_halves_pair<1>(d, a + off_a, b + off_b, kDescHi, idesc_s);
        }
        umma_commit_pair(&sh->s_full[t], 3);
      };
      // O_t += P_t V_j: K = 128 keys in eight steps of 16; P from each CTA's TMEM
      // (8 packed columns per step), V rows are keys (128 bytes each), 16 keys = 2048 bytes.
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t d = tmem_base + static_cast<uint32_t>(2 * kBlockN + t * kD);
        const uint32_t a = tmem_base + static_cast<uint32_t>(t * kBlockN);
        const uint32_t b = v_lo + static_cast<uint32_t>(stage) * kVStage16;
        umma_ts_halves_pair<-1>(d, a, b, kDescHi, idesc_o, accumulate ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          umma_ts_halves_pair<1>(d, a + static_cast<uint32_t>(kk * 8), b + static_cast<uint32_t>(kk * (2048 >> 4)),
                                 kDescHi, idesc_o);
      };

      uint32_t kv_n = 0;               // K/V blocks consumed so far
      uint32_t p_n[2] = {0, 0};        // P hand-offs waited for, per tile
      uint32_t tile_items[2] = {0, 0}; // items in which the tile had work (o_full / o_free phases)
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_full[slot], (n >> 1) & 1, abort_flag)) {
          pair_report(kStatusWaitTimeout, 31, 3);
          break;
        }
        const int idx = sh->item_idx[slot];
        mbar_arrive(&sh->item_empty[slot]);
        if (idx >= total_items)
          break;
        const PairItem w = decode_item(idx, p);
        const int n_max = w.n_max;
        if (!mbar_wait(&sh->q_full, n & 1, abort_flag)) {
          pair_report(kStatusWaitTimeout, 31, 1);
          break;
        }
        {
          const int s0 = kv_n % kStages;
          if (!mbar_wait(&sh->k_full[s0], (kv_n / kStages) & 1, abort_flag)) {
            pair_report(kStatusWaitTimeout, 31, 2);
            break;
          }
          tc_fence_after_sync();
          if (w.n_blocks[0] > 0)
            issue_s(0, s0);
          if (w.n_blocks[1] > 0)
            issue_s(1, s0);
          umma_commit_pair(&sh->k_empty[s0], 3);
          if (n_max == 1)
            umma_commit_pair(&sh->q_empty, 3); // no further Q*K^T in this item
        }
        for (int j = 0; j < n_max && ok; ++j, ++kv_n) {
          const int s = kv_n % kStages;
          const uint32_t ph = (kv_n / kStages) & 1;
          const int s_next = (kv_n + 1) % kStages;
          const uint32_t ph_next = ((kv_n + 1) / kStages) & 1;
          bool have_v = false, have_k_next = false;
          for (int t = 0; t < 2 && ok; ++t) {
            if (j >= w.n_blocks[t])
              continue;
            if (!have_v) {
              if (!mbar_wait(&sh->v_full[s], ph, abort_flag)) {
                pair_report(kStatusWaitTimeout, 31, 30 + s);
                ok = false;
                break;
              }
              have_v = true;
            }
            // K of the next block was requested blocks ago; looking at its barrier
            // ahead of the wait for P keeps that look out of the tile's chain.
            if (j + 1 < w.n_blocks[t] && !have_k_next) {
              if (!mbar_wait(&sh->k_full[s_next], ph_next, abort_flag)) {
                pair_report(kStatusWaitTimeout, 31, 50 + s_next);
                ok = false;
                break;
              }
              have_k_next = true;
            }
            if (!mbar_wait_cluster(&sh->p_full[t], p_n[t] & 1, abort_flag)) {
              pair_report(kStatusWaitTimeout, 31, 40 + t);
              ok = false;
              break;
            }
            ++p_n[t];
            // The first P*V of an item overwrites O_t: the previous item's
            // epilogues (in both CTAs) must have read it out.
            if (j == 0 && tile_items[t] > 0 && !mbar_wait_cluster(&sh->o_free[t], (tile_items[t] - 1) & 1, abort_flag)) {
              pair_report(kStatusWaitTimeout, 31, 45 + t);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(t, s, j > 0);
            if (j + 1 < w.n_blocks[t]) {
              issue_s(t, s_next);
            } else {
              umma_commit_pair(&sh->o_full[t], 3);
              ++tile_items[t];
            }
          }
          if (!ok)
            break;
          umma_commit_pair(&sh->v_empty[s], 3);
          if (have_k_next)
            umma_commit_pair(&sh->k_empty[s_next], 3);
          if (j + 2 == n_max)
            umma_commit_pair(&sh->q_empty, 3); // the last Q*K^T of the item has been issued
        }
      }
    }
  } else if (warp >= 4) {
    // --------------------------------------------------------------- softmax
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int t = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const float c = p.scale_log2e;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + static_cast<uint32_t>(t * kBlockN);
    const uint32_t o_addr = tmem_base + lane_base + static_cast<uint32_t>(2 * kBlockN + t * kD);
    const uint32_t p_full_leader = map_to_cta(&sh->p_full[t], 0);
    const uint32_t o_free_leader = map_to_cta(&sh->o_free[t], 0);
    const uint32_t item_empty_leader[2] = {map_to_cta(&sh->item_empty[0], 0), map_to_cta(&sh->item_empty[1], 0)};
    constexpr bool bf16 = kBf16;
    uint32_t s_n = 0;        // score blocks consumed so far by this tile (s_full phase)
    uint32_t tile_items = 0; // items in which this tile had work (o_full phase)
    bool ok = true;

    for (uint32_t item_n = 0; ok; ++item_n) {
      const int slot = item_n & 1;
      if (!mbar_wait_cluster(&sh->item_full[slot], (item_n >> 1) & 1, abort_flag)) {
        if (lane == 0)
          pair_report(kStatusWaitTimeout, 32 + t, 59);
        break;
      }
      const int idx = sh->item_idx[slot];
      __syncwarp();
      if (lane == 0)
        mbar_arrive_cluster(item_empty_leader[slot]);
      if (idx >= total_items)
        break;
      const PairItem w = decode_item(idx, p);
      const int bh = w.bh;
      const int q_row = w.q_blk * kItemRows + t * kPairM + static_cast<int>(rank) * kBlockM + row;
      const int nb = w.n_blocks[t];
      // Maximum the exponentials are taken against (raw score units): the running
      // row maximum, or with a fixed reference the caller's bound for the whole item.
      float m_used = p.fixed_ref ? p.ref_log2 / c : -INFINITY;
      float l = 0.0f; // running sum of unrounded probabilities

      for (int j = 0; j < nb; ++j) {
        if (!mbar_wait(&sh->s_full[t], s_n & 1, abort_flag)) {
          if (lane == 0)
            pair_report(kStatusWaitTimeout, 32 + t, 60);
          ok = false;
          break;
        }
        ++s_n;
        tc_fence_after_sync();
        uint32_t s[128];
        tmem_ld_32x32b_x32(s_addr + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld_32x32b_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_ld_32x32b_x32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
        tmem_ld_32x32b_x32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
        tmem_ld_wait();

        const int key0 = j * kBlockN;
        const bool need_mask = (p.causal && key0 + kBlockN - 1 > q_row - row) || (key0 + kBlockN > p.seq_k);
        if (need_mask) {
          const int limit = p.causal ? min(q_row, p.seq_k - 1) : p.seq_k - 1; // last visible key
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (key0 + i > limit)
              s[i] = 0xFF800000u; // -inf
        }
        if (!p.fixed_ref) {
          float mx[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            mx[i] = fmaxf(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1]));
#pragma unroll
          for (int i = 32; i < 128; i += 32)
#pragma unroll
            for (int k = 0; k < 16; ++k)
              mx[k] = max3(mx[k], __uint_as_float(s[i + 2 * k]), __uint_as_float(s[i + 2 * k + 1]));
#pragma unroll
          for (int k = 0; k < 5; ++k)
            mx[k] = max3(mx[k], mx[5 + 2 * k], mx[6 + 2 * k]);
          mx[0] = max3(mx[0], mx[1], mx[2]);
          mx[3] = max3(mx[3], mx[4], mx[15]);
          const float m_new = max3(m_used, mx[0], mx[3]);
          // Lazy rescale: only when some row of this warp moved its maximum by more
          // than 2^8; otherwise keep the stale maximum (exact after the final divide).
          // (A block that the causal mask hides from this CTA's whole tile leaves
          // m_new = m_used, which is finite from block 0 on: no rescale, all P = 0.)
          const bool need = (m_new - m_used) * c > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            const float factor = fast_exp2((m_used - m_new) * c);
            l *= factor;
            if (j > 0) {
#pragma unroll 1
              for (int cc = 0; cc < kD; cc += 32) {
                uint32_t o[32];
                tmem_ld_32x32b_x32(o_addr + cc, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
                tmem_st_32x32b_x32(o_addr + cc, o);
              }
            }
            m_used = m_new;
          }
        }
        const float neg_mc = -m_used * c;
        const float2 c2 = make_float2(c, c), nm2 = make_float2(neg_mc, neg_mc);
        float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float2 x =
              __ffma2_rn(make_float2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), c2, nm2);
          float2 pr;
          if (pair_uses_poly<kPoly>(i))
            pr = exp2_poly2(x);
          else
            pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          if (i & 1)
            lb = __fadd2_rn(lb, pr);
          else
            la = __fadd2_rn(la, pr);
          pk[i] = pack2(pr.x, pr.y, bf16);
        }
        l += (la.x + la.y) + (lb.x + lb.y);
        tmem_st_32x32b_x32(s_addr + 0, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
        tmem_st_32x32b_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive_cluster(p_full_leader);
      }

      if (ok && nb > 0) {
        if (!mbar_wait(&sh->o_full[t], tile_items & 1, abort_flag)) {
          if (lane == 0)
            pair_report(kStatusWaitTimeout, 32 + t, 70);
          ok = false;
        } else {
          ++tile_items;
          tc_fence_after_sync();
          const float inv = 1.0f / l;
          const bool live = q_row < p.seq_q;
          // Head dimensions below 128 ran zero-padded (TMA fills the missing
          // columns of Q, K and V with zeros); only the first head_dim columns of
          // O exist in memory.  Output is the I/O type, or f32 on request.
          const int esize = p.out_f32 ? 4 : 2;
          uint8_t *out_row = static_cast<uint8_t *>(p.O) +
                             (static_cast<size_t>(bh) * p.seq_q + static_cast<size_t>(live ? q_row : 0)) *
                                 static_cast<size_t>(p.head_dim) * esize;
#pragma unroll 1
          for (int cc = 0; cc < p.head_dim; cc += 32) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(o_addr + cc, o);
            tmem_ld_wait();
            if (p.out_f32) {
              if (live) {
                float4 *dst = reinterpret_cast<float4 *>(out_row + cc * 4);
#pragma unroll
                for (int v = 0; v < 8; ++v)
                  if (cc + 4 * v < p.head_dim) { // head_dim is a multiple of 16
                    const float4 f = make_float4(__uint_as_float(o[4 * v]) * inv, __uint_as_float(o[4 * v + 1]) * inv,
                                                 __uint_as_float(o[4 * v + 2]) * inv, __uint_as_float(o[4 * v + 3]) * inv);
                    dst[v] = f;
                    if constexpr (kExtra)
                      store_extra_16B(ex, static_cast<size_t>(out_row - static_cast<uint8_t *>(p.O)) + (cc + 4 * v) * 4,
                                      make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w)));
                  }
              }
            } else {
              uint32_t wv[16];
#pragma unroll
              for (int i = 0; i < 16; ++i)
                wv[i] = pack2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv, bf16);
              if (live) {
                uint4 *dst = reinterpret_cast<uint4 *>(out_row + cc * 2);
#pragma unroll
                for (int v = 0; v < 4; ++v)
                  if (cc + 8 * v < p.head_dim) {
                    dst[v] = make_uint4(wv[4 * v], wv[4 * v + 1], wv[4 * v + 2], wv[4 * v + 3]);
                  }
              }
              if constexpr (kExtra) {
                const int first_row = q_row - lane; // a warp's 32 rows are consecutive
                store_extra_chunk_16bit(ex, extra_stage + (warp - 4) * 2048, lane, wv,
                                        (static_cast<size_t>(bh) * p.seq_q + first_row) * p.head_dim * 2 + static_cast<size_t>(cc) * 2,
                                        static_cast<size_t>(p.head_dim) * 2, min(32, max(0, p.seq_q - first_row)),
                                        min(64, (p.head_dim - cc) * 2));
              }
            }
          }
          if (p.lse && live)
            p.lse[static_cast<size_t>(bh) * p.seq_q + q_row] = m_used * p.scale + logf(l);
          // O_t has been read out: the next item's first P*V may overwrite it.
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0)
            mbar_arrive_cluster(o_free_leader);
        }
      }
    } // work items
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

} // namespace

// `tq` and `tv`: boxes of 64 elements x 128 rows over Q and V; K gets a map of
// its own here (64 elements x 64 rows: a CTA loads half of a block's keys).
int launch_flash_attention_pair(const FaParams &p, const FaExtra &extra, const CUtensorMap &tq, const void *K,
                                const CUtensorMap &tv, int poly, int sm_count, cudaStream_t stream) {
  CUtensorMap tk;
  {
    const uint64_t hd = static_cast<uint64_t>(p.head_dim), row_bytes = hd * 2;
    const uint64_t dims[3] = {hd, static_cast<uint64_t>(p.seq_k), static_cast<uint64_t>(p.batch_heads)};
    const uint64_t strides[2] = {row_bytes, row_bytes * static_cast<uint64_t>(p.seq_k)};
    const uint32_t box[3] = {64, 64, 1};
    const int rc = make_tensor_map_16bit(&tk, p.is_bf16, K, 3, dims, strides, box);
    if (rc != WAVE_OK)
      return rc;
  }
  const long long total_items = static_cast<long long>(p.batch_heads) * ((p.seq_q + kItemRows - 1) / kItemRows);
  const long long pairs = total_items < sm_count / 2 ? total_items : sm_count / 2;
  const unsigned grid = static_cast<unsigned>(2 * pairs);
  cudaError_t err = cudaSuccess;
  bool unsafe_budget = false;
  auto launch = [&](auto kernel) {
    // The setmaxnreg arithmetic in the kernel assumes the register count the
    // compiler actually gave it; refuse to launch rather than risk a grow
    // request that can never be satisfied.
    KernelInfo info;
    const int smem_bytes = kSmemBytes + (extra.n > 0 ? kExtraStageBytes : 0);
    err = prepare_kernel(kernel, smem_bytes, &info);
    if (err != cudaSuccess)
      return;
    if ((info.num_regs - kIssueRegs) * 128 < (kSoftmaxRegs - info.num_regs) * 256 || info.num_regs * kThreads > 65536) {
      unsafe_budget = true;
      return;
    }
    kernel<<<grid, kThreads, smem_bytes, stream>>>(tq, tk, tv, p, extra);
    err = cudaGetLastError();
  };
  auto dispatch = [&](auto bf16_tag) {
    constexpr bool B = decltype(bf16_tag)::value;
    if (extra.n > 0) { // further output buffers: the kernel variant whose epilogue writes them (default polynomial share)
      launch(fa_pair_kernel<kDefaultPoly, B, true>);
      return;
    }
    switch (poly) {
    case 1: launch(fa_pair_kernel<1, B, false>); break;
    case 2: launch(fa_pair_kernel<2, B, false>); break;
    case 3: launch(fa_pair_kernel<3, B, false>); break;
    case 4: launch(fa_pair_kernel<4, B, false>); break;
    default: launch(fa_pair_kernel<kDefaultPoly, B, false>); break;
    }
  };
  if (p.is_bf16)
    dispatch(std::true_type{});
  else
    dispatch(std::false_type{});
  if (unsafe_budget) {
    set_last_error("attention kernel was built with a register count its setmaxnreg budget does not cover");
    return WAVE_E_CUDA;
  }
  if (err != cudaSuccess) {
    set_last_error(cudaGetErrorString(err));
    return WAVE_E_CUDA;
  }
  return WAVE_OK;
}

cudaError_t fa_pair_read_status(int out[4], bool clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fa_pair_status, sizeof(int) * 4);
  if (err == cudaSuccess && clear) {
    int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(g_fa_pair_status, zero, sizeof(zero));
  }
  return err;
}

} // namespace wave
