// Flash-attention forward for sm_100a, the decoupled kernel: two 128-row Q
// tiles per CTA like fa_sm100.cu, but K/V blocks of 80 keys, so that tensor
// memory has room for the probabilities NEXT TO the scores:
//     S_0 | S_1 (80 f32 columns each) | P_0 | P_1 (40 columns of 16-bit pairs) | O_0 | O_1 (128 each)
// With 128-key blocks S_0 S_1 O_0 O_1 fill all 512 columns, P has to overwrite
// S, Q*K^T of a tile's next block has to wait for P*V of the current one, and
// one tile's chain softmax -> P*V -> Q*K^T -> softmax paces the kernel.  Here
// a tile's softmax threads pull the score row into registers and release S at
// once: Q*K^T(j+1) runs during softmax(j), P*V(j) during softmax(j+1), and the
// softmax warps do not wait for the tensor core in the steady state.  Three
// threads issue UMMAs (Q*K^T of tile 0 from warp 1, of tile 1 from warp 3, P*V
// of both from warp 2), so a wait of one never holds back the others; warp 0
// loads Q, K and V in the order of use.
//
// Same arithmetic per element as fa_sm100.cu (see there for the reference
// lines: python/mlir/dialects/wave_flash_attention.py:452-728); the running
// maximum moves in steps of 80 keys instead of 128, so results agree with the
// other kernels to rounding, not bit for bit.  No load uses cluster multicast.
// The variants with further output buffers (other GPUs' copies of O) stage a
// tile's O in shared memory and send it with one bulk copy per buffer, or to a
// multicast address with multimem stores from the staged tile.
#include "../../include/wave_cuda.h"
#include "backend_env.h"
#include "fa_sm100.h"
#include "fa_common.cuh"
#include "launch_cache.h"
#include "sm100_ptx.cuh"

#include <string>
#include <type_traits>

namespace wave {

void set_last_error(const char *message); // wave_cuda_backend.cu

__device__ int g_fa_decoupled_status[4]; // [0] code, [1] linear block, [2] role, [3] detail

// Optional stage stamps (clock64) of CTA 0, compiled in with -DWAVE_FA_TRACE:
// [role][block][stamp]; role 0 = the issuing threads (0..2 / 4..6 Q*K^T of tile 0 / 1, 8..12 P*V),
// 1 / 2 = row 0 of softmax tile 0 / 1.
#ifdef WAVE_FA_TRACE
__device__ long long g_fad_trace[3][64][16];
#define FAD_STAMP(role, blk, idx)                                                                  \
  do {                                                                                             \
    if (blockIdx.x == 0 && (blk) < 64)                                                             \
      g_fad_trace[role][blk][idx] = clock64();                                                     \
  } while (0)
#else
#define FAD_STAMP(role, blk, idx)                                                                  \
  do {                                                                                             \
  } while (0)
#endif

namespace {

using namespace fa_detail;

constexpr int kBlockM = 128; // rows per Q tile = UMMA M = TMEM lanes
constexpr int kBlockN = 80;  // keys per K/V block = UMMA N of Q*K^T
constexpr int kD = 128;      // head dimension
constexpr int kThreads = 384;
constexpr int kQSub = kBlockM * 64 * 2;  // [128 rows][64 elements], 128-byte swizzled rows
constexpr int kQTile = 2 * kQSub;
constexpr int kKvSub = kBlockN * 64 * 2; // [80 keys][64 elements]
constexpr int kKvTile = 2 * kKvSub;
constexpr int kStages = 3;               // per ring (K and V have one each)
static_assert(kKvSub % 1024 == 0, "a swizzled sub-tile must start on a 1024-byte boundary");
static_assert(kBlockN % 16 == 0 && kBlockN >= 32 && kBlockN <= 128, "UMMA N / K-step granularity");
constexpr int kSmemTiles = 2 * kQTile + 2 * kStages * kKvTile;
constexpr int kSmemBytes = kSmemTiles + 1024 + 256;
// Tensor-memory columns.
constexpr int kTmemCols = 512;
constexpr int kColS = 0;                            // S_t at kColS + t * kBlockN
constexpr int kColP = 2 * kBlockN;                  // P_t at kColP + t * kPStride
constexpr int kPStride = (kBlockN / 2 + 15) / 16 * 16;
constexpr int kColO = 256;                          // O_t at kColO + t * kD
static_assert(kColP + 2 * kPStride <= kColO, "scores and probabilities do not fit beside the accumulators");
constexpr int kDefaultPoly = 2;
constexpr float kRescaleThreshold = 8.0f; // log2 units (wave_flash_attention.py:563-569)
constexpr int kLaunchRegs = 168;
constexpr int kIssueRegs = 72;
constexpr int kSoftmaxRegs = 216;
static_assert((kLaunchRegs - kIssueRegs) * 128 >= (kSoftmaxRegs - kLaunchRegs) * 256,
              "setmaxnreg.inc would wait forever: warpgroup 0 does not release enough registers");
static_assert(kIssueRegs % 8 == 0 && kSoftmaxRegs % 8 == 0, "setmaxnreg takes multiples of 8");
// The variants with further output buffers add a staging area behind everything
// else: one Q tile's worth of 16-bit O (also used as eight 2 KB per-warp slots
// by the paths that store to the further buffers from registers).
constexpr int kStageBytes = kBlockM * kD * 2;
static_assert(kStageBytes >= kExtraStageBytes, "the per-warp slots live in the staging area");
static_assert(kSmemBytes + kStageBytes <= 227 * 1024, "does not fit the shared memory of an SM");

struct FaShared {
  uint64_t item_full[2], item_empty[2]; // work-item hand-off from the Q/K loader to the other roles
  uint64_t q_full, q_empty;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2];  // scores of the tile's next block are in tensor memory
  uint64_t s_free[2];  // the tile's softmax threads have them in registers
  uint64_t p_full[2];  // probabilities are in tensor memory
  uint64_t pv_done[2]; // P*V has run: P may be overwritten, O is at rest
  uint64_t o_free[2];  // the epilogue has read O out
  uint64_t stg_full;   // further outputs: a tile's O is in the staging area (one arrival per warp of the tile)
  uint64_t stg_free;   // ... and has been read out of it again (one arrival per warp of the tile)
  uint32_t tmem_base;
  int abort_flag;
  int item_idx[2];
};
static_assert(sizeof(FaShared) <= 256, "FaShared outgrew its slot");

struct WorkItem {
  int q_blk, bh;
  int n_blocks[2]; // K/V blocks each Q tile visits (0: tile is past the end of Q)
  int n_max;
};
// Items are numbered head-major with the heaviest causal query block first.
__device__ __forceinline__ WorkItem decode_item(int idx, const FaParams &p) {
  WorkItem w;
  const int nq = (p.seq_q + 2 * kBlockM - 1) / (2 * kBlockM);
  w.bh = idx / nq;
  w.q_blk = nq - 1 - idx % nq;
  const int n_kv_blocks = (p.seq_k + kBlockN - 1) / kBlockN;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0 = w.q_blk * 2 * kBlockM + t * kBlockM;
    int n = 0;
    if (q0 < p.seq_q) {
      n = n_kv_blocks;
      if (p.causal) // the tile's last row sees keys up to q0 + 127
        n = min(n, (q0 + kBlockM - 1) / kBlockN + 1);
    }
    w.n_blocks[t] = n;
  }
  w.n_max = max(w.n_blocks[0], w.n_blocks[1]);
  return w;
}

__device__ __noinline__ void fad_report(int code, int role, int detail) {
  if (atomicCAS(&g_fa_decoupled_status[0], 0, code) == 0) {
    g_fa_decoupled_status[1] = static_cast<int>(blockIdx.x);
    g_fa_decoupled_status[2] = role;
    g_fa_decoupled_status[3] = detail;
  }
}

struct RingPos {
  int stage = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void advance() {
    if (++stage == kStages) {
      stage = 0;
      phase ^= 1;
    }
  }
};

// N consecutive 32-bit columns of this warp's 32 lanes into registers / back.
template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t addr, uint32_t (&r)[N]) {
  static_assert(N % 16 == 0, "multiples of 16 columns");
#pragma unroll
  for (int c = 0; c + 32 <= N; c += 32)
    tmem_ld_32x32b_x32(addr + c, *reinterpret_cast<uint32_t(*)[32]>(&r[c]));
  if constexpr (N % 32 == 16)
    tmem_ld_32x32b_x16(addr + (N - 16), *reinterpret_cast<uint32_t(*)[16]>(&r[N - 16]));
}
template <int N> __device__ __forceinline__ void tmem_st_cols(uint32_t addr, const uint32_t (&r)[N]) {
  static_assert(N % 8 == 0, "multiples of 8 columns");
#pragma unroll
  for (int c = 0; c + 32 <= N; c += 32)
    tmem_st_32x32b_x32(addr + c, *reinterpret_cast<const uint32_t(*)[32]>(&r[c]));
  constexpr int kRest = N % 32, kBase = N - kRest;
  if constexpr (kRest >= 16)
    tmem_st_32x32b_x16(addr + kBase, *reinterpret_cast<const uint32_t(*)[16]>(&r[kBase]));
  if constexpr (kRest % 16 == 8)
    tmem_st_32x32b_x8(addr + (N - 8), *reinterpret_cast<const uint32_t(*)[8]>(&r[N - 8]));
}

// kExtra: the epilogue also writes O to the launch's further output buffers
// (FaExtra); compiled out of the ordinary kernels.
template <int kPoly, bool kBf16, bool kExtra>
__global__ void __launch_bounds__(kThreads, 1)
fa_decoupled_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const FaParams p, const __grid_constant__ FaExtra ex) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = tiles;                                   // 2 tiles
  uint8_t *k_smem = tiles + 2 * kQTile;                      // kStages stages
  uint8_t *v_smem = tiles + 2 * kQTile + kStages * kKvTile;  // kStages stages
  FaShared *sh = reinterpret_cast<FaShared *>(tiles + kSmemTiles);
  volatile int *abort_flag = &sh->abort_flag;
  // the variants with further output buffers: 2 KB per softmax warp behind everything else
  uint8_t *extra_stage = tiles + (kSmemBytes - 1024);
  (void)extra_stage;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_items = p.batch_heads * ((p.seq_q + 2 * kBlockM - 1) / (2 * kBlockM));

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->q_empty, 2); // both Q*K^T threads
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_empty[s], 2); // both Q*K^T threads
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->item_full[s], 1);
      mbar_init(&sh->item_empty[s], 11); // three issuing threads, one lane of each softmax warp
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->s_free[s], 4);  // one lane of each softmax warp of the tile
      mbar_init(&sh->p_full[s], 4);
      mbar_init(&sh->pv_done[s], 1);
      mbar_init(&sh->o_free[s], 4);
    }
    mbar_init(&sh->stg_full, 4);
    mbar_init(&sh->stg_free, 4);
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;

  // Descriptor halves: the high half is the same for Q, K (K-major) and V
  // (MN-major): stride 1024 bytes, version 1, 128-byte swizzle.
  constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
  constexpr uint32_t kQTile16 = kQTile >> 4, kQSub16 = kQSub >> 4;
  constexpr uint32_t kKvTile16 = kKvTile >> 4, kKvSub16 = kKvSub >> 4;

  if (warp < 4)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIssueRegs));
  if (warp == 0) {
    // ------------------------------------- work items, Q, K and V loads
    // One thread loads everything in the order of use: K of block 0, then per
    // block j the K of block j+1 (wanted when softmax j starts) and the V of
    // block j (wanted when it ends).  K and V have rings of their own.
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      RingPos kpos, vpos; // carry over from item to item
      auto load_kv = [&](bool is_k, int blk, int bh) -> bool {
        RingPos &pos = is_k ? kpos : vpos;
        uint64_t *full = is_k ? &sh->k_full[pos.stage] : &sh->v_full[pos.stage];
        uint64_t *empty = is_k ? &sh->k_empty[pos.stage] : &sh->v_empty[pos.stage];
        uint8_t *dst = (is_k ? k_smem : v_smem) + pos.stage * kKvTile;
        if (!mbar_wait(empty, pos.phase ^ 1, abort_flag)) {
          fad_report(kStatusWaitTimeout, 0, (is_k ? 10 : 20) + pos.stage);
          return false;
        }
        mbar_arrive_expect_tx(full, kKvTile);
        for (int c = 0; c < 2; ++c)
          tma_load_3d(dst + c * kKvSub, is_k ? &tm_k : &tm_v, full, c * 64, blk * kBlockN, bh);
        pos.advance();
        return true;
      };
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_empty[slot], ((n >> 1) & 1) ^ 1, abort_flag)) {
          fad_report(kStatusWaitTimeout, 0, 1);
          break;
        }
        const int idx = static_cast<int>(atomicAdd(p.ticket, 1u));
        sh->item_idx[slot] = idx;
        mbar_arrive(&sh->item_full[slot]);
        if (idx >= total_items)
          break;
        const WorkItem w = decode_item(idx, p);
        // Q of the previous item may be overwritten once its last Q*K^T has run.
        if (n > 0 && !mbar_wait(&sh->q_empty, (n - 1) & 1, abort_flag)) {
          fad_report(kStatusWaitTimeout, 0, 2);
          break;
        }
        const int q_tiles = (w.n_blocks[0] > 0) + (w.n_blocks[1] > 0);
        mbar_arrive_expect_tx(&sh->q_full, static_cast<uint32_t>(q_tiles * kQTile));
        for (int t = 0; t < 2; ++t)
          if (w.n_blocks[t] > 0)
            for (int c = 0; c < 2; ++c)
              tma_load_3d(q_smem + t * kQTile + c * kQSub, &tm_q, &sh->q_full, c * 64,
                          w.q_blk * 2 * kBlockM + t * kBlockM, w.bh);
        ok = load_kv(true, 0, w.bh);
        for (int j = 0; j < w.n_max && ok; ++j) {
          if (j + 1 < w.n_max)
            ok = load_kv(true, j + 1, w.bh);
          if (ok)
            ok = load_kv(false, j, w.bh);
        }
      }
      if (!ok)
        bounded_delay(1 << 21);
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------------------------ UMMA issue: S = Q K^T
    // One issuing thread per Q tile (warp 1: tile 0, warp 3: tile 1).  Both walk
    // the K ring through every block of the item; a stage is free again when
    // both have arrived on its barrier -- with a commit behind the tile's
    // Q*K^T, or plainly (after the stage has filled, so that the arrival
    // counts for this use of the stage) when the tile does not visit the block.
    if (lane == 0) {
      const int t = warp == 1 ? 0 : 1;
      const uint32_t idesc_s = umma_idesc_f16(kBlockM, kBlockN, p.is_bf16, 0, 0);
      const uint32_t q_lo = (((smem_u32(q_smem) & 0x3FFFFu) >> 4) | (1u << 16)) + static_cast<uint32_t>(t) * kQTile16;
      const uint32_t k_lo = ((smem_u32(k_smem) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t d = tmem_base + static_cast<uint32_t>(kColS + t * kBlockN);
      bool ok = true;
      RingPos pos;
      uint32_t qk_n = 0; // batches issued on this tile (s_free phases)
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_full[slot], (n >> 1) & 1, abort_flag)) {
          fad_report(kStatusWaitTimeout, 1, 3);
          break;
        }
        const int idx = sh->item_idx[slot];
        mbar_arrive(&sh->item_empty[slot]);
        if (idx >= total_items)
          break;
        const WorkItem w = decode_item(idx, p);
        const int nb = w.n_blocks[t];
        if (!mbar_wait(&sh->q_full, n & 1, abort_flag)) {
          fad_report(kStatusWaitTimeout, 1, 1);
          break;
        }
        for (int j = 0; j < w.n_max; ++j) {
          if (!mbar_wait(&sh->k_full[pos.stage], pos.phase, abort_flag)) {
            fad_report(kStatusWaitTimeout, 1, 10 + pos.stage);
            ok = false;
            break;
          }
          if (j < nb) {
            if (n == 0)
              FAD_STAMP(0, j, 0 + 4 * t);
            // The tile's score columns must be in its softmax threads' registers.
            if (qk_n > 0 && !mbar_wait(&sh->s_free[t], (qk_n - 1) & 1, abort_flag)) {
              fad_report(kStatusWaitTimeout, 1, 60 + t);
              ok = false;
              break;
            }
            ++qk_n;
            tc_fence_after_sync();
            if (n == 0)
              FAD_STAMP(0, j, 1 + 4 * t);
            const uint32_t b = k_lo + static_cast<uint32_t>(pos.stage) * kKvTile16;
            umma_ss_halves<0>(d, q_lo, b, kDescHi, idesc_s);
#pragma unroll
            for (int i = 1; i < 8; ++i) // two 64-element swizzle chunks x four K steps of 16
              umma_ss_halves<1>(d, q_lo + static_cast<uint32_t>((i >> 2) * kQSub16 + (i & 3) * 2),
                                b + static_cast<uint32_t>((i >> 2) * kKvSub16 + (i & 3) * 2), kDescHi, idesc_s);
            umma_commit(&sh->s_full[t]);
            umma_commit(&sh->k_empty[pos.stage]);
            if (n == 0)
              FAD_STAMP(0, j, 2 + 4 * t);
          } else {
            mbar_arrive(&sh->k_empty[pos.stage]);
          }
          pos.advance();
        }
        if (!ok)
          break;
        // Q may be overwritten once both tiles' last Q*K^T have run.
        if (nb > 0)
          umma_commit(&sh->q_empty);
        else
          mbar_arrive(&sh->q_empty);
      }
    }
  } else if (warp == 2) {
    // ----------------------------------------------- UMMA issue: O += P V
    if (lane == 0) {
      const uint32_t idesc_o = umma_idesc_f16(kBlockM, kD, p.is_bf16, 0, 1); // V is MN-major
      const uint32_t v_lo = ((smem_u32(v_smem) & 0x3FFFFu) >> 4) | ((kKvSub16 & 0x3FFFu) << 16);
      bool ok = true;
      RingPos pos;
      uint32_t p_n[2] = {0, 0};        // P hand-offs waited for, per tile
      uint32_t tile_items[2] = {0, 0}; // items in which the tile had work (o_free phases)
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_full[slot], (n >> 1) & 1, abort_flag)) {
          fad_report(kStatusWaitTimeout, 5, 3);
          break;
        }
        const int idx = sh->item_idx[slot];
        mbar_arrive(&sh->item_empty[slot]);
        if (idx >= total_items)
          break;
        const WorkItem w = decode_item(idx, p);
        for (int j = 0; j < w.n_max && ok; ++j) {
          if (!mbar_wait(&sh->v_full[pos.stage], pos.phase, abort_flag)) {
            fad_report(kStatusWaitTimeout, 5, 20 + pos.stage);
            ok = false;
            break;
          }
          for (int t = 0; t < 2; ++t) {
            if (j >= w.n_blocks[t])
              continue;
            if (n == 0)
              FAD_STAMP(0, j, 8 + 2 * t);
            if (!mbar_wait(&sh->p_full[t], p_n[t] & 1, abort_flag)) {
              fad_report(kStatusWaitTimeout, 5, 40 + t);
              ok = false;
              break;
            }
            ++p_n[t];
            // The first P*V of an item overwrites O_t: the previous item's
            // epilogue must have read it out.
            if (j == 0 && tile_items[t] > 0 && !mbar_wait(&sh->o_free[t], (tile_items[t] - 1) & 1, abort_flag)) {
              fad_report(kStatusWaitTimeout, 5, 45 + t);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (n == 0)
              FAD_STAMP(0, j, 9 + 2 * t);
            // K = kBlockN keys in steps of 16; P from tensor memory (8 packed
            // columns per step), V rows are keys (128 bytes each), 16 keys = 2048 bytes.
            const uint32_t d = tmem_base + static_cast<uint32_t>(kColO + t * kD);
            const uint32_t a = tmem_base + static_cast<uint32_t>(kColP + t * kPStride);
            const uint32_t b = v_lo + static_cast<uint32_t>(pos.stage) * kKvTile16;
            umma_ts_halves<-1>(d, a, b, kDescHi, idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
            for (int kk = 1; kk < kBlockN / 16; ++kk)
              umma_ts_halves<1>(d, a + static_cast<uint32_t>(kk * 8), b + static_cast<uint32_t>(kk * (2048 >> 4)), kDescHi,
                                idesc_o);
            umma_commit(&sh->pv_done[t]);
            if (j + 1 == w.n_blocks[t])
              ++tile_items[t];
          }
          if (!ok)
            break;
          umma_commit(&sh->v_empty[pos.stage]);
          pos.advance();
          if (n == 0)
            FAD_STAMP(0, j, 12);
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
    const uint32_t s_addr = tmem_base + lane_base + static_cast<uint32_t>(kColS + t * kBlockN);
    const uint32_t p_addr = tmem_base + lane_base + static_cast<uint32_t>(kColP + t * kPStride);
    const uint32_t o_addr = tmem_base + lane_base + static_cast<uint32_t>(kColO + t * kD);
    constexpr bool bf16 = kBf16;
    uint32_t blk_n = 0; // blocks this tile has taken so far (s_full / pv_done phases)
    bool ok = true;
    // Further outputs in the 16-bit type through plain addresses: a tile's O is
    // staged in shared memory and sent to every further buffer with bulk copies
    // (the tile's rows are one contiguous piece of O), so that no softmax thread
    // waits for stores that cross NVLink.  The two tiles take turns on the one
    // staging area, in the order tile 0, tile 1 of each item.
    const bool bulk_out = kExtra && !p.out_f32; // plain targets: bulk copies; a multicast target: multimem.st from the staged tile
    uint32_t stage_uses = 0; // uses of the staging area before this item (stg_full / stg_free phases)

    for (uint32_t item_n = 0; ok; ++item_n) {
    const int slot = item_n & 1;
    if (!mbar_wait(&sh->item_full[slot], (item_n >> 1) & 1, abort_flag)) {
      if (lane == 0)
        fad_report(kStatusWaitTimeout, 2 + t, 59);
      break;
    }
    const int idx = sh->item_idx[slot];
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&sh->item_empty[slot]);
    if (idx >= total_items)
      break;
    const WorkItem w = decode_item(idx, p);
    const int bh = w.bh;
    const int q_row = w.q_blk * 2 * kBlockM + t * kBlockM + row;
    const int nb = w.n_blocks[t];
    float m_used = p.fixed_ref ? p.ref_log2 / c : -INFINITY;
    float l = 0.0f; // running sum of unrounded probabilities

    for (int j = 0; j < nb; ++j, ++blk_n) {
      if (row == 0 && item_n == 0)
        FAD_STAMP(1 + t, j, 0);
      if (!mbar_wait(&sh->s_full[t], blk_n & 1, abort_flag)) {
        if (lane == 0)
          fad_report(kStatusWaitTimeout, 2 + t, 60);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // Tile 1 holds back once per item, when its first scores are there, so
      // that the two tiles' softmax phases interleave (one in its exponentials
      // while the other finds its maximum or hands P over) instead of meeting
      // on the special-function unit.
      if (t == 1 && j == 0 && p.stagger > 0)
        bounded_delay(p.stagger);
      if (row == 0 && item_n == 0)
        FAD_STAMP(1 + t, j, 1);
      uint32_t s[kBlockN];
      tmem_ld_cols<kBlockN>(s_addr, s);
      tmem_ld_wait();
      // The scores are in registers: the tensor core may write the next block's.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&sh->s_free[t]);
      if (row == 0 && item_n == 0)
        FAD_STAMP(1 + t, j, 2);

      const int key0 = j * kBlockN;
      const bool need_mask = (p.causal && key0 + kBlockN - 1 > q_row - row) || (key0 + kBlockN > p.seq_k);
      if (need_mask) {
        const int limit = p.causal ? min(q_row, p.seq_k - 1) : p.seq_k - 1; // last visible key
#pragma unroll
        for (int i = 0; i < kBlockN; ++i)
          if (key0 + i > limit)
            s[i] = 0xFF800000u; // -inf
      }
      if (!p.fixed_ref) {
        // Sixteen independent chains of three-input maxima (the instruction has a long latency).
        static_assert(kBlockN % 16 == 0 && (kBlockN / 16) % 2 == 1, "the chains below take 16 + 32k columns");
        float mx[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          mx[i] = __uint_as_float(s[i]);
#pragma unroll
        for (int base = 16; base + 32 <= kBlockN; base += 32)
#pragma unroll
          for (int i = 0; i < 16; ++i)
            mx[i] = max3(mx[i], __uint_as_float(s[base + i]), __uint_as_float(s[base + 16 + i]));
#pragma unroll
        for (int k = 0; k < 5; ++k)
          mx[k] = max3(mx[k], mx[5 + 2 * k], mx[6 + 2 * k]);
        mx[0] = max3(mx[0], mx[1], mx[2]);
        mx[3] = max3(mx[3], mx[4], mx[15]);
        const float m_new = max3(m_used, mx[0], mx[3]);
        // Lazy rescale: only when some row of this warp moved its maximum by more
        // than 2^8; otherwise keep the stale maximum (exact after the final divide).
        const bool need = (m_new - m_used) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
          const float factor = fast_exp2((m_used - m_new) * c);
          l *= factor;
          if (j > 0) {
            // O must be at rest: P*V of the previous block has to have run.
            if (!mbar_wait(&sh->pv_done[t], (blk_n - 1) & 1, abort_flag)) {
              if (lane == 0)
                fad_report(kStatusWaitTimeout, 2 + t, 61);
              ok = false;
              break;
            }
            tc_fence_after_sync();
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
      if (row == 0 && item_n == 0)
        FAD_STAMP(1 + t, j, 3);
      const float neg_mc = -m_used * c;
      const float2 c2 = make_float2(c, c), nm2 = make_float2(neg_mc, neg_mc);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
      uint32_t pk[kBlockN / 2];
#pragma unroll
      for (int i = 0; i < kBlockN / 2; ++i) {
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
      if (row == 0 && item_n == 0)
        FAD_STAMP(1 + t, j, 4);
      // The tile's P columns are free once P*V of the block before has read them.
      if (blk_n > 0 && !mbar_wait(&sh->pv_done[t], (blk_n - 1) & 1, abort_flag)) {
        if (lane == 0)
          fad_report(kStatusWaitTimeout, 2 + t, 62);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      tmem_st_cols<kBlockN / 2>(p_addr, pk);
      tmem_st_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&sh->p_full[t]);
      if (row == 0 && item_n == 0)
        FAD_STAMP(1 + t, j, 5);
    }

    if (ok && nb > 0) {
      // The item's last P*V.
      if (!mbar_wait(&sh->pv_done[t], (blk_n - 1) & 1, abort_flag)) {
        if (lane == 0)
          fad_report(kStatusWaitTimeout, 2 + t, 70);
        ok = false;
      } else {
        tc_fence_after_sync();
        const float inv = 1.0f / l;
        const bool live = q_row < p.seq_q;
        const int esize = p.out_f32 ? 4 : 2;
        const uint32_t my_use = stage_uses + ((t == 1 && w.n_blocks[0] > 0) ? 1u : 0u);
        if (bulk_out && my_use > 0 && !mbar_wait(&sh->stg_free, (my_use - 1) & 1, abort_flag)) {
          if (lane == 0)
            fad_report(kStatusWaitTimeout, 2 + t, 71);
          ok = false;
          break;
        }
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
                if (cc + 8 * v < p.head_dim)
                  dst[v] = make_uint4(wv[4 * v], wv[4 * v + 1], wv[4 * v + 2], wv[4 * v + 3]);
            }
            if constexpr (kExtra) { // 16-bit O: into the staging area, row by row as it lies in memory
              uint4 *dst = reinterpret_cast<uint4 *>(extra_stage + static_cast<size_t>(row) * p.head_dim * 2 + cc * 2);
#pragma unroll
              for (int v = 0; v < 4; ++v)
                if (cc + 8 * v < p.head_dim)
                  dst[v] = make_uint4(wv[4 * v], wv[4 * v + 1], wv[4 * v + 2], wv[4 * v + 3]);
            }
          }
        }
        if (p.lse && live)
          p.lse[static_cast<size_t>(bh) * p.seq_q + q_row] = m_used * p.scale + logf(l);
        // O_t has been read out: the next item's first P*V may overwrite it.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&sh->o_free[t]);
        if (bulk_out) {
          fence_proxy_async_smem(); // the staged rows, before the bulk copies read them
          __syncwarp();
          if (lane == 0)
            mbar_arrive(&sh->stg_full);
          const int q0 = q_row - row;
          const int rows_live = min(kBlockM, p.seq_q - q0);
          const uint32_t bytes = static_cast<uint32_t>(rows_live) * static_cast<uint32_t>(p.head_dim) * 2u;
          const size_t off = (static_cast<size_t>(bh) * p.seq_q + q0) * static_cast<size_t>(p.head_dim) * 2;
          if (ex.multimem) {
            // One multimem.st per 16 bytes, the tile's 128 threads side by side
            // (a warp writes 512 contiguous bytes per instruction); the switch
            // delivers each to every GPU's copy.  Every warp needs all rows staged.
            if (!mbar_wait(&sh->stg_full, my_use & 1, abort_flag)) {
              if (lane == 0)
                fad_report(kStatusWaitTimeout, 2 + t, 72);
              ok = false;
            } else {
#pragma unroll 4
              for (uint32_t b = static_cast<uint32_t>(row) * 16u; b < bytes; b += kBlockM * 16u)
                multimem_st_16B(static_cast<uint8_t *>(ex.o[0]) + off + b, *reinterpret_cast<const uint4 *>(extra_stage + b));
              __syncwarp();
              if (lane == 0)
                mbar_arrive(&sh->stg_free);
            }
          } else if (quarter == 0) {
            // The tile's first warp waits for all four; one of its threads sends
            // the tile and waits only until the copies have READ the staging area.
            if (!mbar_wait(&sh->stg_full, my_use & 1, abort_flag)) {
              if (lane == 0)
                fad_report(kStatusWaitTimeout, 2 + t, 72);
              ok = false;
            } else if (lane == 0) {
#pragma unroll 1
              for (int x = 0; x < ex.n; ++x)
                bulk_store_global(static_cast<uint8_t *>(ex.o[x]) + off, extra_stage, bytes);
              tma_store_commit();
              tma_store_wait_read<0>();
              mbar_arrive(&sh->stg_free);
            }
          } else if (lane == 0) {
            mbar_arrive(&sh->stg_free); // this warp does not read the staging area
          }
          __syncwarp();
        }
      }
    }
    stage_uses += (w.n_blocks[0] > 0) + (w.n_blocks[1] > 0);
    } // work items
    if (bulk_out && !ex.multimem && quarter == 0 && lane == 0)
      tma_store_wait<0>(); // this thread's copies have landed before the kernel ends
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

} // namespace

cudaError_t fa_decoupled_read_status(int out[4], bool clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fa_decoupled_status, sizeof(int) * 4);
  if (err == cudaSuccess && clear) {
    int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(g_fa_decoupled_status, zero, sizeof(zero));
  }
  return err;
}

#ifdef WAVE_FA_TRACE
extern "C" int wave_cuda_fad_trace_read(long long *out, int clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fad_trace, sizeof(long long) * 3 * 64 * 16);
  if (err == cudaSuccess && clear) {
    static long long zero[3 * 64 * 16];
    err = cudaMemcpyToSymbol(g_fad_trace, zero, sizeof(zero));
  }
  return err == cudaSuccess ? 0 : -3;
}
#endif

// `tq`: boxes of 64 elements x 128 rows over Q; K and V get maps of their own
// here (64 elements x 80 keys).
namespace {

// Cycles tile 1 holds back at each item's first block.  Left alone the two
// tiles' softmax phases fall into step and meet on the special-function unit;
// an offset lets one tile's exponentials run beside the other's latency-bound
// parts for a while (the phases drift back together within some tens of
// blocks).  Measured sustained, kernels taking turns, 0 -> 400 cycles: B=16 H=32
// S=4096 non-causal 1008..1021 -> 1083..1097 TFLOP/s, causal 967..986 -> 973..984;
// B=2 H=64 S=8192 causal 1036..1054 -> 1062..1089; B=8 H=32 S=2048 causal
// 784..807 -> 775..790 (short items: the wait costs more than it gains);
// 800 and 1200 cycles give less everywhere.
int default_stagger(const FaParams &p) { return (!p.causal || p.seq_k >= 8192) ? 400 : 0; }

} // namespace

int launch_flash_attention_decoupled(const FaParams &p, const FaExtra &extra, const CUtensorMap &tq, const void *K,
                                     const void *V, int poly, int stagger_cycles, int sm_count, cudaStream_t stream) {
  CUtensorMap tk, tv;
  {
    const uint64_t hd = static_cast<uint64_t>(p.head_dim), row_bytes = hd * 2;
    const uint64_t dims[3] = {hd, static_cast<uint64_t>(p.seq_k), static_cast<uint64_t>(p.batch_heads)};
    const uint64_t strides[2] = {row_bytes, row_bytes * static_cast<uint64_t>(p.seq_k)};
    const uint32_t box[3] = {64, static_cast<uint32_t>(kBlockN), 1};
    int rc = make_tensor_map_16bit(&tk, p.is_bf16, K, 3, dims, strides, box);
    if (rc != WAVE_OK)
      return rc;
    rc = make_tensor_map_16bit(&tv, p.is_bf16, V, 3, dims, strides, box);
    if (rc != WAVE_OK)
      return rc;
  }
  const long long total_items =
      static_cast<long long>(p.batch_heads) * ((p.seq_q + 2 * kBlockM - 1) / (2 * kBlockM));
  const unsigned grid = static_cast<unsigned>(total_items < sm_count ? total_items : sm_count);
  cudaError_t err = cudaSuccess;
  bool unsafe_budget = false;
  FaParams params = p;
  params.stagger = stagger_cycles >= 0 ? stagger_cycles : default_stagger(p);
  auto launch = [&](auto kernel) {
    // The setmaxnreg arithmetic in the kernel assumes the register count the
    // compiler actually gave it; refuse to launch rather than risk a grow
    // request that can never be satisfied.
    KernelInfo info;
    const int smem_bytes = kSmemBytes + (extra.n > 0 ? kStageBytes : 0);
    err = prepare_kernel(kernel, smem_bytes, &info);
    if (err != cudaSuccess)
      return;
    if ((info.num_regs - kIssueRegs) * 128 < (kSoftmaxRegs - info.num_regs) * 256 || info.num_regs * kThreads > 65536) {
      unsafe_budget = true;
      return;
    }
    kernel<<<grid, kThreads, smem_bytes, stream>>>(tq, tk, tv, params, extra);
    err = cudaGetLastError();
  };
  auto dispatch = [&](auto bf16_tag) {
    constexpr bool B = decltype(bf16_tag)::value;
    if (extra.n > 0) { // further output buffers: the kernel variant whose epilogue writes them (default polynomial share)
      launch(fa_decoupled_kernel<kDefaultPoly, B, true>);
      return;
    }
    switch (poly) {
    case 0: launch(fa_decoupled_kernel<0, B, false>); break;
    case 1: launch(fa_decoupled_kernel<1, B, false>); break;
    case 3: launch(fa_decoupled_kernel<3, B, false>); break;
    case 4: launch(fa_decoupled_kernel<4, B, false>); break;
    default: launch(fa_decoupled_kernel<kDefaultPoly, B, false>); break;
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

} // namespace wave
