// Flash-attention forward for sm_100a, "streaming" variant: one 128-row Q tile
// per CTA with the score and probability buffers double-buffered in tensor
// memory, so that the tensor core never waits for the softmax of the block it
// has just produced.  Same operator and numerics as fa_sm100.cu (the stand-in
// for the reference's `flash_attention_bf16_gfx950`,
// python/mlir/dialects/wave_flash_attention.py:452-728, 1034-1095): exp2 with
// scale*log2(e) folded into the exponent (:596-600), f32 row sums of the
// unrounded probabilities with 16-bit probabilities feeding P*V (:706-722),
// lazy accumulator rescale with threshold 8 in log2 units (:557-583).
//
// Structure (persistent CTAs, one per SM, 384 threads; a work item is 128 query
// rows of one head, drawn from a ticket counter):
//   warp 0        TMA producer: Q tiles (two slots, by item parity) and K blocks
//                 of 128 keys through a two-stage ring; hands out the work items
//   warp 3        TMA producer: V blocks through a two-stage ring
//   warp 1        UMMA issuer for S(g) = Q K(g)^T (one thread), running ahead of
//                 the softmax by up to two blocks, across item boundaries
//   warp 2        UMMA issuer for O += P(g) V(g) (one thread)
//   warps 4..7    softmax of the even blocks, one thread per query row
//   warps 8..11   softmax of the odd blocks (a row's two threads hand its
//                 running maximum from block to block through shared memory)
// TMEM (512 columns): S[0] | S[1] (128 f32 columns each) | P[0] | P[1] (64
// columns of packed 16-bit pairs each) | O (128).  Because P has columns of its
// own, Q*K^T of block g+1 does not have to wait for P*V of block g, and the
// softmax of block g+1 can start as soon as that of block g has ended.  The
// commit after P*V of block g tells the loader that V's stage is free, the
// softmax warps that P[g&1] may be written again, and the rare accumulator
// rescale of block g+1 that O is at rest.  No load uses cluster multicast.
#include "../../include/wave_cuda.h"
#include "fa_common.cuh"
#include "fa_sm100.h"
#include "launch_cache.h"
#include "sm100_ptx.cuh"

#include <atomic>
#include <cstdlib>
#include <type_traits>

namespace wave {

void set_last_error(const char *message); // wave_cuda_backend.cu
__device__ int g_fa_stream_status[4]; // [0] code, [1] block, [2] role (20..), [3] detail

#ifdef WAVE_FA_TRACE
__device__ long long g_fas_trace[3][64][16];
#ifdef WAVE_FA_TRACE_CLOCK_ONLY // only the start/end clock probe
#define FAS_STAMP(role, blk, idx)
#else
#define FAS_STAMP(role, blk, idx)                                                                  \
  do {                                                                                             \
    if (blockIdx.x == 0 && (blk) < 64) {                                                           \
      unsigned int fa_stamp_clk;                                                                   \
      asm volatile("mov.u32 %0, %%clock;" : "=r"(fa_stamp_clk));                                   \
      fa_trace_smem[((role)*64 + (blk)) * 16 + (idx)] = fa_stamp_clk;                              \
    }                                                                                              \
  } while (0)
#endif
#define FAS_TRACE_SMEM_BYTES (3 * 64 * 16 * 4)
#else
#define FAS_STAMP(role, blk, idx)                                                                  \
  do {                                                                                             \
  } while (0)
#define FAS_TRACE_SMEM_BYTES 0
#endif

namespace {

using namespace fa_detail;

constexpr int kBlockM = 128; // rows of the Q tile = UMMA M = TMEM lanes
constexpr int kBlockN = 128; // keys per K/V block
constexpr int kD = 128;      // head dimension
constexpr int kThreads = 384;
constexpr int kSubTile = 128 * 64 * 2; // [128 rows][64 elements], 128-byte swizzled rows
constexpr int kTile = 2 * kSubTile;    // 128 x 128 16-bit elements
constexpr int kSmemTiles = 2 * kTile /*Q slots*/ + 2 * kTile /*K ring*/ + 2 * kTile /*V ring*/;
constexpr int kSharedStateBytes = 2560;
constexpr int kSmemBytes = kSmemTiles + 1024 + kSharedStateBytes + FAS_TRACE_SMEM_BYTES;
constexpr int kTmemCols = 512;
constexpr uint32_t kTmemS = 0, kTmemP = 256, kTmemO = 384;
constexpr float kRescaleThreshold = 8.0f; // log2 units (wave_flash_attention.py:563-569)
constexpr int kStatusWaitTimeout = 1;
constexpr uint32_t kTraceItem = 3; // which of a CTA's items the optional stage stamps record
// setmaxnreg budget, as in fa_sm100.cu: warpgroup 0 gives registers up, the two
// softmax warpgroups hold a 128-column score row per thread.
constexpr int kLaunchRegs = 168;
constexpr int kIssueRegs = 72;
constexpr int kSoftmaxRegs = 216;
static_assert((kLaunchRegs - kIssueRegs) * 128 >= (kSoftmaxRegs - kLaunchRegs) * 256,
              "setmaxnreg.inc would wait forever: warpgroup 0 does not release enough registers");

struct StreamShared {
  uint64_t item_full[2], item_empty[2]; // work-item hand-off from the loader to the other roles
  uint64_t q_full[2], q_empty[2];       // Q slots, by item parity
  uint64_t k_full[2], v_full[2], v_empty[2];
  uint64_t s_full[2], s_free[2], p_full[2];
  uint64_t o_full, o_free, l_full;
  uint32_t tmem_base;
  int abort_flag;
  int item_idx[2];
  float l_part[2][kBlockM]; // partial row sums of the two threads of a row, for the epilogue
  float row_max[kBlockM];   // per row: the maximum in use after the blocks decided so far
  uint32_t row_seq[kBlockM]; // per row: how many blocks have been decided (global block count)
};
static_assert(sizeof(StreamShared) <= kSharedStateBytes, "shared state does not fit its slot");

// One work item = 128 query rows of one (batch, head).  Items are numbered
// head-major with the heaviest causal query tile of a head first, so that CTAs
// running at the same time share a head's K/V through L2.
struct StreamItem {
  int q_blk, bh, n_blocks;
};
__device__ __forceinline__ StreamItem decode_item(int idx, const FaParams &p) {
  StreamItem w;
  const int nq = (p.seq_q + kBlockM - 1) / kBlockM;
  w.bh = idx / nq;
  w.q_blk = nq - 1 - idx % nq;
  const int n_kv_blocks = (p.seq_k + kBlockN - 1) / kBlockN;
  w.n_blocks = p.causal ? min(n_kv_blocks, w.q_blk + 1) : n_kv_blocks;
  return w;
}

__device__ __noinline__ void fas_report(int code, int role, int detail) {
  if (atomicCAS(&g_fa_stream_status[0], 0, code) == 0) {
    g_fa_stream_status[1] = static_cast<int>(blockIdx.x);
    g_fa_stream_status[2] = 20 + role; // roles 20.. : the streaming kernel
    g_fa_stream_status[3] = detail;
  }
}

// kExtra: the epilogue also writes O to the launch's further output buffers
// (FaExtra); compiled out of the ordinary kernels.
template <int kPoly, bool kBf16, bool kExtra>
__global__ void __launch_bounds__(kThreads, 1)
fa_stream_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const FaParams p, const __grid_constant__ FaExtra ex) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = tiles;             // 2 slots
  uint8_t *k_smem = tiles + 2 * kTile; // 2 stages
  uint8_t *v_smem = tiles + 4 * kTile; // 2 stages
  StreamShared *sh = reinterpret_cast<StreamShared *>(tiles + kSmemTiles);
  volatile int *abort_flag = &sh->abort_flag;
  // the variants with further output buffers: 2 KB per softmax warp behind everything else
  uint8_t *extra_stage = tiles + (kSmemBytes - 1024);
  (void)extra_stage;
#ifdef WAVE_FA_TRACE
  volatile unsigned int *fa_trace_smem =
      reinterpret_cast<volatile unsigned int *>(tiles + kSmemTiles + kSharedStateBytes);
  for (int i = threadIdx.x; i < 3 * 64 * 16; i += kThreads)
    fa_trace_smem[i] = 0;
#endif

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_items = p.batch_heads * ((p.seq_q + kBlockM - 1) / kBlockM);

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->item_full[s], 1);
      mbar_init(&sh->item_empty[s], 11); // the V loader, the two UMMA threads and one lane of each softmax warp
      mbar_init(&sh->q_full[s], 1);
      mbar_init(&sh->q_empty[s], 1);
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->v_empty[s], 1);
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->s_free[s], 4); // one lane of each warp of the buffer's warpgroup, once its scores are in registers
      mbar_init(&sh->p_full[s], 4); // the same, once its rows of P are stored
    }
    mbar_init(&sh->o_full, 1);
    mbar_init(&sh->o_free, 8); // one lane of each softmax warp, once its part of O has been read out
    mbar_init(&sh->l_full, 8);
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (threadIdx.x < kBlockM) {
    sh->row_max[threadIdx.x] = -INFINITY;
    sh->row_seq[threadIdx.x] = 0;
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = sh->tmem_base;
#ifdef WAVE_FA_TRACE
  if (threadIdx.x == 64 && blockIdx.x == 0) { // SM clock against wall time over the CTA's life
    unsigned long long ns;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
    g_fas_trace[1][63][0] = clock64();
    g_fas_trace[1][63][1] = static_cast<long long>(ns);
  }
#endif

  // A "previous phase" parity: waiting for the phase before the one block g (or
  // item n) completes passes at once on a barrier nobody has used yet.
  auto prev_parity = [](uint32_t count) { return ((count >> 1) & 1u) ^ 1u; };
  auto this_parity = [](uint32_t count) { return (count >> 1) & 1u; };

  if (warp < 4)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIssueRegs));
  if (warp == 0) {
    // ---------------------------------------------------------------- loads
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      bool ok = true;
      uint32_t g = 0; // K/V blocks requested so far
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_empty[slot], prev_parity(n), abort_flag)) {
          fas_report(kStatusWaitTimeout, 0, 1);
          break;
        }
        const int idx = static_cast<int>(atomicAdd(p.ticket, 1u));
        sh->item_idx[slot] = idx;
        mbar_arrive(&sh->item_full[slot]);
        if (idx >= total_items)
          break;
        const StreamItem w = decode_item(idx, p);
        // The slot's previous Q (item n-2) has been used by its last Q*K^T.
        if (!mbar_wait(&sh->q_empty[slot], prev_parity(n), abort_flag)) {
          fas_report(kStatusWaitTimeout, 0, 2);
          break;
        }
        mbar_arrive_expect_tx(&sh->q_full[slot], kTile);
        for (int c = 0; c < 2; ++c)
          tma_load_3d(q_smem + slot * kTile + c * kSubTile, &tm_q, &sh->q_full[slot], c * 64, w.q_blk * kBlockM,
                      w.bh);
        for (int j = 0; j < w.n_blocks && ok; ++j, ++g) {
          const int s = g & 1;
          // K's stage is free once Q*K^T of block g-2 has run: that is "S(g-2) is ready".
          if (!mbar_wait(&sh->s_full[s], prev_parity(g), abort_flag)) {
            fas_report(kStatusWaitTimeout, 0, 10 + s);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&sh->k_full[s], kTile);
          for (int c = 0; c < 2; ++c)
            tma_load_3d(k_smem + s * kTile + c * kSubTile, &tm_k, &sh->k_full[s], c * 64, j * kBlockN, w.bh);
        }
      }
      if (!ok)
        bounded_delay(1 << 21);
    }
  } else if (warp == 3) {
    // -------------------------------------------------------------- V loads
    // A thread of its own: Q*K^T runs about two blocks ahead of P*V, so K's
    // stages come free well before V's; one thread loading K(g), V(g), K(g+1)
    // in turn would hold every K back behind a V that has to wait.
    if (lane == 0) {
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      uint32_t g = 0;
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_full[slot], this_parity(n), abort_flag)) {
          fas_report(kStatusWaitTimeout, 0, 4);
          break;
        }
        const int idx = sh->item_idx[slot];
        mbar_arrive(&sh->item_empty[slot]);
        if (idx >= total_items)
          break;
        const StreamItem w = decode_item(idx, p);
        for (int j = 0; j < w.n_blocks && ok; ++j, ++g) {
          const int s = g & 1;
          // V's stage is free once P*V of block g-2 has run.
          if (!mbar_wait(&sh->v_empty[s], prev_parity(g), abort_flag)) {
            fas_report(kStatusWaitTimeout, 0, 20 + s);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&sh->v_full[s], kTile);
          for (int c = 0; c < 2; ++c)
            tma_load_3d(v_smem + s * kTile + c * kSubTile, &tm_v, &sh->v_full[s], c * 64, j * kBlockN, w.bh);
        }
      }
      if (!ok)
        bounded_delay(1 << 21);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------- UMMA issue: Q*K^T
    // Issuing one 128 x 128 x 16 instruction occupies the issuing thread for
    // about as long as the tensor core works on it (~70 cycles measured, with
    // an empty queue too), so whatever else that thread does (barrier looks,
    // commits, loop control) is time the tensor core stands idle.  The two kinds
    // of product therefore have a thread each (this warp and the next): while
    // one thread is between two batches the other keeps the tensor core fed.
    // This thread runs ahead of the softmax by up to two blocks, across item
    // boundaries (the next item's Q sits in the other Q slot).
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_f16(kBlockM, kBlockN, p.is_bf16, 0, 0);
      // Descriptor halves (see umma_desc_kmajor_sw128).
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kTile16 = kTile >> 4, kSub16 = kSubTile >> 4;
      const uint32_t q_lo = ((smem_u32(q_smem) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t k_lo = ((smem_u32(k_smem) & 0x3FFFFu) >> 4) | (1u << 16);
      uint32_t g = 0; // global block counter
      for (uint32_t item_n = 0;; ++item_n) {
        const int slot = item_n & 1;
        if (!mbar_wait(&sh->item_full[slot], this_parity(item_n), abort_flag)) {
          fas_report(kStatusWaitTimeout, 1, 3);
          break;
        }
        const int idx = sh->item_idx[slot];
        mbar_arrive(&sh->item_empty[slot]);
        if (idx >= total_items)
          break;
        const int nb = decode_item(idx, p).n_blocks;
        if (!mbar_wait(&sh->q_full[slot], this_parity(item_n), abort_flag)) {
          fas_report(kStatusWaitTimeout, 1, 1);
          break;
        }
        const uint32_t qa = q_lo + static_cast<uint32_t>(slot) * kTile16;
        bool ok = true;
        for (int j = 0; j < nb; ++j, ++g) {
          const uint32_t b = g & 1;
          if (item_n == kTraceItem)
            FAS_STAMP(0, j, 0);
          // K(g) has landed; S[b] (scores of block g-2) has been read into registers.
          if (!mbar_wait(&sh->k_full[b], this_parity(g), abort_flag) ||
              !mbar_wait(&sh->s_free[b], prev_parity(g), abort_flag)) {
            fas_report(kStatusWaitTimeout, 1, 10 + b);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (item_n == kTraceItem)
            FAS_STAMP(0, j, 1);
          const uint32_t d = tmem_base + kTmemS + b * kBlockN;
          const uint32_t kb = k_lo + b * kTile16;
          umma_ss_halves<0>(d, qa, kb, kDescHi, idesc_s);
#pragma unroll
          for (int i = 1; i < 8; ++i) {
            const uint32_t off = static_cast<uint32_t>((i >> 2) * kSub16 + (i & 3) * 2);
            umma_ss_halves<1>(d, qa + off, kb + off, kDescHi, idesc_s);
          }
          umma_commit(&sh->s_full[b]);
          if (item_n == kTraceItem)
            FAS_STAMP(0, j, 2);
        }
        if (!ok)
          break;
        umma_commit(&sh->q_empty[slot]); // the item's last Q*K^T has been issued
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------ UMMA issue: P*V
    if (lane == 0) {
      const uint32_t idesc_o = umma_idesc_f16(kBlockM, kD, p.is_bf16, 0, 1); // V is MN-major
      // Descriptor halves (see umma_desc_mnmajor_sw128).
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kTile16 = kTile >> 4, kSub16 = kSubTile >> 4;
      const uint32_t v_lo = ((smem_u32(v_smem) & 0x3FFFFu) >> 4) | ((kSub16 & 0x3FFFu) << 16);
      const uint32_t d = tmem_base + kTmemO;
      uint32_t g = 0; // global block counter
      for (uint32_t item_n = 0;; ++item_n) {
        const int slot = item_n & 1;
        if (!mbar_wait(&sh->item_full[slot], this_parity(item_n), abort_flag)) {
          fas_report(kStatusWaitTimeout, 2, 3);
          break;
        }
        const int idx = sh->item_idx[slot];
        mbar_arrive(&sh->item_empty[slot]);
        if (idx >= total_items)
          break;
        const int nb = decode_item(idx, p).n_blocks;
        bool ok = true;
        for (int j = 0; j < nb; ++j, ++g) {
          const uint32_t b = g & 1;
          if (item_n == kTraceItem)
            FAS_STAMP(0, j, 4);
          // V(g) has landed and the block's softmax warpgroup has stored P(g).
          // The first P*V of an item overwrites O: both warpgroups must have
          // read the previous item's O out (only one of them stores this P).
          if (!mbar_wait(&sh->v_full[b], this_parity(g), abort_flag) ||
              !mbar_wait(&sh->p_full[b], this_parity(g), abort_flag) ||
              (j == 0 && item_n > 0 && !mbar_wait(&sh->o_free, (item_n - 1) & 1, abort_flag))) {
            fas_report(kStatusWaitTimeout, 2, 40 + b);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (item_n == kTraceItem)
            FAS_STAMP(0, j, 5);
          // O += P[b] V(g): eight steps of 16 keys; P from TMEM (8 packed columns per step)
          const uint32_t a = tmem_base + kTmemP + b * (kBlockN / 2);
          const uint32_t vb = v_lo + b * kTile16;
          umma_ts_halves<-1>(d, a, vb, kDescHi, idesc_o, j > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 8; ++kk)
            umma_ts_halves<1>(d, a + static_cast<uint32_t>(kk * 8), vb + static_cast<uint32_t>(kk * (2048 >> 4)),
                              kDescHi, idesc_o);
          umma_commit(&sh->v_empty[b]); // V's stage and P[b] may be written again
          if (item_n == kTraceItem)
            FAS_STAMP(0, j, 6);
        }
        if (!ok)
          break;
        umma_commit(&sh->o_full);
      }
    }
  } else if (warp >= 4) {
    // --------------------------------------------------------------- softmax
    // Two warpgroups: warps 4..7 take the even blocks (buffers S[0], P[0]),
    // warps 8..11 the odd ones, one thread per query row each, so a row has two
    // threads that work on alternate blocks, half a period apart: while one is
    // in its exponentials (special-function unit) the other loads and scans
    // the next block (ALU).  The running maximum of a row is handed from block
    // to block through shared memory (`row_max`, `row_seq`): the thread of block
    // g may only decide about a rescale once the decision of block g-1 is
    // published, which the other thread does right after scanning its block.
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int quarter = warp & 3;
    const int wg = (warp - 4) >> 2; // parity of the blocks this thread takes; also its half of O in the epilogue
    const int row = quarter * 32 + lane;
    const float c = p.scale_log2e;
    // Fixed reference in score units (ref_log2 is in units of the exponent), or none.
    const float m_fixed = p.fixed_ref ? p.ref_log2 / c : -INFINITY;
    constexpr bool bf16 = kBf16;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + kTmemS + static_cast<uint32_t>(wg * kBlockN);
    const uint32_t p_addr = tmem_base + lane_base + kTmemP + static_cast<uint32_t>(wg * (kBlockN / 2));
    const uint32_t o_addr = tmem_base + lane_base + kTmemO;
    volatile float *row_max = sh->row_max;
    volatile uint32_t *row_seq = sh->row_seq;
    uint32_t g = 0; // global block counter (all blocks, both parities)
    bool ok = true;

    // Waits until the decisions of all blocks before `blk` are published and
    // returns the row's maximum in use after them.
    auto max_before = [&](uint32_t blk, float &m_out) -> bool {
      if (static_cast<int>(row_seq[row] - blk) < 0) {
        const long long start = clock64();
        while (static_cast<int>(row_seq[row] - blk) < 0) {
          if (*abort_flag)
            return false;
          if (clock64() - start > kWaitLimitCycles) {
            *abort_flag = 1;
            return false;
          }
        }
      }
      __threadfence_block();
      m_out = row_max[row];
      return true;
    };

    for (uint32_t item_n = 0; ok; ++item_n) {
      const int slot = item_n & 1;
      if (!mbar_wait(&sh->item_full[slot], this_parity(item_n), abort_flag)) {
        if (lane == 0)
          fas_report(kStatusWaitTimeout, 3 + wg, 59);
        break;
      }
      const int idx = sh->item_idx[slot];
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&sh->item_empty[slot]);
      if (idx >= total_items)
        break;
      const StreamItem w = decode_item(idx, p);
      const int q_row = w.q_blk * kBlockM + row;
      const int nb = w.n_blocks;
      float m_seen = m_fixed; // the row maximum this thread's sum l is relative to
      float l = 0.0f;           // sum of the unrounded probabilities of this thread's blocks

      for (int j = 0; j < nb; ++j, ++g) {
        if ((g & 1u) != static_cast<uint32_t>(wg))
          continue;
        if (row == 0 && item_n == kTraceItem)
          FAS_STAMP(1 + wg, j, 0);
        if (p.fixed_ref && p.stagger > 0 && j == 1) {
          // Hold the item's second block back once, so that the two warpgroups'
          // exponential phases do not coincide for the rest of the item.
          uint32_t t0, t1;
          asm volatile("mov.u32 %0, %%clock;" : "=r"(t0));
          do {
            asm volatile("mov.u32 %0, %%clock;" : "=r"(t1));
          } while (t1 - t0 < static_cast<uint32_t>(p.stagger));
        }
        if (!mbar_wait(&sh->s_full[wg], this_parity(g), abort_flag)) {
          if (lane == 0)
            fas_report(kStatusWaitTimeout, 3 + wg, 60);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        if (row == 0 && item_n == kTraceItem)
          FAS_STAMP(1 + wg, j, 1);
        uint32_t s[128];
        tmem_ld_32x32b_x32(s_addr + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld_32x32b_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_ld_32x32b_x32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
        tmem_ld_32x32b_x32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
        tmem_ld_wait();
        // The scores are in registers: S[wg] may take the scores of block g+2.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&sh->s_free[wg]);
        if (row == 0 && item_n == kTraceItem)
          FAS_STAMP(1 + wg, j, 2);

        const int key0 = j * kBlockN;
        const bool need_mask = (p.causal && key0 + kBlockN - 1 > q_row - row) || (key0 + kBlockN > p.seq_k);
        if (need_mask) {
          const int limit = p.causal ? min(q_row, p.seq_k - 1) : p.seq_k - 1; // last visible key
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (key0 + i > limit)
              s[i] = 0xFF800000u; // -inf
        }
        // With a fixed reference (the caller's bound on |q| and |k|) there is no
        // maximum to find, hand over or rescale by.
        float m_used = m_fixed;
        if (!p.fixed_ref) {
          float mx[8];
#pragma unroll
          for (int k = 0; k < 8; ++k)
            mx[k] = fmaxf(__uint_as_float(s[2 * k]), __uint_as_float(s[2 * k + 1]));
#pragma unroll
          for (int i = 16; i < 128; i += 16)
#pragma unroll
            for (int k = 0; k < 8; ++k)
              mx[k] = max3(mx[k], __uint_as_float(s[i + 2 * k]), __uint_as_float(s[i + 2 * k + 1]));
          const float m_blk = max3(max3(mx[0], mx[1], mx[2]), max3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]));
          // The maximum in use after the blocks before this one (none for the
          // first block of an item).
          float m_prev = -INFINITY;
          if (!max_before(g, m_prev)) {
            if (lane == 0)
              fas_report(kStatusWaitTimeout, 3 + wg, 63);
            ok = false;
            break;
          }
          if (j == 0)
            m_prev = -INFINITY;
          // The other thread of the row may have raised the maximum since this
          // thread last added to its sum.
          if (m_prev != m_seen) {
            l *= fast_exp2((m_seen - m_prev) * c); // m_seen = -inf only with l = 0
            if (m_seen == -INFINITY)
              l = 0.0f;
          }
          m_used = m_prev;
          const float m_new = fmaxf(m_prev, m_blk);
          // Lazy rescale: only when some row of this warp moved its maximum by more
          // than 2^8; otherwise keep the stale maximum (exact after the final divide).
          const bool need = (m_new - m_prev) * c > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            const float factor = fast_exp2((m_prev - m_new) * c);
            l *= factor;
            if (j > 0) {
              // O must be at rest: P*V of block g-1 has ended (its commit says so)
              // and P*V of block g waits for this block's P.
              if (!mbar_wait(&sh->v_empty[(g - 1) & 1], this_parity(g - 1), abort_flag)) {
                if (lane == 0)
                  fas_report(kStatusWaitTimeout, 3 + wg, 61);
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
        m_seen = m_used;
        if (!p.fixed_ref) {
          // Publish the decision: the other thread of the row may now decide about block g+1.
          row_max[row] = m_used;
          __threadfence_block();
          row_seq[row] = g + 1;
        }
        if (row == 0 && item_n == kTraceItem)
          FAS_STAMP(1 + wg, j, 3);
        const float neg_mc = -m_used * c;
        const float2 c2 = make_float2(c, c), nm2 = make_float2(neg_mc, neg_mc);
        float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float2 v =
              __ffma2_rn(make_float2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), c2, nm2);
          float2 pr;
          if (pair_uses_poly<kPoly>(i))
            pr = exp2_poly2(v);
          else
            pr = make_float2(fast_exp2(v.x), fast_exp2(v.y));
          if (i & 1)
            lb = __fadd2_rn(lb, pr);
          else
            la = __fadd2_rn(la, pr);
          pk[i] = pack2(pr.x, pr.y, bf16);
        }
        l += (la.x + la.y) + (lb.x + lb.y);
        if (row == 0 && item_n == kTraceItem)
          FAS_STAMP(1 + wg, j, 4);
        // P[wg] must be free: P*V of block g-2 has ended (normally long ago).
        if (!mbar_wait(&sh->v_empty[wg], prev_parity(g), abort_flag)) {
          if (lane == 0)
            fas_report(kStatusWaitTimeout, 3 + wg, 62);
          ok = false;
          break;
        }
        tmem_st_32x32b_x32(p_addr + 0, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
        tmem_st_32x32b_x32(p_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
        tmem_st_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&sh->p_full[wg]);
        if (row == 0 && item_n == kTraceItem)
          FAS_STAMP(1 + wg, j, 5);
      }
      if (!ok)
        break;

      // ---- epilogue: O / l, this thread's 64 columns of its row.  g now counts
      // all blocks of the item: bring this thread's sum to the final maximum.
      float m_final = m_fixed;
      if (!p.fixed_ref && !max_before(g, m_final)) {
        if (lane == 0)
          fas_report(kStatusWaitTimeout, 3 + wg, 64);
        break;
      }
      if (m_final != m_seen)
        l = (m_seen == -INFINITY) ? 0.0f : l * fast_exp2((m_seen - m_final) * c);
      if (!mbar_wait(&sh->o_full, item_n & 1, abort_flag)) {
        if (lane == 0)
          fas_report(kStatusWaitTimeout, 3 + wg, 70);
        break;
      }
      tc_fence_after_sync();
      sh->l_part[wg][row] = l;
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&sh->l_full);
      if (!mbar_wait(&sh->l_full, item_n & 1, abort_flag)) {
        if (lane == 0)
          fas_report(kStatusWaitTimeout, 3 + wg, 71);
        break;
      }
      const float l_row = l + sh->l_part[1 - wg][row];
      const float inv = 1.0f / l_row;
      const bool live = q_row < p.seq_q;
      // Head dimensions below 128 ran zero-padded (TMA fills the missing columns
      // of Q, K and V with zeros); only the first head_dim columns of O exist in
      // memory.  Output is the I/O type, or f32 on request.
      const int esize = p.out_f32 ? 4 : 2;
      uint8_t *out_row = static_cast<uint8_t *>(p.O) +
                         (static_cast<size_t>(w.bh) * p.seq_q + static_cast<size_t>(live ? q_row : 0)) *
                             static_cast<size_t>(p.head_dim) * esize;
#pragma unroll 1
      for (int cc = 64 * wg; cc < 64 * wg + 64 && cc < p.head_dim; cc += 32) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(o_addr + static_cast<uint32_t>(cc), o);
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
          uint32_t wd[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            wd[i] = pack2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv, bf16);
          if (live) {
            uint4 *dst = reinterpret_cast<uint4 *>(out_row + cc * 2);
#pragma unroll
            for (int v = 0; v < 4; ++v)
              if (cc + 8 * v < p.head_dim) {
                dst[v] = make_uint4(wd[4 * v], wd[4 * v + 1], wd[4 * v + 2], wd[4 * v + 3]);
              }
          }
          if constexpr (kExtra) {
            const int first_row = q_row - lane; // a warp's 32 rows are consecutive
            store_extra_chunk_16bit(ex, extra_stage + (warp - 4) * 2048, lane, wd,
                                    (static_cast<size_t>(w.bh) * p.seq_q + first_row) * p.head_dim * 2 + static_cast<size_t>(cc) * 2,
                                    static_cast<size_t>(p.head_dim) * 2, min(32, max(0, p.seq_q - first_row)),
                                    min(64, (p.head_dim - cc) * 2));
          }
        }
      }
      if (p.lse && live && wg == 0)
        p.lse[static_cast<size_t>(w.bh) * p.seq_q + q_row] = m_final * p.scale + logf(l_row);
      // O has been read out: the next item's first P*V may overwrite it.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&sh->o_free);
    } // work items
  }

  tc_fence_before_sync();
  __syncthreads();
#ifdef WAVE_FA_TRACE
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < 3 * 64 * 16; i += kThreads)
      if (i / 16 != 64 + 63) // [1][63][*] holds the clock probe
        (&g_fas_trace[0][0][0])[i] = fa_trace_smem[i];
  }
  if (threadIdx.x == 64 && blockIdx.x == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
    g_fas_trace[1][63][2] = clock64();
    g_fas_trace[1][63][3] = static_cast<long long>(ns);
  }
#endif
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

} // namespace

cudaError_t fa_stream_read_status(int out[4], bool clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fa_stream_status, sizeof(int) * 4);
  if (err == cudaSuccess && clear) {
    int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(g_fa_stream_status, zero, sizeof(zero));
  }
  return err;
}

#ifdef WAVE_FA_TRACE
extern "C" int wave_cuda_fas_trace_read(long long *out, int clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fas_trace, sizeof(long long) * 3 * 64 * 16);
  if (err == cudaSuccess && clear) {
    static long long zero[3 * 64 * 16];
    err = cudaMemcpyToSymbol(g_fas_trace, zero, sizeof(zero));
  }
  return err == cudaSuccess ? 0 : -3;
}
#endif

int launch_flash_attention_stream(const FaParams &p, const FaExtra &extra, const CUtensorMap &tq, const CUtensorMap &tk,
                                  const CUtensorMap &tv, int poly, int sm_count, cudaStream_t stream) {
  const long long total_items = static_cast<long long>(p.batch_heads) * ((p.seq_q + kBlockM - 1) / kBlockM);
  const unsigned grid = static_cast<unsigned>(total_items < sm_count ? total_items : sm_count);
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
      launch(fa_stream_kernel<2, B, true>);
      return;
    }
    // A quarter of the exponentials on the FMA pipe is this kernel's measured
    // best (causal B=2 H=64 S=8192, sustained: 893 -> 1049 TFLOP/s); `poly` < 0 asks for it.
    switch (poly) {
    case 0: launch(fa_stream_kernel<0, B, false>); break;
    case 1: launch(fa_stream_kernel<1, B, false>); break;
    case 3: launch(fa_stream_kernel<3, B, false>); break;
    case 4: launch(fa_stream_kernel<4, B, false>); break;
    default: launch(fa_stream_kernel<2, B, false>); break;
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
