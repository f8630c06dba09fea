// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T [+causal]) V,
// (B, H, S, D=128) bf16/f16 in and out, f32 online-softmax statistics.  This is
// the B200 stand-in for the kernel the reference generates as
// `flash_attention_bf16_gfx950` (python/mlir/dialects/wave_flash_attention.py:
// 452-728, 1034-1095, 1685-1731): BLOCK_M 256 per workgroup, exp2 with
// scale*log2(e) folded into the exponent (:596-600), f32 row sums of the
// unrounded probabilities with 16-bit probabilities feeding P*V (:706-722),
// and the lazy accumulator rescale with threshold 8 in log2 units (:557-583).
//
// Structure (persistent CTAs, one per SM, 384 threads; a work item is 256 query
// rows of one head, drawn from a ticket counter so that the causal triangle
// balances itself and the prologue/epilogue of one item overlaps the next):
//   warp 0        TMA producer: two 128-row Q tiles once, then K and V blocks
//                 of 128 keys through two-stage rings (128B-swizzled smem)
//   warp 1        UMMA issuer (one thread): S_t = Q_t K^T (both operands from
//                 shared memory) and O_t += P_t V (P from tensor memory, V from
//                 shared memory as an MN-major operand), t = 0, 1
//   warps 4..7    softmax for Q tile 0: one thread per query row
//   warps 8..11   softmax for Q tile 1
// The two Q tiles ping-pong: while one tile's rows are in the exponentials the
// tensor core works on the other tile.  TMEM: S_0 | S_1 | O_0 | O_1, 128 f32
// columns each; P_t overwrites the first 64 columns of S_t as packed 16-bit
// pairs.  Tensor-core operations of one tile are issued in program order
// (PV_t(j) before S_t(j+1)), which is what makes the S/P aliasing safe.
// No load uses cluster multicast.  The causal mask (key <= query) is an
// extension: the reference's Wave kernel is non-causal.
#include "../../include/wave_cuda.h"
#include "backend_env.h"
#include "fa_sm100.h"
#include "fa_common.cuh"
#include "launch_cache.h"
#include "sm100_ptx.cuh"

#include <mutex>
#include <string>
#include <cstdlib>
#include <cstring>
#include <type_traits>

namespace wave {

void set_last_error(const char *message); // wave_cuda_backend.cu

__device__ int g_fa_status[4]; // [0] code, [1] linear block, [2] role, [3] detail

// Work-item ticket counters: one per launch in flight (a ring guarded by
// events, see ticket_acquire), cleared by the launcher on the launch's stream.
constexpr unsigned kTicketSlots = 64;
__device__ unsigned int g_fa_tickets[kTicketSlots];

// Optional stage stamps (clock64) for one CTA, compiled in with -DWAVE_FA_TRACE:
// [role][block][stamp].  Role 0 = UMMA thread, 1 = softmax tile 0 (row 0),
// 2 = softmax tile 1 (row 0).
#ifdef WAVE_FA_TRACE
__device__ long long g_fa_trace[3][64][16];
#ifdef WAVE_FA_TRACE_CLOCK_ONLY // only the start/end clock probe
#define FA_STAMP(role, blk, idx)
#else
// Stamps go to shared memory (a 32-bit clock read and one shared store) and
// are copied out when the CTA ends.
#define FA_STAMP(role, blk, idx)                                                                   \
  do {                                                                                             \
    if (blockIdx.x == 0 && (blk) < 64) {                                                           \
      unsigned int fa_stamp_clk;                                                                   \
      asm volatile("mov.u32 %0, %%clock;" : "=r"(fa_stamp_clk));                                   \
      fa_trace_smem[((role)*64 + (blk)) * 16 + (idx)] = fa_stamp_clk;                              \
    }                                                                                              \
  } while (0)
#endif
#define FA_TRACE_SMEM_BYTES (3 * 64 * 16 * 4)
#else
#define FA_STAMP(role, blk, idx)                                                                   \
  do {                                                                                             \
  } while (0)
#define FA_TRACE_SMEM_BYTES 0
#endif

namespace {

using namespace fa_detail;

constexpr int kBlockM = 128; // rows per Q tile = UMMA M = TMEM lanes
constexpr int kBlockN = 128; // keys per K/V block
constexpr int kD = 128;      // head dimension
constexpr int kThreads = 384;            // warpgroup 0: loader + UMMA warps; warpgroups 1, 2: softmax
constexpr int kSubTile = 128 * 64 * 2;  // [128 rows][64 elements], 128-byte swizzled rows
constexpr int kTile = 2 * kSubTile;     // 128 x 128 16-bit elements
constexpr int kSmemTiles = 2 * kTile /*Q*/ + 2 * kTile /*K ring*/ + 2 * kTile /*V ring*/;
constexpr int kSmemBytes = kSmemTiles + 1024 + 256 + FA_TRACE_SMEM_BYTES;
constexpr int kTmemCols = 512;
// Of every 8 column pairs, how many evaluate 2^x with exp2_poly2 instead of the
// special-function unit.  Measured on B200 (causal, B=16 H=32 S=4096): 0 -> 1014,
// 1 -> 1011, 2 -> 966, 3 -> 958, 4 -> 975 TFLOP/s: the kernel is paced by the
// S/P hand-offs between the softmax warps and the tensor core, not by the
// special-function unit, so the default keeps every exponential on it.
constexpr int kDefaultPoly = 0;
constexpr int kFixedRefStagger = 900;
constexpr float kRescaleThreshold = 8.0f;
// setmaxnreg budget.  The kernel starts with kLaunchRegs per thread (12 warps,
// one CTA per SM); warpgroup 0 shrinks to kIssueRegs and the two softmax
// warpgroups grow to kSoftmaxRegs.  The grow request blocks until the registers
// exist, so what warpgroup 0 releases must cover what the other two ask for.
constexpr int kLaunchRegs = 168;
constexpr int kIssueRegs = 72;
constexpr int kSoftmaxRegs = 216;
static_assert((kLaunchRegs - kIssueRegs) * 128 >= (kSoftmaxRegs - kLaunchRegs) * 256,
              "setmaxnreg.inc would wait forever: warpgroup 0 does not release enough registers");
static_assert(kIssueRegs % 8 == 0 && kSoftmaxRegs % 8 == 0, "setmaxnreg takes multiples of 8"); // log2 units (wave_flash_attention.py:563-569)

struct FaShared {
  uint64_t item_full[2], item_empty[2]; // work-item hand-off from the loader to the other roles
  uint64_t q_full, q_empty;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], p_full[2], o_full[2], o_free[2];
  uint32_t tmem_base;
  int abort_flag;
  int item_idx[2];
};

// One work item = 256 query rows (two tiles) of one (batch, head).  Items are
// numbered head-major with the heaviest causal query block of a head first, so
// that CTAs running at the same time share a head's K/V through L2.
struct WorkItem {
  int q_blk, bh;
  int n_blocks[2]; // K/V blocks each Q tile visits (0: tile is past the end of Q)
  int n_max;
};
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
      if (p.causal)
        n = min(n, q0 / kBlockN + 1);
    }
    w.n_blocks[t] = n;
  }
  w.n_max = max(w.n_blocks[0], w.n_blocks[1]);
  return w;
}

// Out of line: the report sits on many cold paths and would otherwise bloat the hot loops.
__device__ __noinline__ void fa_report(int code, int role, int detail) {
  if (atomicCAS(&g_fa_status[0], 0, code) == 0) {
    g_fa_status[1] = static_cast<int>(blockIdx.y * gridDim.x + blockIdx.x);
    g_fa_status[2] = role;
    g_fa_status[3] = detail;
  }
}

// kExtra: the epilogue also writes O to the launch's further output buffers
// (FaExtra); compiled out of the ordinary kernels.
template <int kPoly, bool kBf16, bool kExtra>
__global__ void __launch_bounds__(kThreads, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const FaParams p, const __grid_constant__ FaExtra ex) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *q_smem = tiles;              // 2 tiles
  uint8_t *k_smem = tiles + 2 * kTile;  // 2 stages
  uint8_t *v_smem = tiles + 4 * kTile;  // 2 stages
  FaShared *sh = reinterpret_cast<FaShared *>(tiles + kSmemTiles);
  volatile int *abort_flag = &sh->abort_flag;
  // the variants with further output buffers: 2 KB per softmax warp behind everything else
  uint8_t *extra_stage = tiles + (kSmemBytes - 1024);
  (void)extra_stage;
#ifdef WAVE_FA_TRACE
  volatile unsigned int *fa_trace_smem = reinterpret_cast<volatile unsigned int *>(tiles + kSmemTiles + 256);
  for (int i = threadIdx.x; i < 3 * 64 * 16; i += kThreads)
    fa_trace_smem[i] = 0;
#endif

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_items = p.batch_heads * ((p.seq_q + 2 * kBlockM - 1) / (2 * kBlockM));

  if (threadIdx.x == 0) {
    mbar_init(&sh->q_full, 1);
    mbar_init(&sh->q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->item_full[s], 1);
      mbar_init(&sh->item_empty[s], 9); // the UMMA thread and one lane of each softmax warp
      mbar_init(&sh->k_full[s], 1);
      mbar_init(&sh->k_empty[s], 1);
      mbar_init(&sh->v_full[s], 1);
      mbar_init(&sh->v_empty[s], 1);
      mbar_init(&sh->s_full[s], 1);
      mbar_init(&sh->p_full[s], kBlockM); // every softmax thread of the tile arrives
      mbar_init(&sh->o_full[s], 1);
      mbar_init(&sh->o_free[s], 4);       // one lane of each softmax warp of the tile
    }
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
#ifdef WAVE_FA_TRACE
  if (threadIdx.x == 64 && blockIdx.x == 0) { // SM clock against wall time over the CTA's life
    unsigned long long ns;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
    g_fa_trace[1][63][0] = clock64();
    g_fa_trace[1][63][1] = static_cast<long long>(ns);
  }
#endif

  // Register budget (setmaxnreg must be the first thing each warpgroup does on
  // its own path): warpgroup 0 (loader, UMMA issuer, two idle warps) gives
  // registers up, the softmax warpgroups hold a 128-column score row per thread.
  if (warp < 4)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIssueRegs));
  if (warp == 0) {
    // ---------------------------------------------------------------- loads
    // The loader also hands out work: it draws the next item from a global
    // ticket counter (CTAs are persistent, one per SM, so the draw balances
    // the causal triangle by itself) and publishes it to the other roles.
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      uint32_t kv_n = 0; // K/V blocks loaded so far: ring stage and phase carry over from item to item
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_empty[slot], ((n >> 1) & 1) ^ 1, abort_flag)) {
          fa_report(kStatusWaitTimeout, 0, 1);
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
          fa_report(kStatusWaitTimeout, 0, 2);
          break;
        }
        const int q_tiles = (w.n_blocks[0] > 0) + (w.n_blocks[1] > 0);
        mbar_arrive_expect_tx(&sh->q_full, static_cast<uint32_t>(q_tiles * kTile));
        for (int t = 0; t < 2; ++t)
          if (w.n_blocks[t] > 0)
            for (int c = 0; c < 2; ++c)
              tma_load_3d(q_smem + t * kTile + c * kSubTile, &tm_q, &sh->q_full, c * 64,
                          w.q_blk * 2 * kBlockM + t * kBlockM, w.bh);
        for (int j = 0; j < w.n_max && ok; ++j, ++kv_n) {
          const int s = kv_n & 1;
          const uint32_t ph = (kv_n >> 1) & 1;
          if (!mbar_wait(&sh->k_empty[s], ph ^ 1, abort_flag)) {
            fa_report(kStatusWaitTimeout, 0, 10 + s);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&sh->k_full[s], kTile);
          for (int c = 0; c < 2; ++c)
            tma_load_3d(k_smem + s * kTile + c * kSubTile, &tm_k, &sh->k_full[s], c * 64, j * kBlockN, w.bh);
          if (!mbar_wait(&sh->v_empty[s], ph ^ 1, abort_flag)) {
            fa_report(kStatusWaitTimeout, 0, 20 + s);
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
    // ------------------------------------------------------------ UMMA issue
    // One thread feeds the tensor core.  It can queue only about two
    // instructions (128 cycles of work at 128 x 128 x 16), so every cycle it
    // spends between two issues beyond that leaves the tensor core idle: the
    // descriptors are stepped with one 32-bit add per operand, and the common
    // case (both tiles have a P*V for this block and a Q*K^T for the next) runs
    // in a loop of its own without the bookkeeping of the ragged cases.
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_f16(kBlockM, kBlockN, p.is_bf16, 0, 0);
      const uint32_t idesc_o = umma_idesc_f16(kBlockM, kD, p.is_bf16, 0, 1); // V is MN-major
      // Descriptor halves (see umma_desc_kmajor_sw128 / umma_desc_mnmajor_sw128):
      // the high half is the same for Q, K (K-major) and V (MN-major): stride
      // 1024 bytes, version 1, 128-byte swizzle.
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
      constexpr uint32_t kTile16 = kTile >> 4, kSub16 = kSubTile >> 4;
      const uint32_t q_lo = ((smem_u32(q_smem) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t k_lo = ((smem_u32(k_smem) & 0x3FFFFu) >> 4) | (1u << 16);
      const uint32_t v_lo = ((smem_u32(v_smem) & 0x3FFFFu) >> 4) | ((kSub16 & 0x3FFFu) << 16);
      bool ok = true;

      // S_t = Q_t K_j^T : K = head dim, two 64-element swizzle chunks x four UMMA K steps
      auto issue_s = [&](int t, int stage) {
        const uint32_t d = tmem_base + static_cast<uint32_t>(t * kBlockN);
        const uint32_t a = q_lo + static_cast<uint32_t>(t) * kTile16;
        const uint32_t b = k_lo + static_cast<uint32_t>(stage) * kTile16;
        umma_ss_halves<0>(d, a, b, kDescHi, idesc_s);
#pragma unroll
        for (int i = 1; i < 8; ++i) {
          const uint32_t off = static_cast<uint32_t>((i >> 2) * kSub16 + (i & 3) * 2);
          umma_ss_halves<1>(d, a + off, b + off, kDescHi, idesc_s);
        }
        umma_commit(&sh->s_full[t]);
      };
      // O_t += P_t V_j : K = 128 keys in eight steps of 16; P from TMEM (8 packed
      // columns per step), V rows are keys (128 bytes each), 16 keys = 2048 bytes.
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t d = tmem_base + static_cast<uint32_t>(2 * kBlockN + t * kD);
        const uint32_t a = tmem_base + static_cast<uint32_t>(t * kBlockN);
        const uint32_t b = v_lo + static_cast<uint32_t>(stage) * kTile16;
        umma_ts_halves<-1>(d, a, b, kDescHi, idesc_o, accumulate ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < 8; ++kk)
          umma_ts_halves<1>(d, a + static_cast<uint32_t>(kk * 8), b + static_cast<uint32_t>(kk * (2048 >> 4)), kDescHi,
                            idesc_o);
      };

      // Running counts that carry barrier phases from item to item.
      uint32_t kv_n = 0;              // K/V blocks consumed so far
      uint32_t p_n[2] = {0, 0};       // P hand-offs waited for, per tile
      uint32_t tile_items[2] = {0, 0}; // items in which the tile had work (o_full / o_free phases)
      for (uint32_t n = 0; ok; ++n) {
        const int slot = n & 1;
        if (!mbar_wait(&sh->item_full[slot], (n >> 1) & 1, abort_flag)) {
          fa_report(kStatusWaitTimeout, 1, 3);
          break;
        }
        const int idx = sh->item_idx[slot];
        mbar_arrive(&sh->item_empty[slot]);
        if (idx >= total_items)
          break;
        const WorkItem w = decode_item(idx, p);
        const int n_max = w.n_max, nb0 = w.n_blocks[0], nb1 = w.n_blocks[1];
        if (!mbar_wait(&sh->q_full, n & 1, abort_flag)) {
          fa_report(kStatusWaitTimeout, 1, 1);
          break;
        }
        {
          const int s0 = kv_n & 1;
          if (!mbar_wait(&sh->k_full[s0], (kv_n >> 1) & 1, abort_flag)) {
            fa_report(kStatusWaitTimeout, 1, 2);
            break;
          }
          tc_fence_after_sync();
          if (nb0 > 0)
            issue_s(0, s0);
          if (nb1 > 0)
            issue_s(1, s0);
          umma_commit(&sh->k_empty[s0]);
          if (n_max == 1)
            umma_commit(&sh->q_empty); // no further Q*K^T in this item
        }
        int j = 0;
        // ---- common case: both tiles have P*V(j) and Q*K^T(j+1)
        const int n_fast = min(nb0, nb1) - 1;
        for (; j < n_fast; ++j, ++kv_n) {
          const int s = kv_n & 1, s_next = s ^ 1;
          const uint32_t ph = (kv_n >> 1) & 1, ph_next = ((kv_n + 1) >> 1) & 1;
          if (n == 0)
            FA_STAMP(0, j, 9);
          if (!mbar_wait(&sh->v_full[s], ph, abort_flag)) {
            fa_report(kStatusWaitTimeout, 1, 30 + s);
            ok = false;
            break;
          }
          // K of the next block was requested a whole block ago; looking at
          // its barrier here, ahead of the wait for P, keeps that look out of
          // the tile's softmax -> P*V -> Q*K^T -> softmax chain.
          if (!mbar_wait(&sh->k_full[s_next], ph_next, abort_flag)) {
            fa_report(kStatusWaitTimeout, 1, 50 + s_next);
            ok = false;
            break;
          }
          if (n == 0)
            FA_STAMP(0, j, 0);
          if (!mbar_wait(&sh->p_full[0], p_n[0] & 1, abort_flag)) {
            fa_report(kStatusWaitTimeout, 1, 40);
            ok = false;
            break;
          }
          ++p_n[0];
          if (n == 0)
            FA_STAMP(0, j, 1);
          // The first P*V of an item overwrites O_t: the previous item's
          // epilogue must have read it out.
          if (j == 0 && tile_items[0] > 0 && !mbar_wait(&sh->o_free[0], (tile_items[0] - 1) & 1, abort_flag)) {
            fa_report(kStatusWaitTimeout, 1, 45);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          issue_pv(0, s, j > 0);
          if (n == 0)
            FA_STAMP(0, j, 3);
          issue_s(0, s_next);
          if (n == 0)
            FA_STAMP(0, j, 2);
          if (!mbar_wait(&sh->p_full[1], p_n[1] & 1, abort_flag)) {
            fa_report(kStatusWaitTimeout, 1, 41);
            ok = false;
            break;
          }
          ++p_n[1];
          if (n == 0)
            FA_STAMP(0, j, 5);
          if (j == 0 && tile_items[1] > 0 && !mbar_wait(&sh->o_free[1], (tile_items[1] - 1) & 1, abort_flag)) {
            fa_report(kStatusWaitTimeout, 1, 46);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          issue_pv(1, s, j > 0);
          if (n == 0)
            FA_STAMP(0, j, 7);
          issue_s(1, s_next);
          if (n == 0)
            FA_STAMP(0, j, 6);
          umma_commit(&sh->v_empty[s]);
          umma_commit(&sh->k_empty[s_next]);
          if (j + 2 == n_max)
            umma_commit(&sh->q_empty); // the last Q*K^T of the item has been issued
          if (n == 0)
            FA_STAMP(0, j, 8);
        }
        // ---- ragged tail: a tile without work, or the last block(s) of the item
        for (; j < n_max && ok; ++j, ++kv_n) {
          const int s = kv_n & 1;
          const uint32_t ph = (kv_n >> 1) & 1;
          const int s_next = (kv_n + 1) & 1;
          const uint32_t ph_next = ((kv_n + 1) >> 1) & 1;
          bool have_v = false, have_k_next = false;
          for (int t = 0; t < 2 && ok; ++t) {
            if (j >= w.n_blocks[t])
              continue;
            if (!have_v) {
              if (!mbar_wait(&sh->v_full[s], ph, abort_flag)) {
                fa_report(kStatusWaitTimeout, 1, 30 + s);
                ok = false;
                break;
              }
              have_v = true;
            }
            if (!mbar_wait(&sh->p_full[t], p_n[t] & 1, abort_flag)) {
              fa_report(kStatusWaitTimeout, 1, 40 + t);
              ok = false;
              break;
            }
            ++p_n[t];
            if (j == 0 && tile_items[t] > 0 && !mbar_wait(&sh->o_free[t], (tile_items[t] - 1) & 1, abort_flag)) {
              fa_report(kStatusWaitTimeout, 1, 45 + t);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(t, s, j > 0);
            if (j + 1 < w.n_blocks[t]) {
              if (!have_k_next) {
                if (!mbar_wait(&sh->k_full[s_next], ph_next, abort_flag)) {
                  fa_report(kStatusWaitTimeout, 1, 50 + s_next);
                  ok = false;
                  break;
                }
                tc_fence_after_sync();
                have_k_next = true;
              }
              issue_s(t, s_next);
            } else {
              umma_commit(&sh->o_full[t]);
              ++tile_items[t];
            }
          }
          if (!ok)
            break;
          umma_commit(&sh->v_empty[s]);
          if (have_k_next)
            umma_commit(&sh->k_empty[s_next]);
          if (j + 2 == n_max)
            umma_commit(&sh->q_empty); // the last Q*K^T of the item has been issued
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
    constexpr bool bf16 = kBf16;
    uint32_t s_n = 0;        // score blocks consumed so far by this tile (s_full phase)
    uint32_t tile_items = 0; // items in which this tile had work (o_full phase)
    bool ok = true;

    for (uint32_t item_n = 0; ok; ++item_n) {
    const int slot = item_n & 1;
    if (!mbar_wait(&sh->item_full[slot], (item_n >> 1) & 1, abort_flag)) {
      if (lane == 0)
        fa_report(kStatusWaitTimeout, 2 + t, 59);
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
    // Maximum the exponentials are taken against (raw score units): the running
    // row maximum, or with a fixed reference the caller's bound for the whole item.
    float m_used = p.fixed_ref ? p.ref_log2 / c : -INFINITY;
    float l = 0.0f; // running sum of unrounded probabilities

    for (int j = 0; j < nb; ++j) {
      if (row == 0 && item_n == 0)
        FA_STAMP(1 + t, j, 0);
      if (!mbar_wait(&sh->s_full[t], s_n & 1, abort_flag)) {
        if (lane == 0)
          fa_report(kStatusWaitTimeout, 2 + t, 60);
        ok = false;
        break;
      }
      ++s_n;
      tc_fence_after_sync();
      if (row == 0 && item_n == 0)
        FA_STAMP(1 + t, j, 1);
      uint32_t s[128];
      tmem_ld_32x32b_x32(s_addr + 0, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_32x32b_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_32x32b_x32(s_addr + 64, *reinterpret_cast<uint32_t(*)[32]>(&s[64]));
      tmem_ld_32x32b_x32(s_addr + 96, *reinterpret_cast<uint32_t(*)[32]>(&s[96]));
      tmem_ld_wait();
      if (row == 0 && item_n == 0)
        FA_STAMP(1 + t, j, 2);

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
        // Sixteen independent chains: a three-input maximum has a long latency
        // (a chain of 16 took ~245 cycles), so the depth is kept at four.
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
      if (row == 0 && item_n == 0)
        FA_STAMP(1 + t, j, 3);
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
      if (row == 0 && item_n == 0)
        FA_STAMP(1 + t, j, 4);
      tmem_st_32x32b_x32(s_addr + 0, *reinterpret_cast<uint32_t(*)[32]>(&pk[0]));
      tmem_st_32x32b_x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&pk[32]));
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&sh->p_full[t]);
      if (row == 0 && item_n == 0)
        FA_STAMP(1 + t, j, 5);
    }

    if (ok && nb > 0) {
      if (!mbar_wait(&sh->o_full[t], tile_items & 1, abort_flag)) {
        if (lane == 0)
          fa_report(kStatusWaitTimeout, 2 + t, 70);
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
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              w[i] = pack2(__uint_as_float(o[2 * i]) * inv, __uint_as_float(o[2 * i + 1]) * inv, bf16);
            if (live) {
              uint4 *dst = reinterpret_cast<uint4 *>(out_row + cc * 2);
#pragma unroll
              for (int v = 0; v < 4; ++v)
                if (cc + 8 * v < p.head_dim) {
                  dst[v] = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
                }
            }
            if constexpr (kExtra) {
              const int first_row = q_row - lane; // a warp's 32 rows are consecutive
              store_extra_chunk_16bit(ex, extra_stage + (warp - 4) * 2048, lane, w,
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
          mbar_arrive(&sh->o_free[t]);
      }
    }
    } // work items
  }

  tc_fence_before_sync();
  __syncthreads();
#ifdef WAVE_FA_TRACE
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < 3 * 64 * 16; i += kThreads)
      if (i / 16 != 64 + 63) // [1][63][*] holds the clock probe
        (&g_fa_trace[0][0][0])[i] = fa_trace_smem[i];
  }
  if (threadIdx.x == 64 && blockIdx.x == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
    g_fa_trace[1][63][2] = clock64();
    g_fa_trace[1][63][3] = static_cast<long long>(ns);
  }
#endif
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

} // namespace

// ---------------------------------------------------------------- ticket ring
// Every launch draws its work items from one of kTicketSlots device counters.
// Slots are handed out round-robin per device; a slot carries an event recorded
// behind the launch that last used it, and the next user of the slot makes its
// stream wait for that event before it clears the counter.  A launch therefore
// never shares a counter with one that is still running, however many launches
// are queued on however many streams; the price is that launch k + kTicketSlots
// starts only after launch k has ended.  Under stream capture the event guard
// is left out (an event recorded outside the capture cannot be waited for
// inside it): a captured launch keeps the slot it was captured with, so two
// graphs that hold the same slot must not be replayed at the same time.
namespace {

constexpr int kMaxTicketDevices = 64;
struct TicketRing {
  cudaEvent_t done[kTicketSlots] = {};
  bool recorded[kTicketSlots] = {};
  unsigned next = 0;
  unsigned int *base = nullptr; // device address of g_fa_tickets on this device
};
std::mutex g_ticket_mu;
TicketRing g_ticket_rings[kMaxTicketDevices];

struct TicketSlot {
  unsigned int *counter = nullptr;
  int device = -1;
  unsigned index = 0;
  bool capturing = false;
};

int ticket_fail(cudaError_t err, const char *what) {
  std::string msg = std::string(what) + ": " + cudaGetErrorString(err);
  set_last_error(msg.c_str());
  return WAVE_E_CUDA;
}

// Picks the next slot of the current device's ring, orders `stream` behind the
// slot's previous launch and clears the counter on `stream`.  The caller holds
// g_ticket_mu from here until ticket_launched has run, so that no other host
// thread can come round to the same slot in between.
int ticket_acquire(cudaStream_t stream, TicketSlot *out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess)
    return ticket_fail(err, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxTicketDevices) {
    set_last_error("device ordinal out of range for the attention ticket ring");
    return WAVE_E_CUDA;
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) {
    cudaGetLastError();
    cap = cudaStreamCaptureStatusNone;
  }
  TicketRing &ring = g_ticket_rings[dev];
  if (!ring.base) {
    void *base = nullptr;
    if ((err = cudaGetSymbolAddress(&base, g_fa_tickets)) != cudaSuccess)
      return ticket_fail(err, "cudaGetSymbolAddress (attention tickets)");
    ring.base = static_cast<unsigned int *>(base);
  }
  TicketSlot s;
  s.device = dev;
  s.index = ring.next++ % kTicketSlots;
  s.counter = ring.base + s.index;
  s.capturing = cap != cudaStreamCaptureStatusNone;
  if (!s.capturing && ring.recorded[s.index] &&
      (err = cudaStreamWaitEvent(stream, ring.done[s.index], 0)) != cudaSuccess)
    return ticket_fail(err, "cudaStreamWaitEvent (attention ticket slot)");
  if ((err = cudaMemsetAsync(s.counter, 0, sizeof(unsigned int), stream)) != cudaSuccess)
    return ticket_fail(err, "cudaMemsetAsync (attention ticket)");
  *out = s;
  return WAVE_OK;
}

// Marks the end of the slot's launch on `stream` (called after the kernel has
// been enqueued, also when the enqueue failed: the memset is on the stream).
void ticket_launched(const TicketSlot &s, cudaStream_t stream) {
  if (s.device < 0 || s.capturing)
    return;
  TicketRing &ring = g_ticket_rings[s.device];
  if (!ring.done[s.index] &&
      cudaEventCreateWithFlags(&ring.done[s.index], cudaEventDisableTiming) != cudaSuccess) {
    cudaGetLastError();
    ring.done[s.index] = nullptr;
    ring.recorded[s.index] = false;
    return;
  }
  ring.recorded[s.index] = cudaEventRecord(ring.done[s.index], stream) == cudaSuccess;
}

} // namespace

int launch_flash_attention(const FaParams &p, const FaExtra &extra, const void *Q, const void *K, const void *V,
                           int sm_count, cudaStream_t stream) {
  if (p.head_dim < 16 || p.head_dim > kD || p.head_dim % 16)
    return WAVE_E_UNSUPPORTED;
  CUtensorMap tq, tk, tv;
  const uint32_t box[3] = {64, 128, 1};
  const uint64_t hd = static_cast<uint64_t>(p.head_dim);
  const uint64_t row_bytes = hd * 2;
  {
    const uint64_t dims[3] = {hd, static_cast<uint64_t>(p.seq_q), static_cast<uint64_t>(p.batch_heads)};
    const uint64_t strides[2] = {row_bytes, row_bytes * static_cast<uint64_t>(p.seq_q)};
    int rc = make_tensor_map_16bit(&tq, p.is_bf16, Q, 3, dims, strides, box);
    if (rc != WAVE_OK)
      return rc;
  }
  {
    const uint64_t dims[3] = {hd, static_cast<uint64_t>(p.seq_k), static_cast<uint64_t>(p.batch_heads)};
    const uint64_t strides[2] = {row_bytes, row_bytes * static_cast<uint64_t>(p.seq_k)};
    int rc = make_tensor_map_16bit(&tk, p.is_bf16, K, 3, dims, strides, box);
    if (rc != WAVE_OK)
      return rc;
    rc = make_tensor_map_16bit(&tv, p.is_bf16, V, 3, dims, strides, box);
    if (rc != WAVE_OK)
      return rc;
  }
  // Share of the exponentials evaluated on the FMA pipe, in eighths (a tuning
  // knob for measurements; the default is the measured best).
  const EnvKnobs env = env_knobs();
  int poly = env.fa_poly; // -1: each kernel's own default
  // Persistent CTAs, one per SM, draw work items (256 query rows of one head)
  // from a ticket counter.  Each launch takes the next of a ring of counters
  // and clears it on its stream, behind the launch that last used that counter,
  // so launches that overlap on the GPU do not share one.
  const long long total_items =
      static_cast<long long>(p.batch_heads) * ((p.seq_q + 2 * kBlockM - 1) / (2 * kBlockM));
  const unsigned grid = static_cast<unsigned>(total_items < sm_count ? total_items : sm_count);
  cudaError_t err = cudaSuccess;
  FaParams params = p;
  // Streaming kernel with a fixed softmax reference: cycles the warpgroup of an
  // item's second K/V block holds back once, so that the two warpgroups' phases
  // interleave instead of coinciding.  Measured sustained, variants taking turns
  // (non-causal / causal TFLOP/s, 0 -> 800..1000 cycles): B=2 H=64 S=8192
  // 1244/1154 -> 1259..1279/1171..1175; B=16 H=32 S=4096 1185/1032 ->
  // 1211/1058; B=8 H=32 S=2048 1059/830 -> 1097..1103/837..840; 1600 loses again.
  params.stagger = p.fixed_ref ? kFixedRefStagger : 0;
  if (env.fa_stagger >= 0)
    params.stagger = env.fa_stagger;
  std::lock_guard<std::mutex> ticket_lock(g_ticket_mu);
  TicketSlot slot;
  if (int rc = ticket_acquire(stream, &slot); rc != WAVE_OK)
    return rc;
  params.ticket = slot.counter;
  // Which kernel.  Left alone the launcher takes the decoupled kernel
  // (fa_decoupled_sm100.cu) for every shape; WAVE_CUDA_FA_KERNEL=
  // pingpong|stream|pair|decoupled forces one (a knob for measurements and the
  // tests; results agree to rounding).  Measured on one B200, inputs uniform in
  // [-1, 1), TFLOP/s sustained with the kernels taking turns / in 10-launch
  // bursts from idle, ping-pong | streaming | decoupled:
  //   causal, adaptive   S=1024 551|542|625 / 668|624|704   S=2048 723|735|800 / 859|842|906
  //                      S=4096 886|928|985 / 1095|1036|1113  S=8192 952|1051|1069 / 1184|1151|1213
  //   full, adaptive     S=1024 821|819|874 / 1004|942|993   S=2048 938|975|980 / 1140|1089|1125
  //                      S=4096 1010|1085|1085 / 1244|1196|1238  S=8192 1045|1155|1135 / 1299|1251|1290
  //   causal, fixed ref  S=1024 572|590|633 / 699|686|725   S=4096 873|1026|1040 / 1125|1127|1171
  //   full, fixed ref    S=2048 924|1076|1049 / 1163|1174|1199  S=8192 1031|1213|1246 / 1330|1331|1396
  // (B*H = 1024, 256, 512, 128 heads for the four lengths).
  {
    const int kernel = env.fa_kernel ? env.fa_kernel : 4;
    if (kernel == 2) {
      const int rc = launch_flash_attention_stream(params, extra, tq, tk, tv, poly, sm_count, stream);
      ticket_launched(slot, stream);
      return rc;
    }
    if (kernel == 4) {
      const int rc = launch_flash_attention_decoupled(params, extra, tq, K, V, poly, env.fa_stagger, sm_count, stream);
      ticket_launched(slot, stream);
      return rc;
    }
    // The CTA-pair kernel needs an even number of SMs.
    if (kernel == 3 && sm_count >= 2) {
      const int rc = launch_flash_attention_pair(params, extra, tq, K, tv, poly, sm_count, stream);
      ticket_launched(slot, stream);
      return rc;
    }
  }
  if (poly < 0)
    poly = kDefaultPoly;
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
    kernel<<<grid, kThreads, smem_bytes, stream>>>(tq, tk, tv, params, extra);
    err = cudaGetLastError();
  };
  auto dispatch = [&](auto bf16_tag) {
    constexpr bool B = decltype(bf16_tag)::value;
    if (extra.n > 0) { // further output buffers: the kernel variant whose epilogue writes them (default polynomial share)
      launch(fa_fwd_kernel<kDefaultPoly, B, true>);
      return;
    }
    switch (poly) {
    case 0: launch(fa_fwd_kernel<0, B, false>); break;
    case 1: launch(fa_fwd_kernel<1, B, false>); break;
    case 2: launch(fa_fwd_kernel<2, B, false>); break;
    case 3: launch(fa_fwd_kernel<3, B, false>); break;
    case 4: launch(fa_fwd_kernel<4, B, false>); break;
    default: launch(fa_fwd_kernel<kDefaultPoly, B, false>); break;
    }
  };
  if (p.is_bf16)
    dispatch(std::true_type{});
  else
    dispatch(std::false_type{});
  ticket_launched(slot, stream);
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

#ifdef WAVE_FA_TRACE
extern "C" int wave_cuda_fa_trace_read(long long *out, int clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fa_trace, sizeof(long long) * 3 * 64 * 16);
  if (err == cudaSuccess && clear) {
    static long long zero[3 * 64 * 16];
    err = cudaMemcpyToSymbol(g_fa_trace, zero, sizeof(zero));
  }
  return err == cudaSuccess ? 0 : -3;
}
#endif

// Status of both attention kernels: the first one that reported something.
cudaError_t fa_read_status(int out[4], bool clear) {
  cudaError_t err = cudaMemcpyFromSymbol(out, g_fa_status, sizeof(int) * 4);
  if (err == cudaSuccess && clear) {
    int zero[4] = {0, 0, 0, 0};
    err = cudaMemcpyToSymbol(g_fa_status, zero, sizeof(zero));
  }
  if (err != cudaSuccess)
    return err;
  int other[4];
  err = fa_stream_read_status(other, clear);
  if (err == cudaSuccess && out[0] == 0 && other[0] != 0)
    for (int i = 0; i < 4; ++i)
      out[i] = other[i];
  if (err != cudaSuccess)
    return err;
  err = fa_pair_read_status(other, clear);
  if (err == cudaSuccess && out[0] == 0 && other[0] != 0)
    for (int i = 0; i < 4; ++i)
      out[i] = other[i];
  if (err != cudaSuccess)
    return err;
  err = fa_decoupled_read_status(other, clear);
  if (err == cudaSuccess && out[0] == 0 && other[0] != 0)
    for (int i = 0; i < 4; ++i)
      out[i] = other[i];
  return err;
}

} // namespace wave
