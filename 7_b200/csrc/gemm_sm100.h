// Internal interface between the C-ABI backend and the sm_100a GEMM kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#define WAVE_GEMM_IN_F16 0
#define WAVE_GEMM_IN_BF16 1
#define WAVE_GEMM_OUT_F32 0
#define WAVE_GEMM_OUT_F16 1
#define WAVE_GEMM_OUT_BF16 2

namespace wave {

// Kernel-space problem: D[M x N] = A[M x K] * B[N x K]^T.  The backend may
// have swapped the caller's operands (skinny M), in which case stride_m and
// stride_n are swapped too and the caller's C comes out in its own layout.
struct GemmParams {
  int M, N, K;
  void *C;
  long long stride_m, stride_n; // element strides of D in the output buffer
  int in_type, out_type;
  int num_m_blocks, num_n_blocks, num_tiles, k_iters;
  int group_m;
  int split_from;      // CTA-pair kernel: tiles [split_from, num_tiles) run as two half-width work items each
  int pair_tile_n;     // CTA-pair kernel, 256-column instantiation: columns of a tile (a multiple of 32 in (128, 256])
  int dp_tiles;        // tiles [0, dp_tiles) are whole tiles dealt round-robin over the grid
  int streamk_workers; // >0: tiles [dp_tiles, num_tiles) are split Stream-K style over that many workers (= grid)
  float *scratch;      // Stream-K: [workers][2][128 x tile_n] f32 partial tiles
  int *counters;       // Stream-K: one arrival counter per output tile, zero on entry and exit
  // tile-packed output (16 x 16 tiles in workgroup -> wave -> per-wave-tile order)
  int tile_packed, tp_bm, tp_bn, tp_wmt, tp_wnt, tp_n_blocks;
  // order of the 256 values inside a tile: 0 row-major, 1 MFMA wave64, 2 WMMA wave32, 3 MFMA wave32 fragments
  int tp_fragment;
  int c_tma; // whole tiles leave through TMA stores (row-major 16-bit C, tiles of at least 64 columns)
  // L2 eviction hints on the operand loads: 0 none, 1 A "evict last" + B "evict first", 2 A "evict last" only
  int l2_hints;
  // CTA-pair kernel, TMA-store epilogue: every finished 128 x 64 piece of C is
  // also written, with plain 16-byte stores from the staging tile, to the same
  // place in `n_extra` further buffers (other GPUs' copies of C, mapped into
  // this process: the all-gather of the column blocks happens tile by tile
  // while the kernel computes).  Same strides as C.
  int n_extra;
  void *extra_c[7];
  // extra_c[0] is an NVLink multicast address (one store reaches every GPU bound
  // to the multicast object, replicated in the switch): written with multimem.st.
  int extra_multimem;
  // Test builds only (-DWAVE_WAIT_TEST): the one-CTA kernel's producer leaves out
  // the last K step of every segment, so that the UMMA thread's wait for it runs
  // out and the bounded-wait unwind can be observed.  Always 0 in the product.
  int test_skip_last_k;
  int pdl; // host side only: launch with programmatic stream serialization
};

int gemm_tile_m();
int gemm_tile_k();
cudaError_t launch_gemm(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, const CUtensorMap &tmap_c,
                        const GemmParams &p, int tile_n, int grid, cudaStream_t stream);
cudaError_t gemm_read_status(int out[4], bool clear);

// CTA-pair kernel (256 x 256 or 256 x 128 tiles, tcgen05 cta_group::2):
// data-parallel, optionally with a Stream-K tail over all pairs (streamk_workers
// = grid / 2, scratch [workers][2][2][128 x 256] f32, counters [tail tiles][2]).
// gemm_pair_tile_n() is the wide tile.
int gemm_pair_tile_m();
int gemm_pair_tile_n();
int gemm_pair_box_rows();
cudaError_t launch_gemm_pair(const CUtensorMap &tmap_a, const CUtensorMap &tmap_b, const CUtensorMap &tmap_b_half,
                             const CUtensorMap &tmap_c, const GemmParams &p, const CUtensorMap *extra_maps, int tile_n,
                             int grid, cudaStream_t stream);
cudaError_t gemm_pair_read_status(int out[4], bool clear);

} // namespace wave
