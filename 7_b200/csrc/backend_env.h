// Environment knobs of libwave_cuda.so, shared by its translation units.
// They steer choices the library otherwise makes by itself (which kernel, which
// tail treatment, ...) and exist for measurements; results never depend on them.
// The environment is read once, at the first call that needs a knob, and again
// only on wave_cuda_reload_env().
#pragma once

namespace wave {

struct EnvKnobs {
  int gemm_kernel = 0;           // WAVE_CUDA_GEMM_KERNEL: 0 auto, 1 single, 2 pair, 3 pair128
  bool gemm_split_tail = true;   // WAVE_CUDA_GEMM_SPLIT_TAIL=0: no half-width items in a sparse last round
  int gemm_streamk_tail = 1;     // WAVE_CUDA_GEMM_STREAMK_TAIL: 0 never, 1 where the cost model says it pays, 2 whenever possible
  int gemm_pair_tile_n = 0;      // WAVE_CUDA_GEMM_PAIR_TILE_N: width of the CTA-pair kernel's tiles (a multiple of 32 in (128, 256]), 0 = chosen
  bool gemm_tma_store = true;    // WAVE_CUDA_GEMM_TMA_STORE=0: per-thread stores instead of the TMA-store epilogue
  int gemm_l2_hints = 2;         // WAVE_CUDA_GEMM_L2_HINTS: 0 none, 1 A evict-last + B evict-first, 2 A evict-last only
  bool gemm_col_swap = true;     // WAVE_CUDA_GEMM_COL_SWAP=0: column-major 16-bit C without the operand swap
  bool gemm_pdl = true;          // WAVE_CUDA_GEMM_PDL=0: GEMM launches without programmatic dependent launch
  int fa_kernel = 0;             // WAVE_CUDA_FA_KERNEL: 0 auto, 1 pingpong, 2 stream, 3 pair, 4 decoupled
  int fa_poly = -1;              // WAVE_CUDA_FA_POLY: eighths of the exponentials on the FMA pipe, -1 = each kernel's default
  int fa_stagger = -1;           // WAVE_CUDA_FA_STAGGER: cycles, -1 = the library's default
};

EnvKnobs env_knobs();
void reload_env_knobs();

} // namespace wave
