// Internal interface between the C-ABI backend and the sm_100a flash-attention
// forward kernel.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wave {

struct FaParams {
  int batch_heads, seq_q, seq_k, head_dim;
  int causal, is_bf16;
  int out_f32;       // O is f32 instead of the 16-bit I/O type
  float scale;       // softmax scale applied to q.k
  float scale_log2e; // scale * log2(e): scores enter exp2 as fma(s, scale_log2e, -max)
  int fixed_ref;     // exponentials against the constant ref_log2 instead of the running row maximum
  int stagger;       // streaming kernel, fixed reference: cycles the odd-block warpgroup holds back at each item's start
  float ref_log2;    // that constant, in log2 units of the scaled scores
  void *O;           // [batch_heads][seq_q][head_dim], the I/O type or f32
  float *lse;        // optional [batch_heads][seq_q] natural-log sum-exp, or null
  unsigned int *ticket; // device counter, zero at launch: the persistent CTAs draw work items from it
};

// Further output buffers of a launch: every 16 bytes of O the epilogue stores
// go, at the same offset, to `n` more buffers too (other GPUs' copies of the
// full O when the (batch, head) slabs of a sharded problem are gathered inside
// the kernel); with `multimem`, o[0] is an NVLink multicast address and one
// multimem.st reaches every GPU.  The log-sum-exp is written locally only.
// A kernel parameter of its own, and only of the kernel variants that use it:
// the ordinary kernels' parameter block and code are unchanged by it.
struct FaExtra {
  int n, multimem;
  void *o[7];
};

// Builds the tensor maps and launches.  Returns a WAVE_* code (0 = ok).
int launch_flash_attention(const FaParams &p, const FaExtra &extra, const void *Q, const void *K, const void *V,
                           int sm_count, cudaStream_t stream);
cudaError_t fa_read_status(int out[4], bool clear);
// The streaming kernel (fa_stream_sm100.cu): one 128-row Q tile per CTA, score
// and probability buffers double-buffered in tensor memory.  `p.ticket` must
// point at a zeroed work-item counter.
int launch_flash_attention_stream(const FaParams &p, const FaExtra &extra, const CUtensorMap &tq, const CUtensorMap &tk,
                                  const CUtensorMap &tv, int poly, int sm_count, cudaStream_t stream);
cudaError_t fa_stream_read_status(int out[4], bool clear);
// The CTA-pair kernel (fa_pair_sm100.cu): 512-row work items on 2-CTA clusters,
// tcgen05 cta_group::2.  `tq` / `tv` have boxes of 64 elements x 128 rows; K's
// map (64 x 64) is built inside.  `p.ticket` as above.
int launch_flash_attention_pair(const FaParams &p, const FaExtra &extra, const CUtensorMap &tq, const void *K,
                                const CUtensorMap &tv, int poly, int sm_count, cudaStream_t stream);
cudaError_t fa_pair_read_status(int out[4], bool clear);
// The decoupled kernel (fa_decoupled_sm100.cu): 256-row work items, 80-key
// blocks, P beside S in tensor memory so that Q*K^T of a tile's next block runs
// during its softmax.  `tq` has boxes of 64 elements x 128 rows; K's and V's
// maps (64 x 80) are built inside.  `stagger_cycles` < 0: the kernel's own
// default (it replaces p.stagger).  `p.ticket` as above.
int launch_flash_attention_decoupled(const FaParams &p, const FaExtra &extra, const CUtensorMap &tq, const void *K,
                                     const void *V, int poly, int stagger_cycles, int sm_count, cudaStream_t stream);
cudaError_t fa_decoupled_read_status(int out[4], bool clear);

// Provided by the backend: rank-2/3 tensor map over 16-bit elements with the
// 128-byte swizzle and zero fill outside the tensor.
int make_tensor_map_16bit(CUtensorMap *map, int is_bf16, const void *base, int rank, const uint64_t *dims,
                          const uint64_t *strides_bytes, const uint32_t *box);

} // namespace wave
