/*
 * wave_cuda.h -- C ABI of the B200 (sm_100a) backend for the two dense kernels
 * the Wave compiler produces: the tiled f16/bf16 GEMM and the flash-attention
 * forward.  The library (libwave_cuda.so) stands where the reference's AMDGPU
 * assembly emission (lib/Target/Wave/AMDGPU.cpp, WaveCompileKernels.cpp) and
 * its ROCm launch (hipModuleLoad / hipModuleLaunchKernel in the calibrate
 * runners, mgpu* in mlir-runner) stand today, for these two kernels only.
 *
 * Conventions: every function returns 0 on success or a negative WAVE_E_* code
 * and never exits the process; wave_cuda_last_error() gives the message of the
 * calling thread's last failure.  The caller owns every device buffer.  Plain
 * pointers and sizes only; `stream` is a cudaStream_t passed as void*.
 * There is no CPU fallback: without a CUDA device every compute entry point
 * fails with WAVE_E_CUDA.
 */
#ifndef WAVE_CUDA_H
#define WAVE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes ------------------------------------------------------- */
#define WAVE_OK 0
#define WAVE_E_INVALID (-1)     /* argument validation failed (runner exit code 2) */
#define WAVE_E_UNSUPPORTED (-2) /* legal in the reference, outside this backend    */
#define WAVE_E_CUDA (-3)        /* a CUDA call failed (runner exit code 1)          */
#define WAVE_E_DEVICE_STATUS (-4) /* a kernel reported a bounded wait that ran out */
#define WAVE_E_NOT_FOUND (-5)

/* ---- element types and layouts ---------------------------------------- */
#define WAVE_F16 0
#define WAVE_BF16 1
#define WAVE_F32 2
#define WAVE_ROW_MAJOR 0 /* C[m*ldc + n]   (wave_matmul.py:1040) */
#define WAVE_COL_MAJOR 1 /* C[n*ldc + m]   (wave_matmul.py:1040) */
#define WAVE_TILE_PACKED 2 /* 16x16 tiles one after another, row-major inside a tile, in
                              workgroup -> wave -> per-wave-tile order: the order in which
                              compute_wmma_f16_matmul_reference_buffer emits them
                              (wave_matmul.py:1025-1028, 1106-1139) */
/* The same tile order, with the 256 values of a tile in the order of the AMD
 * accumulator fragments that the reference's timed runner checks
 * (getOutputCoordinate / getAccumulatorRow, wave-matmul-calibrate-runner.cpp:
 * 809-836): slot = lane * values_per_lane + v, column = lane % 16, and row
 *   MFMA, wave64: (lane / 16) * 4 + v   (4 values per lane)
 *   WMMA, wave32: (lane / 16) + 2 * v   (8 values per lane)
 *   MFMA, wave32: (lane / 16) * 8 + v   (8 values per lane) */
#define WAVE_TILE_PACKED_MFMA64 3
#define WAVE_TILE_PACKED_WMMA32 4
#define WAVE_TILE_PACKED_MFMA32 5

const char *wave_cuda_last_error(void);
const char *wave_cuda_version(void);

/* The WAVE_CUDA_* environment variables named below are measurement knobs.
 * The library reads them once, at the first call that needs one; a process
 * that changes its environment afterwards calls this to have them read again.
 * (The reference's tools take the corresponding choices as command-line
 * flags, wave-matmul-calibrate.py:1170; there is no reference function.) */
void wave_cuda_reload_env(void);

/* ---- mlir-runner host ABI ---------------------------------------------- *
 * Same seven symbols as runtime/wave_runtime.cpp:46-74: a rank-1 strided
 * memref descriptor {base, data, offset, size, stride} -> data + offset, the
 * address handed to the kernel as a `!wave.ptr<T, #wave.global>`.           */
void *_mlir_ciface_wave_memref_to_ptr_global_i32(void *memref1d);
void *_mlir_ciface_wave_memref_to_ptr_global_i8(void *memref1d);
void *_mlir_ciface_wave_memref_to_ptr_global_f32(void *memref1d);
void *_mlir_ciface_wave_memref_to_ptr_global_f16(void *memref1d);
void *_mlir_ciface_wave_memref_to_ptr_global_bf16(void *memref1d);
void *_mlir_ciface_wave_memref_to_ptr_global_i64(void *memref1d);
void *_mlir_ciface_wave_memref_to_ptr_global_f64(void *memref1d);

/* ---- tiled GEMM --------------------------------------------------------- *
 * C[M x N] = A[M x K] * B, with B stored N x K row-major (the reference keeps
 * B transposed: wave_matmul.py:328-332), f32 accumulation, one final
 * round-to-nearest-even to out_type.  The descriptor carries what the
 * reference bakes into the kernel at code generation (_MatmulConfig,
 * wave_matmul.py:288-530) and what its runner takes as flags
 * (wave-matmul-calibrate-runner.cpp:36-64).  The tiling knobs never change
 * results; they choose the CTA tile:
 *   16*bm*wave_m_tiles x 16*bn*wave_n_tiles, snapped to a legal UMMA shape
 *   (rows 128; columns the next of 16/32/64/128/256).
 * Requested tiles of at least 256 x 256 run on CTA pairs (tcgen05
 * cta_group::2, 256 x 256 tiles) where those fill the machine at least as well
 * as 128 x 256 tiles on single CTAs.  A last round of tiles that would leave
 * CTA pairs idle runs as half-width items or, with streamk_workers = 0 and a
 * workspace, has its K iterations dealt over all pairs (Stream-K tail).
 * Column-major 16-bit C is computed as the row-major C^T = B * A^T (operands
 * swapped inside the library; bit-identical results).  Launches carry the
 * programmatic-stream-serialization attribute: a kernel's set-up may overlap
 * the end of the kernel before it on the stream, its first access to global
 * memory waits for that kernel to be complete.  The environment
 * variables WAVE_CUDA_GEMM_KERNEL=pair|pair128|single,
 * WAVE_CUDA_GEMM_SPLIT_TAIL=0, WAVE_CUDA_GEMM_STREAMK_TAIL=0,
 * WAVE_CUDA_GEMM_TMA_STORE=0, WAVE_CUDA_GEMM_COL_SWAP=0,
 * WAVE_CUDA_GEMM_L2_HINTS=0|1|2 and WAVE_CUDA_GEMM_PDL=0 override the choices
 * (knobs for measurements; results do not change).                           */
typedef struct wave_gemm_desc {
  int M, N, K;                 /* positive multiples of 16 (wave_matmul.py:533-536)      */
  int bm, bn;                  /* waves per workgroup along M / N; bn a power of two      */
  int wave_m_tiles, wave_n_tiles, wave_k_tiles; /* 16x16 tiles per wave, K slices per step */
  int in_type;                 /* WAVE_F16 | WAVE_BF16                                      */
  int out_type;                /* WAVE_F32 | WAVE_F16 | WAVE_BF16                           */
  int out_layout;              /* WAVE_ROW_MAJOR | WAVE_COL_MAJOR | WAVE_TILE_PACKED[_...]  */
  int cta_group_m;             /* grouped-M rasterisation (wave_matmul.py:1267-1272); >= 1 */
  int streamk_workers;         /* 0 auto, 1 plain tiles, >1 persistent Stream-K grid
                                  (--streamk-workers, wave-matmul-calibrate.py:1170)      */
  int ldc;                     /* leading dimension of C in elements; 0 = N (row-major) or
                                  M (column-major).  Lets a rank write its column shard
                                  into a larger C in place.                                */
} wave_gemm_desc;

/* Fills the descriptor with the runner's defaults (bm 1, bn 2, tiles 1, f16 in,
 * f32 out, row-major: runner.cpp:36-64). */
void wave_cuda_gemm_desc_init(wave_gemm_desc *desc, int M, int N, int K);

/* Same rules and messages as _validate_positive_shape / _validate_tile_shape
 * (wave_matmul.py:533-619).  Needs no GPU. */
int wave_cuda_gemm_validate(const wave_gemm_desc *desc);

/* Bytes of device workspace wave_cuda_gemm needs for this descriptor: f32
 * partial tiles then int32 arrival counters (zero on entry; the kernel leaves
 * them zero).  Both are 0 when the launch does not split K.  Mirrors
 * getStreamKWorkspaceSizes (runner.cpp:393-408).  Needs no GPU unless
 * streamk_workers is 0 (auto), which asks the device for its SM count. */
int wave_cuda_gemm_workspace_bytes(const wave_gemm_desc *desc, size_t *scratch_bytes, size_t *counter_bytes);

/* Launches the GEMM on `stream`.  A, B, C are device pointers, 16-byte
 * aligned; `workspace` is scratch_bytes + counter_bytes (counters follow the
 * scratch, zero-initialised by the caller once) or NULL when both are 0.
 * Replaces hipModuleLaunchKernel with {&A,&B,&C,&trip} / the Stream-K block
 * {&A,&B,&C,&scratch,&counters,&workers} (runner.cpp:1790-1791, 1811-1816).  */
int wave_cuda_gemm(const wave_gemm_desc *desc, const void *A, const void *B, void *C, void *workspace,
                   void *stream);

/* No counterpart in the reference, which is single-device.  The GEMM with its
 * result written to several buffers at once: C_targets[0] exactly as
 * wave_cuda_gemm writes C, and every finished 128 x 64 piece of it also, with
 * one more TMA store each out of the epilogue's staging tile, to
 * C_targets[1 .. n_targets-1] at the same offsets and leading dimension.  This
 * is the all-gather of an N-column-sharded GEMM fused into the kernel: rank r
 * of a job whose ranks hold peer-mapped copies of the full C (column-major:
 * rank r's block starts n_begin * ldc elements in) passes the address of ITS
 * block inside every rank's copy, its own first, and the blocks travel over
 * NVLink tile by tile while the tensor cores work on the next tile, instead of
 * in a collective after the kernel.  The stores are complete when the kernel
 * is; another GPU may read its copy once it has synchronised with this stream
 * (a barrier across the ranks).  1 <= n_targets <= 8.  Needs the CTA-pair
 * kernel's TMA-store epilogue: 16-bit C, row- or column-major, M and N of at
 * least 256, tiling knobs asking for 256 x 256 tiles; otherwise
 * WAVE_E_UNSUPPORTED.  Uses no workspace. */
int wave_cuda_gemm_multi_output(const wave_gemm_desc *desc, const void *A, const void *B, void *const *C_targets,
                                int n_targets, void *stream);

/* The same with the other copies reached through ONE NVLink multicast address
 * (NVLS): `C_multicast` is the block's place inside a multicast mapping of the
 * ranks' copies of C (every GPU bound to the multicast object receives each
 * store, replicated in the switch, this GPU's own copy included), so a tile
 * leaves the GPU once instead of once per peer.  Written with multimem.st from
 * the epilogue; `C_local` is written as wave_cuda_gemm writes C.  Same limits
 * as wave_cuda_gemm_multi_output; no counterpart in the reference. */
int wave_cuda_gemm_multicast_output(const wave_gemm_desc *desc, const void *A, const void *B, void *C_local,
                                    void *C_multicast, void *stream);

/* Host-buffer form (what the mlir-runner host main does with host-registered
 * memrefs, wave_matmul.py:6926-6937): copies A and B to the device, runs,
 * copies C back, all on `stream`, then synchronises it.  Device staging
 * buffers are cached in the library and grow on demand. */
int wave_cuda_gemm_host(const wave_gemm_desc *desc, const void *A_host, const void *B_host, void *C_host,
                        void *stream);

/* The same call for one rank of an N-column-sharded GEMM: B and C are the
 * rank's column block in host memory, A (replicated on every rank) is already
 * on the device, 16-byte aligned and ready on `stream` -- e.g. gathered over
 * NVLink from the M/ranks rows each rank copied from its host, instead of
 * every rank copying the whole of A over PCIe.  (The reference is
 * single-device; its host main registers A, B and C alike,
 * wave_matmul.py:6926-6937.) */
int wave_cuda_gemm_host_a_resident(const wave_gemm_desc *desc, const void *A_device, const void *B_host,
                                   void *C_host, void *stream);

/* No counterpart in the reference.  Stream-K GEMM for callers that cannot
 * supply (or allocate) the workspace wave_cuda_gemm asks for: hosts written to
 * the reference's plain {A, B, C, trip} argument list, which has no workspace
 * slot; processes whose device memory is wholly owned by another allocator;
 * paths on which a device allocation must not happen.  The partial tiles and
 * counters live in one fixed WAVE_CUDA_STATIC_WORKSPACE_BYTES area inside the
 * library's device image (held by every GPU that loads the library until the
 * process exits); nothing is allocated or freed.  A descriptor that needs more
 * than the area holds is refused with WAVE_E_INVALID when it names a worker
 * count; with streamk_workers = 0 (automatic) a plan that does not fit runs as
 * whole tiles instead, without a workspace.  The first call on a
 * device looks the area's address up and should be made before any stream
 * capture.  Every call shares the area: calls whose kernels overlap on the GPU
 * race and must be serialised by the caller.  Same arguments and results as
 * wave_cuda_gemm with a caller workspace. */
#define WAVE_CUDA_STATIC_WORKSPACE_BYTES (8 * 1024 * 1024)
int wave_cuda_gemm_streamk_static(const wave_gemm_desc *desc, const void *A, const void *B, void *C, void *stream);

/* Launch geometry the backend chose (tile rows, tile columns, grid size,
 * Stream-K workers or 0, operands swapped or not) -- the counterpart of the
 * runner's `grid:` / `shape:` lines (runner.cpp:1881-1908). */
int wave_cuda_gemm_plan(const wave_gemm_desc *desc, int *tile_m, int *tile_n, int *grid, int *streamk_workers,
                        int *swapped);

/* The same for a GPU of `sm_count` SMs that need not be present (no device is
 * asked for anything): what the backend would launch there, with or without a
 * workspace, and the workspace it would want.  For planning tools and tests. */
int wave_cuda_gemm_plan_for_sms(const wave_gemm_desc *desc, int sm_count, int have_workspace, int *tile_m, int *tile_n,
                                int *grid, int *streamk_workers, int *swapped, size_t *scratch_bytes,
                                size_t *counter_bytes);

/* ---- flash-attention forward ------------------------------------------- *
 * O = softmax(scale * Q K^T [+ causal mask]) V per (batch, head).  Layout
 * (B, H, S, D) contiguous, the same bytes as the gfx950 runner's [B*H][S][D]
 * (wave_flash_attention.py:242-254; operator surface
 * integrations/tlx/workloads/amd_fa_wave.py:1671-1682).  f32 online-softmax
 * statistics, exp2 with scale*log2(e) folded into the exponent
 * (wave_flash_attention.py:596-600), probabilities rounded to io_type before
 * P*V, output rounded once to io_type.  `causal` keeps key <= query (top-left
 * aligned; an extension, the reference's Wave kernel is non-causal).
 * Four kernels compute it: 256-row work items whose two Q tiles take K/V in
 * blocks of 80 keys with scores and probabilities side by side in tensor
 * memory (the one the library uses); the same tiles ping-ponging over 128-key
 * blocks; 128-row work items with double-buffered scores; CTA pairs on 512-row
 * work items.  WAVE_CUDA_FA_KERNEL=decoupled|pingpong|stream|pair forces one,
 * WAVE_CUDA_FA_POLY=0..4 sets the eighths of the exponentials evaluated as a
 * polynomial on the FMA pipe, WAVE_CUDA_FA_STAGGER=<cycles> the one-off offset
 * between the two softmax warpgroups (measurement knobs; the results agree
 * within the rounding of the exponential and of the running maximum's steps).
 * Launches in flight: each launch draws its work items from one of 64 device
 * counters per GPU, handed out in turn.  The launch that comes round to a
 * counter is ordered (by an event) behind the launch that used it 64 launches
 * earlier, so any number of launches may be queued on any number of streams;
 * at most 64 of them run side by side.  Under stream capture that ordering is
 * left out: two captured graphs that hold the same counter (captured 64
 * launches apart) must not be replayed at the same time.
 */
typedef struct wave_fa_desc {
  int batch, heads;
  int seq_q, seq_k; /* multiples of 16 */
  int head_dim;     /* 128 is the reference production kernel's only value
                       (wave_flash_attention.py:43-60) and the tuned one; multiples of 16
                       up to 128 (the toy kernel's 16/32/64, wave_attention.py) run
                       zero-padded to 128 */
  float scale;      /* 0 = 1/sqrt(head_dim) */
  int causal;
  int io_type;      /* WAVE_BF16 | WAVE_F16 */
  int out_f32;      /* non-zero: O is f32 (the toy kernel `flash_attention_f32`, f16 in /
                       f32 out, wave_attention.py:18); zero: O has io_type */
  float qk_max_abs; /* 0: adaptive running row maximum.  > 0: a bound on |q| and |k|
                       entries that selects the reference's fixed-reference
                       specialisation (wave_flash_attention.py:50, 64-75, 108-113,
                       602-609; amd_fa_wave.py:1582-1611): every exponential is taken
                       against the constant log2(e) * head_dim * scale * qk_max_abs^2,
                       no row maximum is searched and the accumulator is never
                       rescaled.  Twice that constant must stay below 126. */
} wave_fa_desc;

int wave_cuda_fa_validate(const wave_fa_desc *desc);

/* Q, K, V, O device pointers (16-byte aligned); lse_or_null, when given,
 * receives the natural-log sum-exp of the scaled scores per row, f32
 * [batch*heads][seq_q].  Replaces hipModuleLaunchKernel with {&Q,&K,&V,&O}
 * (wave-fa-gfx950-runner.cpp:396-402, 446). */
int wave_cuda_flash_attention_fwd(const wave_fa_desc *desc, const void *Q, const void *K, const void *V, void *O,
                                  float *lse_or_null, void *stream);

/* No counterpart in the reference (single-device).  The forward with O written
 * to several buffers at once, for the gather of (batch, head)-sharded attention
 * inside the kernel: O_targets[0] as above, and every 16 bytes of O the epilogue
 * stores also to O_targets[1 .. n_targets-1] at the same offset (other ranks'
 * copies of the full O, mapped into this process; rank r passes the address of
 * ITS slab inside each copy).  The multicast form sends each piece once to an
 * NVLink multicast address (multimem.st) that reaches every rank's copy.  The
 * log-sum-exp goes to `lse_or_null` only.  Stores are complete when the kernel
 * is; synchronise the ranks before reading a copy.  1 <= n_targets <= 8. */
int wave_cuda_flash_attention_fwd_multi_output(const wave_fa_desc *desc, const void *Q, const void *K, const void *V,
                                               void *const *O_targets, int n_targets, float *lse_or_null, void *stream);
int wave_cuda_flash_attention_fwd_multicast_output(const wave_fa_desc *desc, const void *Q, const void *K,
                                                   const void *V, void *O_local, void *O_multicast,
                                                   float *lse_or_null, void *stream);

int wave_cuda_flash_attention_fwd_host(const wave_fa_desc *desc, const void *Q_host, const void *K_host,
                                       const void *V_host, void *O_host, void *stream);

/* ---- name-based launch facade ------------------------------------------ *
 * Keeps the runners' call shape (hipModuleGetFunction by kernel name, then a
 * launch with a void* args[] block of pointers-to-values): names
 * "wmma_f16_matmul_tiled" (args {&A,&B,&C,&trip}), "gfx950_f16_streamk_gemm"
 * (args {&A,&B,&C,&scratch,&counters,&workers}), "flash_attention_bf16_gfx950"
 * and "flash_attention_f32" (args {&Q,&K,&V,&O})
 * (wave_matmul.py:777-779; wave_flash_attention.py:16; wave_attention.py:18).
 * `desc` is a wave_gemm_desc or wave_fa_desc and is copied into the handle. */
int wave_cuda_module_get_function(const char *kernel_name, const void *desc, void **fn);
int wave_cuda_launch(void *fn, void **args, void *stream);
void wave_cuda_function_release(void *fn);

/* ---- device status ------------------------------------------------------ *
 * Every device-side wait is bounded; a wait that runs out records
 * {code, block, role, detail} and the kernel unwinds.  This synchronises the
 * device, returns WAVE_E_DEVICE_STATUS if any kernel since the last call
 * reported a problem (details in out4 if non-NULL), and clears the record. */
int wave_cuda_check_device_status(int *out4);

#ifdef __cplusplus
}
#endif
#endif /* WAVE_CUDA_H */
