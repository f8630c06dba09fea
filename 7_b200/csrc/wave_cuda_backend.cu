// Host side of libwave_cuda.so: the C ABI declared in include/wave_cuda.h.
// It is the CUDA sibling of the reference's runtime/wave_runtime.cpp (the
// memref -> pointer shims are restated here) plus what the reference's
// calibrate runners do on the host around a launch: argument validation
// (python/mlir/dialects/wave_matmul.py:533-619), launch geometry
// (wave-matmul-calibrate-runner.cpp:1744-1764), Stream-K workspace sizing
// (runner.cpp:393-408) and the kernel-argument blocks (runner.cpp:1790-1816).
// There is no CPU fallback anywhere in this file.
#include "../../include/wave_cuda.h"
#include "backend_env.h"
#include "fa_sm100.h"
#include "gemm_sm100.h"

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <initializer_list>
#include <string>
#include <vector>

namespace {

thread_local std::string g_last_error;

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int cuda_fail(cudaError_t err, const char *what) {
  return fail(WAVE_E_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// ---------------------------------------------------------------- tensor maps
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

} // namespace

namespace wave {

// The WAVE_CUDA_* environment knobs are read once (at the first call that needs
// them) and again only when the caller asks with wave_cuda_reload_env().
namespace {
std::mutex g_env_mu;
EnvKnobs g_env;
bool g_env_loaded = false;

EnvKnobs read_env() {
  EnvKnobs e;
  if (const char *v = getenv("WAVE_CUDA_GEMM_KERNEL"))
    e.gemm_kernel = !strcmp(v, "single") ? 1 : !strcmp(v, "pair") ? 2 : !strcmp(v, "pair128") ? 3 : 0;
  if (const char *v = getenv("WAVE_CUDA_GEMM_SPLIT_TAIL"))
    e.gemm_split_tail = strcmp(v, "0") != 0;
  if (const char *v = getenv("WAVE_CUDA_GEMM_STREAMK_TAIL"))
    e.gemm_streamk_tail = !strcmp(v, "0") ? 0 : !strcmp(v, "force") ? 2 : 1;
  if (const char *v = getenv("WAVE_CUDA_GEMM_PAIR_TILE_N")) {
    const int n = atoi(v);
    e.gemm_pair_tile_n = (n > 128 && n <= 256 && n % 32 == 0) ? n : 0;
  }
  if (const char *v = getenv("WAVE_CUDA_GEMM_TMA_STORE"))
    e.gemm_tma_store = strcmp(v, "0") != 0;
  if (const char *v = getenv("WAVE_CUDA_GEMM_L2_HINTS"))
    e.gemm_l2_hints = atoi(v);
  if (const char *v = getenv("WAVE_CUDA_GEMM_COL_SWAP"))
    e.gemm_col_swap = strcmp(v, "0") != 0;
  if (const char *v = getenv("WAVE_CUDA_GEMM_PDL"))
    e.gemm_pdl = strcmp(v, "0") != 0;
  if (const char *v = getenv("WAVE_CUDA_FA_KERNEL"))
    e.fa_kernel = !strcmp(v, "pingpong") ? 1 : !strcmp(v, "stream") ? 2 : !strcmp(v, "pair") ? 3 : !strcmp(v, "decoupled") ? 4 : 0;
  if (const char *v = getenv("WAVE_CUDA_FA_POLY"))
    e.fa_poly = atoi(v);
  if (const char *v = getenv("WAVE_CUDA_FA_STAGGER")) {
    const int cycles = atoi(v);
    e.fa_stagger = cycles < 0 ? 0 : (cycles > 100000 ? 100000 : cycles); // a bounded spin, whatever is asked
  }
  return e;
}
} // namespace

EnvKnobs env_knobs() {
  std::lock_guard<std::mutex> lock(g_env_mu);
  if (!g_env_loaded) {
    g_env = read_env();
    g_env_loaded = true;
  }
  return g_env;
}

void reload_env_knobs() {
  std::lock_guard<std::mutex> lock(g_env_mu);
  g_env = read_env();
  g_env_loaded = true;
}

// Lets the library's other translation units record a failure message.
void set_last_error(const char *message) { g_last_error = message ? message : ""; }

// rank-2 or rank-3 map over 16-bit elements, 128-byte swizzle, zero fill
// outside the tensor.  dims/strides innermost first; strides in bytes for
// dims 1.. (dim 0 is contiguous).
int make_tensor_map_16bit(CUtensorMap *map, int is_bf16, const void *base, int rank, const uint64_t *dims,
                          const uint64_t *strides_bytes, const uint32_t *box) {
  EncodeTiledFn fn = encode_fn();
  if (!fn)
    return fail(WAVE_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[3], gstr[2];
  cuuint32_t bdim[3], estr[3];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i)
    gstr[i] = strides_bytes[i];
  CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  static_cast<cuuint32_t>(rank), const_cast<void *>(base), gdim, gstr, bdim, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(WAVE_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu x %llu, box %u x %u)",
                static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]),
                static_cast<unsigned long long>(dims[1]), box[0], box[1]);
  return WAVE_OK;
}

} // namespace wave

namespace {

int sm_count(int *out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess)
    return cuda_fail(err, "cudaGetDevice");
  int sms = 0;
  err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (err != cudaSuccess)
    return cuda_fail(err, "cudaDeviceGetAttribute");
  *out = sms;
  return WAVE_OK;
}

int elem_size(int type) { return type == WAVE_F32 ? 4 : 2; }

bool is_tile_packed(int layout) { return layout >= WAVE_TILE_PACKED && layout <= WAVE_TILE_PACKED_MFMA32; }

// ---------------------------------------------------------------- GEMM plan
struct GemmPlan {
  bool pair;          // CTA-pair kernel: 256 x 256 or 256 x 128 tiles, two CTAs per tile
  int tile_m;         // kernel-space tile rows
  bool swapped;       // kernel computes C^T = B * A^T (skinny M)
  int Mk, Nk;         // kernel-space extents
  int tile_n;         // kernel-space tile columns
  int num_m, num_n, k_iters;
  int grid;
  int streamk_workers; // 0 = data-parallel
  int dp_tiles;        // whole tiles dealt round-robin before the Stream-K part (all of them if no Stream-K)
  int split_from;      // CTA-pair kernel: tiles from this one on run as two half-width work items
  size_t scratch_bytes, counter_bytes;
};

// Steady-state rate of the one-CTA kernel relative to the 256 x 256 pair tile
// (8192^3 bf16, measured: 1381 against 1507 TFLOP/s).
constexpr double kSingleRate = 0.915;

// Duration of a round of half-width (256 x 128) work items of the CTA-pair
// kernel relative to a round of whole tiles: half the work at 0.69 of the rate.
constexpr double kHalfItemCost = 0.72;

// What the Stream-K treatment of a partly filled last round costs on top of
// its share of a round, in rounds: every pair writes f32 partial tiles, and the
// last arriver of a tile reads them all back and stores C after everybody else
// has finished, so that latency is exposed at the end of the kernel.  Measured
// on 8192 x {1024, 2048, 8192} x 8192 bf16 (54, 34 and 62 tail tiles on 74
// pairs): 0.55 to 1.1 rounds.
constexpr double kStreamKTailOverhead = 0.75;

// Relative duration of a round of 256 x n tiles of the CTA-pair kernel (n = 256:
// 1).  A narrower tile saves less time than columns: per flop it moves more
// operand bytes from L2, and under the power cap time follows energy rather
// than tensor-pipe cycles.  Measured on 8192 x 2048 x 8192 bf16, sustained and
// interleaved: a round of 224-column tiles 0.93 to 0.99, of 192-column tiles
// 0.90 to 0.92 of a round of 256-column ones; 128 (the narrow instantiation) 0.72.
double pair_tile_cost(int n) {
  switch (n) {
  case 256: return 1.0;
  case 224: return 0.95;
  case 192: return 0.92;
  case 160: return 0.88;
  }
  return 1.0;
}

// How the CTA-pair kernel treats a last round of `tail` whole tiles on `pairs`
// CTA pairs, and what that round then costs in rounds of whole tiles.
enum class PairTail { kWhole, kHalfItems, kStreamK };
struct PairTailChoice {
  PairTail how;
  double rounds;
};
PairTailChoice pair_tail_choice(long long tail, long long pairs, int k_iters, int tile_n, bool streamk_allowed,
                                const wave::EnvKnobs &env) {
  PairTailChoice best{PairTail::kWhole, tail > 0 ? 1.0 : 0.0};
  if (tail <= 0)
    return best;
  // twice as many half-width items, if those still fit one round
  if (env.gemm_split_tail && tile_n == 256 && 2 * tail <= pairs && kHalfItemCost < best.rounds)
    best = {PairTail::kHalfItems, kHalfItemCost};
  // the tail's K iterations dealt evenly over all pairs
  if (streamk_allowed && env.gemm_streamk_tail && k_iters >= 8 && tail * k_iters >= pairs) {
    const double cost = static_cast<double>(tail) / static_cast<double>(pairs) + kStreamKTailOverhead;
    if (cost < best.rounds || env.gemm_streamk_tail == 2)
      best = {PairTail::kStreamK, cost};
  }
  return best;
}

// Tile width of the CTA-pair kernel for a problem of num_m x Nk in kernel
// space: the multiple of 32 in (128, 256] whose rounds of tiles, weighted by
// the cost of a tile of that width, are fewest.  Narrower tiles make more of
// them, which can turn a badly filled last round into a full one: 8192 x 1024
// (an eighth of the 8192-column problem) is 128 tiles of 256 columns, 1.73
// rounds on 74 pairs, but exactly two rounds of 148 tiles of 224 columns.
struct PairWidthChoice {
  int tile_n;
  double cost; // rounds of 256-column tiles
  PairTailChoice tail;
};
PairWidthChoice pair_width_choice(long long num_m, int Nk, long long pairs, int k_iters, bool streamk_allowed,
                                  const wave::EnvKnobs &env) {
  PairWidthChoice best{256, 0.0, {PairTail::kWhole, 0.0}};
  bool first = true;
  for (int n = 256; n > 128; n -= 32) {
    if (env.gemm_pair_tile_n && n != env.gemm_pair_tile_n)
      continue;
    const long long tiles = num_m * ((Nk + n - 1) / n);
    const PairTailChoice tail = pair_tail_choice(tiles % pairs, pairs, k_iters, n, streamk_allowed, env);
    const double cost = (static_cast<double>(tiles / pairs) + tail.rounds) * pair_tile_cost(n);
    if (first || cost < best.cost * 0.97) { // a narrower tile must win by a margin
      best = {n, cost, tail};
      first = false;
    }
  }
  return best;
}

int snap_tile_n(int want) {
  const int options[5] = {16, 32, 64, 128, 256};
  for (int o : options)
    if (want <= o)
      return o;
  return 256;
}

// `sms` <= 0 means "unknown" (no device query): only legal when the
// descriptor does not ask for automatic Stream-K.
// `need_pair`: the caller needs the CTA-pair kernel's epilogue (output to
// several buffers); the size heuristic is then not allowed to pick the
// one-CTA kernel.
int make_plan(const wave_gemm_desc &d, int sms, bool have_workspace, GemmPlan *plan, bool need_pair = false) {
  wave::EnvKnobs env = wave::env_knobs();
  if (need_pair && env.gemm_kernel != 3)
    env.gemm_kernel = 2;
  const int tile_m = wave::gemm_tile_m(), tile_k = wave::gemm_tile_k();
  const int want_m = 16 * d.bm * d.wave_m_tiles, want_n = 16 * d.bn * d.wave_n_tiles;
  GemmPlan p{};
  // A 128-row UMMA wastes most of its rows on a skinny M; put N on the rows
  // instead and M on the (narrow) column tile.
  const bool skinny = d.M < tile_m && d.N > d.M && !is_tile_packed(d.out_layout);
  // Column-major 16-bit C (offset n*ld + m, wave_matmul.py:1040) is the
  // row-major output of C^T = B * A^T: swapping the operands lets the tiles
  // leave through the TMA-store epilogue (whole 128-byte rows) instead of one
  // 2-byte store per thread and element.  Products and the k-ascending f32
  // accumulation are the same either way, so the result is bit-identical.
  // (Only where the swapped tile is wide enough for that epilogue: the knobs'
  // M tile becomes the kernel's column tile.)
  const bool col_swap = !skinny && env.gemm_col_swap && d.out_layout == WAVE_COL_MAJOR && d.out_type != WAVE_F32 &&
                        d.M >= 64 && d.N >= tile_m && snap_tile_n(want_m) >= 64;
  p.swapped = skinny || col_swap;
  p.Mk = p.swapped ? d.N : d.M;
  p.Nk = p.swapped ? d.M : d.N;
  const int want_mk = p.swapped ? want_n : want_m, want_nk = p.swapped ? want_m : want_n;
  p.tile_n = snap_tile_n(want_nk);
  const int cap = snap_tile_n(p.Nk);
  if (p.tile_n > cap)
    p.tile_n = cap;
  p.tile_m = tile_m;
  const bool auto_streamk = d.streamk_workers == 0 && sms > 0 && have_workspace;
  // Large tiles on a large problem go to the CTA-pair kernel (whole tiles, with
  // an automatic Stream-K tail when there is a workspace; explicit worker counts
  // are the one-CTA kernel's).
  p.pair = !skinny && want_mk >= wave::gemm_pair_tile_m() && want_nk >= wave::gemm_pair_tile_n() &&
           p.Mk >= wave::gemm_pair_tile_m() && p.Nk >= wave::gemm_pair_tile_n() && d.streamk_workers <= 1;
  // WAVE_CUDA_GEMM_KERNEL=pair|single overrides the size heuristic below (the
  // tiling knobs and shape must still allow the pair kernel).
  if (env.gemm_kernel == 1)
    p.pair = false;
  PairTailChoice tail_choice{PairTail::kWhole, 0.0};
  if (p.pair) {
    p.tile_m = wave::gemm_pair_tile_m();
    p.tile_n = wave::gemm_pair_tile_n();
    const long long num_m = (p.Mk + 255) / 256;
    const long long pairs = sms / 2;
    const int k_iters = (d.K + tile_k - 1) / tile_k;
    double rounds_wide = 0.0;
    if (sms > 0) {
      const PairWidthChoice w = pair_width_choice(num_m, p.Nk, pairs, k_iters, auto_streamk, env);
      p.tile_n = w.tile_n;
      tail_choice = w.tail;
      rounds_wide = w.cost;
    }
    const long long wide = num_m * ((p.Nk + p.tile_n - 1) / p.tile_n);
    // WAVE_CUDA_GEMM_KERNEL=pair128 forces the narrow pair tile (never chosen
    // automatically: its 256 x 128 x 16 MMAs run at 0.69 of the wide tile's rate).
    if (env.gemm_kernel == 3) {
      p.tile_n = 128;
      tail_choice = {PairTail::kWhole, 1.0};
    } else if (sms > 0 && env.gemm_kernel != 2) {
      // Choose between the pair tiles and the one-CTA kernel's 128 x 256 tiles
      // by how well each fills its rounds of tiles, weighted by the one-CTA
      // kernel's measured steady-state rate relative to the pair's.
      const long long wide256 = num_m * ((p.Nk + 255) / 256);
      const long long single = static_cast<long long>((p.Mk + 127) / 128) * ((p.Nk + 255) / 256);
      const long long r_wide = (wide + pairs - 1) / pairs, r_single = (single + sms - 1) / sms;
      const double f_wide = static_cast<double>(wide256) / (rounds_wide * static_cast<double>(pairs));
      const double f_single = kSingleRate * static_cast<double>(single) / static_cast<double>(r_single * sms);
      // A single round is all prologue and epilogue: the smaller tile's shorter tail wins there
      // (unless the pair kernel spreads that round's K iterations over every pair).
      if (f_single > f_wide || (r_wide == 1 && r_single == 1 && tail_choice.how != PairTail::kStreamK))
        p.pair = false;
    }
  }
  if (!p.pair) {
    p.tile_m = tile_m;
    p.tile_n = snap_tile_n(want_nk);
    if (p.tile_n > cap)
      p.tile_n = cap;
  }
  p.num_m = (p.Mk + p.tile_m - 1) / p.tile_m;
  p.num_n = (p.Nk + p.tile_n - 1) / p.tile_n;
  p.k_iters = (d.K + tile_k - 1) / tile_k;
  const long long tiles = static_cast<long long>(p.num_m) * p.num_n;
  const long long total_iters = tiles * p.k_iters;
  if (tiles > 0x3FFFFFFF)
    return fail(WAVE_E_INVALID, "too many output tiles");
  int workers = d.streamk_workers;
  long long dp_tiles = 0; // explicit worker counts are pure Stream-K, as in the reference
  if (workers == 0) {     // auto
    workers = 1;
    if (auto_streamk && p.pair) {
      // CTA-pair kernel: whole tiles for the full rounds, the last round's K
      // iterations dealt over all pairs when pair_tail_choice found that cheaper
      // than leaving pairs idle.
      if (tail_choice.how == PairTail::kStreamK) {
        const long long pairs = sms / 2;
        workers = static_cast<int>(pairs);
        dp_tiles = tiles - tiles % pairs;
      }
    } else if (auto_streamk && p.k_iters >= 8) {
      const long long full = tiles / sms, rem = tiles % sms;
      if (full < 2) {
        // at most one full round of tiles: split everything when the machine would be badly filled
        const long long waves = (tiles + sms - 1) / sms;
        if (static_cast<double>(tiles) / static_cast<double>(waves * sms) < 0.8 && total_iters >= sms)
          workers = sms;
      } else if (rem != 0 && rem * 4 < sms && rem * p.k_iters >= sms) {
        // several full rounds plus a nearly empty last one: whole tiles for
        // the full rounds, Stream-K only for the tail.  (With a fuller tail the
        // partial-tile traffic and the final reduction cost more than the idle
        // SMs: 4096^3 f16, 3.46 rounds, measured 1111 TFLOP/s split against
        // 1227 whole-tile.)
        workers = sms;
        dp_tiles = full * sms;
      }
    }
  }
  if (workers > 1) {
    const long long sk_iters = (tiles - dp_tiles) * p.k_iters;
    if (workers > sk_iters)
      return fail(WAVE_E_INVALID, "workers must be in [1, total_iterations]; got workers=%d, total_iterations=%lld",
                  workers, sk_iters);
    p.streamk_workers = workers;
    p.dp_tiles = static_cast<int>(dp_tiles);
    p.split_from = static_cast<int>(tiles);
    p.grid = p.pair ? 2 * workers : workers;
    // per worker two partial tiles: 128 x tile_n f32 (one CTA) or 256 x 256 (a CTA pair);
    // one arrival counter per Stream-K tile (per CTA of the pair)
    p.scratch_bytes = static_cast<size_t>(workers) * 2 * p.tile_m * (p.pair ? 256 : p.tile_n) * sizeof(float);
    p.counter_bytes = static_cast<size_t>(tiles - dp_tiles) * (p.pair ? 2 : 1) * sizeof(int);
  } else {
    p.streamk_workers = 0;
    p.dp_tiles = static_cast<int>(tiles);
    p.grid = sms > 0 ? static_cast<int>(tiles < sms ? tiles : sms) : static_cast<int>(tiles);
    p.split_from = static_cast<int>(tiles);
    if (p.pair) {
      long long items = tiles;
      if (sms > 0 && p.tile_n == 256 && tail_choice.how == PairTail::kHalfItems) {
        p.split_from = static_cast<int>(tiles - tiles % (sms / 2));
        items += tiles % (sms / 2);
      }
      const long long pairs = sms > 0 ? (items < sms / 2 ? items : sms / 2) : items;
      p.grid = static_cast<int>(2 * pairs);
    }
  }
  *plan = p;
  return WAVE_OK;
}

// ------------------------------------------------------- host staging arena
// State of the host-buffer calls, one per device ordinal: a staging arena that
// grows on demand and the three streams of the copy/compute pipeline.  A host
// call holds its device's mutex from the first copy to the last
// synchronisation, so calls on different GPUs run side by side and calls on
// one GPU take turns on its arena.
constexpr int kMaxDevices = 64;
struct HostPipeline {
  cudaStream_t h2d = nullptr, compute = nullptr, d2h = nullptr;
};
struct DeviceHostState {
  std::mutex mu;
  void *arena = nullptr;
  size_t arena_bytes = 0;
  HostPipeline pipeline;
  bool have_pipeline = false;
};
DeviceHostState g_host_state[kMaxDevices];

int host_state_for_current_device(DeviceHostState **out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess)
    return cuda_fail(err, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices)
    return fail(WAVE_E_CUDA, "device ordinal %d is outside the %d this library keeps host-call state for", dev,
                kMaxDevices);
  *out = &g_host_state[dev];
  return WAVE_OK;
}

// Caller holds st.mu and has st's device current.
int arena_reserve(DeviceHostState &st, size_t bytes, void **out) {
  if (st.arena_bytes < bytes) {
    if (st.arena)
      cudaFree(st.arena); // synchronises the device: nothing of an earlier call is still in flight on it
    st.arena = nullptr;
    st.arena_bytes = 0;
    cudaError_t err = cudaMalloc(&st.arena, bytes);
    if (err != cudaSuccess)
      return cuda_fail(err, "cudaMalloc (host-call staging)");
    st.arena_bytes = bytes;
  }
  *out = st.arena;
  return WAVE_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Streams of the host-buffer pipeline (created on the device's first large call).
HostPipeline *host_pipeline(DeviceHostState &st) {
  if (!st.have_pipeline) {
    HostPipeline hp;
    if (cudaStreamCreateWithFlags(&hp.h2d, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&hp.compute, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&hp.d2h, cudaStreamNonBlocking) != cudaSuccess) {
      for (cudaStream_t q : {hp.h2d, hp.compute, hp.d2h})
        if (q)
          cudaStreamDestroy(q);
      return nullptr;
    }
    st.pipeline = hp;
    st.have_pipeline = true;
  }
  return &st.pipeline;
}

// Columns of C per pipeline step of the host-buffer GEMM, or 0 to copy, compute
// and copy back in one piece: worth it only when the copies are large, and the
// block must keep the descriptor's tiling rules valid (a multiple of
// 16*bn*wave_n_tiles) and fill whole 256-column tiles.
int host_pipeline_chunk(const wave_gemm_desc &d, size_t copy_bytes, size_t min_bytes = 64u << 20) {
  if (copy_bytes < min_bytes || is_tile_packed(d.out_layout) || d.ldc != 0 || d.streamk_workers > 1)
    return 0;
  const int unit = 16 * d.bn * d.wave_n_tiles;
  for (int parts : {8, 6, 4, 3, 2}) {
    if (d.N % parts)
      continue;
    const int chunk = d.N / parts;
    if (chunk % unit == 0 && chunk % 256 == 0 && chunk >= 512)
      return chunk;
  }
  return 0;
}

struct FnHandle {
  int kind; // 0 gemm, 1 stream-K gemm, 2 flash attention
  wave_gemm_desc gemm;
  wave_fa_desc fa;
};

struct MemRef1D {
  void *base;
  char *data;
  int64_t offset;
  int64_t size;
  int64_t stride;
};
template <int ElemBytes> void *memref_ptr(void *m) {
  MemRef1D *d = static_cast<MemRef1D *>(m);
  return d->data + d->offset * ElemBytes;
}

} // namespace

extern "C" {

const char *wave_cuda_last_error(void) { return g_last_error.c_str(); }
const char *wave_cuda_version(void) { return "wave_cuda sm_100a 0.2"; }
void wave_cuda_reload_env(void) { wave::reload_env_knobs(); }

// runtime/wave_runtime.cpp:35-40, 46-74: data + offset (in elements).
void *_mlir_ciface_wave_memref_to_ptr_global_i32(void *m) { return memref_ptr<4>(m); }
void *_mlir_ciface_wave_memref_to_ptr_global_i8(void *m) { return memref_ptr<1>(m); }
void *_mlir_ciface_wave_memref_to_ptr_global_f32(void *m) { return memref_ptr<4>(m); }
void *_mlir_ciface_wave_memref_to_ptr_global_f16(void *m) { return memref_ptr<2>(m); }
void *_mlir_ciface_wave_memref_to_ptr_global_bf16(void *m) { return memref_ptr<2>(m); }
void *_mlir_ciface_wave_memref_to_ptr_global_i64(void *m) { return memref_ptr<8>(m); }
void *_mlir_ciface_wave_memref_to_ptr_global_f64(void *m) { return memref_ptr<8>(m); }

void wave_cuda_gemm_desc_init(wave_gemm_desc *d, int M, int N, int K) {
  memset(d, 0, sizeof *d);
  d->M = M;
  d->N = N;
  d->K = K;
  d->bm = 1;
  d->bn = 2;
  d->wave_m_tiles = d->wave_n_tiles = d->wave_k_tiles = 1;
  d->in_type = WAVE_F16;
  d->out_type = WAVE_F32;
  d->out_layout = WAVE_ROW_MAJOR;
  d->cta_group_m = 1;
  d->streamk_workers = 1;
  d->ldc = 0;
}

int wave_cuda_gemm_validate(const wave_gemm_desc *d) {
  if (!d)
    return fail(WAVE_E_INVALID, "descriptor is null");
  // wave_matmul.py:533-536
  const int dims[3] = {d->M, d->N, d->K};
  const char *names[3] = {"M", "N", "K"};
  for (int i = 0; i < 3; ++i)
    if (dims[i] <= 0 || dims[i] % 16 != 0)
      return fail(WAVE_E_INVALID, "%s must be a positive multiple of 16; got %d", names[i], dims[i]);
  // wave_matmul.py:537-538
  if (d->bm < 1 || d->bn < 1)
    return fail(WAVE_E_INVALID, "BM and BN must be >= 1; got BM=%d, BN=%d", d->bm, d->bn);
  // wave_matmul.py:556-560
  if (d->cta_group_m < 1)
    return fail(WAVE_E_INVALID, "cta_group_m must be >= 1; got %d", d->cta_group_m);
  // wave_matmul.py:563-570
  if (d->wave_m_tiles < 1 || d->wave_n_tiles < 1 || d->wave_k_tiles < 1)
    return fail(WAVE_E_INVALID,
                "wave_m_tiles, wave_n_tiles and wave_k_tiles must be >= 1; got wave_m_tiles=%d, "
                "wave_n_tiles=%d, wave_k_tiles=%d",
                d->wave_m_tiles, d->wave_n_tiles, d->wave_k_tiles);
  if (d->out_type != WAVE_F32 && d->out_type != WAVE_F16 && d->out_type != WAVE_BF16)
    return fail(WAVE_E_INVALID, "output_type must be one of f32, f16, bf16; got %d", d->out_type);
  if (d->out_layout != WAVE_ROW_MAJOR && d->out_layout != WAVE_COL_MAJOR && !is_tile_packed(d->out_layout))
    return fail(WAVE_E_INVALID, "output_layout must be one of row-major, column-major, tile-packed; got %d",
                d->out_layout);
  if (d->in_type != WAVE_F16 && d->in_type != WAVE_BF16)
    return fail(WAVE_E_UNSUPPORTED, "input_type must be one of f16, bf16; got %d (mxfp4 is outside this backend)",
                d->in_type);
  // wave_matmul.py:575-579
  if (!is_pow2(d->bn))
    return fail(WAVE_E_INVALID,
                "BN must be a positive power of two (for the wave-id decomposition); got BN=%d", d->bn);
  // wave_matmul.py:580-591
  const int m_tiles = d->bm * d->wave_m_tiles, n_tiles = d->bn * d->wave_n_tiles;
  if ((d->M / 16) % m_tiles != 0)
    return fail(WAVE_E_INVALID, "BM * wave_m_tiles (=%d) must divide M/16 (=%d)", m_tiles, d->M / 16);
  if ((d->N / 16) % n_tiles != 0)
    return fail(WAVE_E_INVALID, "BN * wave_n_tiles (=%d) must divide N/16 (=%d)", n_tiles, d->N / 16);
  // wave_matmul.py:597-601 with k_tile = 16
  if ((d->K / 16) % d->wave_k_tiles != 0)
    return fail(WAVE_E_INVALID, "wave_k_tiles (=%d) must divide K/16 (=%d)", d->wave_k_tiles, d->K / 16);
  // wave_matmul.py:603-607
  if (d->bm * d->bn > 32)
    return fail(WAVE_E_INVALID, "BM * BN must be <= 32 (RDNA3 workgroup wave cap); got BM=%d, BN=%d (product=%d)",
                d->bm, d->bn, d->bm * d->bn);
  // wave_matmul.py:615-619
  const int m_blocks = (d->M / 16) / m_tiles;
  if (m_blocks % d->cta_group_m != 0)
    return fail(WAVE_E_INVALID,
                "cta_group_m currently requires M_blocks to divide evenly; got M_blocks=%d, cta_group_m=%d",
                m_blocks, d->cta_group_m);
  if (d->streamk_workers < 0)
    return fail(WAVE_E_INVALID, "streamk_workers must be >= 0; got %d", d->streamk_workers);
  if (is_tile_packed(d->out_layout) && d->ldc != 0)
    return fail(WAVE_E_INVALID, "ldc must be 0 with tile-packed output; got %d", d->ldc);
  const int min_ld = d->out_layout == WAVE_ROW_MAJOR ? d->N : d->M;
  if (d->ldc != 0 && (d->ldc < min_ld || d->ldc % 16 != 0))
    return fail(WAVE_E_INVALID, "ldc must be 0 or a multiple of 16 that is >= %d; got %d", min_ld, d->ldc);
  return WAVE_OK;
}

int wave_cuda_gemm_workspace_bytes(const wave_gemm_desc *d, size_t *scratch_bytes, size_t *counter_bytes) {
  int rc = wave_cuda_gemm_validate(d);
  if (rc != WAVE_OK)
    return rc;
  int sms = -1;
  if (d->streamk_workers == 0 && (rc = sm_count(&sms)) != WAVE_OK)
    return rc;
  GemmPlan plan;
  if ((rc = make_plan(*d, sms, true, &plan)) != WAVE_OK)
    return rc;
  if (scratch_bytes)
    *scratch_bytes = plan.scratch_bytes;
  if (counter_bytes)
    *counter_bytes = plan.counter_bytes;
  return WAVE_OK;
}

int wave_cuda_gemm_plan_for_sms(const wave_gemm_desc *d, int sm_count, int have_workspace, int *tile_m, int *tile_n,
                                int *grid, int *streamk_workers, int *swapped, size_t *scratch_bytes,
                                size_t *counter_bytes) {
  int rc = wave_cuda_gemm_validate(d);
  if (rc != WAVE_OK)
    return rc;
  if (sm_count < 2)
    return fail(WAVE_E_INVALID, "sm_count must be at least 2; got %d", sm_count);
  GemmPlan plan;
  if ((rc = make_plan(*d, sm_count, have_workspace != 0, &plan)) != WAVE_OK)
    return rc;
  if (tile_m)
    *tile_m = plan.tile_m;
  if (tile_n)
    *tile_n = plan.tile_n;
  if (grid)
    *grid = plan.grid;
  if (streamk_workers)
    *streamk_workers = plan.streamk_workers;
  if (swapped)
    *swapped = plan.swapped ? 1 : 0;
  if (scratch_bytes)
    *scratch_bytes = plan.scratch_bytes;
  if (counter_bytes)
    *counter_bytes = plan.counter_bytes;
  return WAVE_OK;
}

int wave_cuda_gemm_plan(const wave_gemm_desc *d, int *tile_m, int *tile_n, int *grid, int *streamk_workers,
                        int *swapped) {
  int rc = wave_cuda_gemm_validate(d);
  if (rc != WAVE_OK)
    return rc;
  int sms = 0;
  if ((rc = sm_count(&sms)) != WAVE_OK)
    return rc;
  GemmPlan plan;
  if ((rc = make_plan(*d, sms, true, &plan)) != WAVE_OK)
    return rc;
  if (tile_m)
    *tile_m = plan.tile_m;
  if (tile_n)
    *tile_n = plan.tile_n;
  if (grid)
    *grid = plan.grid;
  if (streamk_workers)
    *streamk_workers = plan.streamk_workers;
  if (swapped)
    *swapped = plan.swapped ? 1 : 0;
  return WAVE_OK;
}

} // extern "C"

namespace {
int gemm_launch(const wave_gemm_desc *d, const void *A, const void *B, void *C, void *workspace, void *stream,
                void *const *extra_c, int n_extra, bool extra_multimem = false);
}

extern "C" {

int wave_cuda_gemm(const wave_gemm_desc *d, const void *A, const void *B, void *C, void *workspace,
                   void *stream) {
  return gemm_launch(d, A, B, C, workspace, stream, nullptr, 0);
}

int wave_cuda_gemm_multi_output(const wave_gemm_desc *d, const void *A, const void *B, void *const *C_targets,
                                int n_targets, void *stream) {
  if (!C_targets || n_targets < 1 || n_targets > 8)
    return fail(WAVE_E_INVALID, "n_targets must be between 1 and 8; got %d", n_targets);
  for (int i = 0; i < n_targets; ++i)
    if (!C_targets[i] || (reinterpret_cast<uintptr_t>(C_targets[i]) & 15))
      return fail(WAVE_E_INVALID, "every output target must be a non-null, 16-byte aligned device pointer");
  return gemm_launch(d, A, B, C_targets[0], nullptr, stream, C_targets + 1, n_targets - 1);
}

int wave_cuda_gemm_multicast_output(const wave_gemm_desc *d, const void *A, const void *B, void *C_local,
                                    void *C_multicast, void *stream) {
  if (!C_multicast || (reinterpret_cast<uintptr_t>(C_multicast) & 15))
    return fail(WAVE_E_INVALID, "the multicast target must be a non-null, 16-byte aligned address");
  void *const extra[1] = {C_multicast};
  return gemm_launch(d, A, B, C_local, nullptr, stream, extra, 1, true);
}

} // extern "C"

namespace {

int gemm_launch(const wave_gemm_desc *d, const void *A, const void *B, void *C, void *workspace, void *stream,
                void *const *extra_c, int n_extra, bool extra_multimem) {
  int rc = wave_cuda_gemm_validate(d);
  if (rc != WAVE_OK)
    return rc;
  if (!A || !B || !C)
    return fail(WAVE_E_INVALID, "A, B and C must be non-null device pointers");
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15)
    return fail(WAVE_E_INVALID, "A, B and C must be 16-byte aligned");
  int sms = 0;
  if ((rc = sm_count(&sms)) != WAVE_OK)
    return rc;
  GemmPlan plan;
  if ((rc = make_plan(*d, sms, workspace != nullptr, &plan, n_extra > 0)) != WAVE_OK)
    return rc;
  if (plan.streamk_workers > 0 && !workspace)
    return fail(WAVE_E_INVALID, "Stream-K with %d workers needs a workspace of %zu + %zu bytes",
                plan.streamk_workers, plan.scratch_bytes, plan.counter_bytes);

  const int tile_m = wave::gemm_tile_m(), tile_k = wave::gemm_tile_k();
  const void *Ak = plan.swapped ? B : A;
  const void *Bk = plan.swapped ? A : B;
  CUtensorMap ta, tb, tbh;
  const int bf16 = d->in_type == WAVE_BF16;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(d->K), static_cast<uint64_t>(plan.Mk)};
    const uint64_t strides[1] = {static_cast<uint64_t>(d->K) * 2};
    const uint32_t box[2] = {static_cast<uint32_t>(tile_k),
                             static_cast<uint32_t>(plan.pair ? wave::gemm_pair_box_rows() : tile_m)};
    if ((rc = wave::make_tensor_map_16bit(&ta, bf16, Ak, 2, dims, strides, box)) != WAVE_OK)
      return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(d->K), static_cast<uint64_t>(plan.Nk)};
    const uint64_t strides[1] = {static_cast<uint64_t>(d->K) * 2};
    const uint32_t box[2] = {static_cast<uint32_t>(tile_k),
                             static_cast<uint32_t>(plan.pair ? plan.tile_n / 2 : plan.tile_n)};
    if ((rc = wave::make_tensor_map_16bit(&tb, bf16, Bk, 2, dims, strides, box)) != WAVE_OK)
      return rc;
    tbh = tb;
    if (plan.pair && plan.split_from < plan.num_m * plan.num_n) {
      const uint32_t half_box[2] = {static_cast<uint32_t>(tile_k), static_cast<uint32_t>(plan.tile_n / 4)};
      if ((rc = wave::make_tensor_map_16bit(&tbh, bf16, Bk, 2, dims, strides, half_box)) != WAVE_OK)
        return rc;
    }
  }

  wave::GemmParams p{};
  p.M = plan.Mk;
  p.N = plan.Nk;
  p.K = d->K;
  p.C = C;
  const long long ld = d->ldc ? d->ldc : (d->out_layout == WAVE_ROW_MAJOR ? d->N : d->M);
  // caller-space strides of C[m][n]
  long long sm = d->out_layout == WAVE_ROW_MAJOR ? ld : 1;
  long long sn = d->out_layout == WAVE_ROW_MAJOR ? 1 : ld;
  p.stride_m = plan.swapped ? sn : sm; // kernel rows are the caller's n when swapped
  p.stride_n = plan.swapped ? sm : sn;
  p.in_type = bf16 ? WAVE_GEMM_IN_BF16 : WAVE_GEMM_IN_F16;
  p.out_type = d->out_type == WAVE_F32 ? WAVE_GEMM_OUT_F32 : d->out_type == WAVE_F16 ? WAVE_GEMM_OUT_F16
                                                                                       : WAVE_GEMM_OUT_BF16;
  p.num_m_blocks = plan.num_m;
  p.num_n_blocks = plan.num_n;
  p.num_tiles = plan.num_m * plan.num_n;
  p.k_iters = plan.k_iters;
  p.split_from = plan.split_from;
  // The descriptor's cta_group_m counts the reference's (smaller) workgroup
  // tiles; keep the same number of rows per group, at least one row block.
  {
    const int wg_rows = plan.swapped ? 16 * d->bn * d->wave_n_tiles : 16 * d->bm * d->wave_m_tiles;
    long long rows = static_cast<long long>(d->cta_group_m) * wg_rows;
    int g = static_cast<int>(rows / plan.tile_m);
    if (d->cta_group_m == 1)
      g = 2048 / plan.tile_m; // the reference's "no grouping" default: use the backend's own
    if (g < 1)
      g = 1;
    if (g > plan.num_m)
      g = plan.num_m;
    p.group_m = g;
  }
  if (is_tile_packed(d->out_layout)) {
    p.tile_packed = 1;
    p.tp_fragment = d->out_layout - WAVE_TILE_PACKED; // 0 row-major tiles, 1 MFMA wave64, 2 WMMA wave32, 3 MFMA wave32
    p.tp_bm = d->bm;
    p.tp_bn = d->bn;
    p.tp_wmt = d->wave_m_tiles;
    p.tp_wnt = d->wave_n_tiles;
    p.tp_n_blocks = (d->N / 16) / (d->bn * d->wave_n_tiles);
  }
#ifdef WAVE_WAIT_TEST
  if (const char *v = getenv("WAVE_CUDA_TEST_SKIP_LAST_K")) // test builds only; read on every launch
    p.test_skip_last_k = strcmp(v, "1") == 0 ? 1 : 0;
#endif
  p.streamk_workers = plan.streamk_workers;
  p.dp_tiles = plan.dp_tiles;
  p.scratch = static_cast<float *>(workspace);
  p.counters = workspace ? reinterpret_cast<int *>(static_cast<char *>(workspace) + plan.scratch_bytes) : nullptr;

  // 16-bit output whose kernel-space rows are contiguous (row-major C, or
  // column-major C computed as C^T) leaves whole tiles of at least 64 columns
  // through TMA stores (WAVE_CUDA_GEMM_TMA_STORE=0 keeps the per-thread stores,
  // for measurements).
  const wave::EnvKnobs env = wave::env_knobs();
  p.l2_hints = env.gemm_l2_hints;
  p.pdl = env.gemm_pdl ? 1 : 0;
  CUtensorMap tc = ta;
  if ((plan.pair || plan.tile_n >= 64) && p.stride_n == 1 && !p.tile_packed && d->out_type != WAVE_F32 &&
      plan.Nk >= 64 && env.gemm_tma_store) {
    const uint64_t dims[2] = {static_cast<uint64_t>(plan.Nk), static_cast<uint64_t>(plan.Mk)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ld) * 2};
    const uint32_t box[2] = {64, static_cast<uint32_t>(wave::gemm_pair_box_rows())};
    if ((rc = wave::make_tensor_map_16bit(&tc, d->out_type == WAVE_BF16, C, 2, dims, strides, box)) != WAVE_OK)
      return rc;
    p.c_tma = 1;
  }
  if (n_extra > 0) {
    // Further copies of C are written from the TMA-store epilogue of the CTA-pair kernel only.
    if (!plan.pair || !p.c_tma || plan.streamk_workers > 0)
      return fail(WAVE_E_UNSUPPORTED,
                  "several output targets need the CTA-pair kernel's TMA-store epilogue: 16-bit C, row-major or "
                  "column-major, M and N of at least 256 and tiling knobs asking for 256 x 256 tiles");
    p.n_extra = n_extra;
    p.extra_multimem = extra_multimem ? 1 : 0;
    for (int i = 0; i < n_extra; ++i)
      p.extra_c[i] = extra_c[i];
  }
  // Plain further targets (peer GPUs' copies of C) get a tensor map each: the
  // kernel sends them every finished piece with one more TMA store.
  CUtensorMap extra_maps[7];
  const bool tma_extra = n_extra > 0 && !extra_multimem;
  if (tma_extra) {
    const uint64_t dims[2] = {static_cast<uint64_t>(plan.Nk), static_cast<uint64_t>(plan.Mk)};
    const uint64_t strides[1] = {static_cast<uint64_t>(ld) * 2};
    const uint32_t box[2] = {64, static_cast<uint32_t>(wave::gemm_pair_box_rows())};
    for (int i = 0; i < n_extra; ++i)
      if ((rc = wave::make_tensor_map_16bit(&extra_maps[i], d->out_type == WAVE_BF16, extra_c[i], 2, dims, strides, box)) !=
          WAVE_OK)
        return rc;
  }
  cudaError_t err = plan.pair ? wave::launch_gemm_pair(ta, tb, tbh, tc, p, tma_extra ? extra_maps : nullptr, plan.tile_n,
                                                       plan.grid, static_cast<cudaStream_t>(stream))
                              : wave::launch_gemm(ta, tb, tc, p, plan.tile_n, plan.grid, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess)
    return cuda_fail(err, "gemm launch");
  return WAVE_OK;
}

// Host-buffer GEMM.  `A` is a host pointer, or with `a_on_device` a device
// pointer whose contents are ready on `stream` (a rank of a sharded problem
// receives the replicated A over NVLink rather than once more over PCIe).
int gemm_host_impl(const wave_gemm_desc *d, const void *A, bool a_on_device, const void *B_host, void *C_host,
                   void *stream) {
  const void *A_host = A;
  int rc = wave_cuda_gemm_validate(d);
  if (rc != WAVE_OK)
    return rc;
  if (!A || !B_host || !C_host)
    return fail(WAVE_E_INVALID, "A, B and C must be non-null pointers");
  if (a_on_device && (reinterpret_cast<uintptr_t>(A) & 15))
    return fail(WAVE_E_INVALID, "a device-resident A must be 16-byte aligned");
  size_t scratch = 0, counters = 0;
  if ((rc = wave_cuda_gemm_workspace_bytes(d, &scratch, &counters)) != WAVE_OK)
    return rc;
  const size_t a_bytes = a_on_device ? 0 : static_cast<size_t>(d->M) * d->K * 2;
  const size_t b_bytes = static_cast<size_t>(d->N) * d->K * 2;
  const size_t ld = d->ldc ? d->ldc : (d->out_layout == WAVE_ROW_MAJOR ? d->N : d->M);
  const size_t c_bytes = ld * (d->out_layout == WAVE_ROW_MAJOR ? d->M : d->N) * elem_size(d->out_type);
  const size_t off_b = align_up(a_bytes, 256), off_c = off_b + align_up(b_bytes, 256);
  const size_t off_ws = off_c + align_up(c_bytes, 256);
  const size_t total = off_ws + align_up(scratch, 256) + align_up(counters, 256);
  DeviceHostState *state = nullptr;
  if ((rc = host_state_for_current_device(&state)) != WAVE_OK)
    return rc;
  std::lock_guard<std::mutex> lock(state->mu);
  void *base = nullptr;
  if ((rc = arena_reserve(*state, total, &base)) != WAVE_OK)
    return rc;
  char *dev = static_cast<char *>(base);
  const char *a_dev = a_on_device ? static_cast<const char *>(A) : dev;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err;

  // Large problems are pipelined by column blocks of C: while block i is
  // being computed, block i+1 of B is on its way to the device and block i-1
  // of C on its way back (PCIe is full duplex), so the call costs about
  // "copy A + copy B" instead of "copy A + copy B + compute + copy C".
  // (With A already on the device -- a rank's block of a sharded problem -- the
  // copies are smaller and the pipeline pays from 16 MB on: B can start on its
  // way while the caller's stream is still producing A.)
  const int chunk = host_pipeline_chunk(*d, b_bytes + c_bytes, a_on_device ? (16u << 20) : (64u << 20));
  if (chunk > 0) {
    HostPipeline *hp = host_pipeline(*state);
    if (!hp)
      return fail(WAVE_E_CUDA, "could not create the streams of the host-call pipeline");
    const int nchunks = d->N / chunk;
    const size_t es = elem_size(d->out_type);
    std::vector<cudaEvent_t> ev(2 * nchunks + 2, nullptr);
    bool failed = false;
    auto check = [&](cudaError_t e, const char *what) {
      if (e != cudaSuccess && !failed) {
        failed = true;
        cuda_fail(e, what);
      }
    };
    for (cudaEvent_t &e : ev)
      check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "create event");
    cudaEvent_t ev_start = ev[2 * nchunks], ev_a = ev[2 * nchunks + 1];
    if (!failed) {
      check(cudaEventRecord(ev_start, s), "record");
      for (cudaStream_t q : {hp->h2d, hp->compute, hp->d2h})
        if (!(a_on_device && q == hp->h2d)) // B comes from the host: it need not wait for the caller's A
          check(cudaStreamWaitEvent(q, ev_start, 0), "order after the caller's stream");
      if (!a_on_device)
        check(cudaMemcpyAsync(dev, A_host, a_bytes, cudaMemcpyHostToDevice, hp->h2d), "copy A to device");
      check(cudaEventRecord(ev_a, hp->h2d), "record");
      check(cudaStreamWaitEvent(hp->compute, ev_a, 0), "wait for A");
      wave_gemm_desc sub = *d;
      sub.N = chunk;
      sub.streamk_workers = 1;
      sub.ldc = d->out_layout == WAVE_ROW_MAJOR ? d->N : d->M;
      for (int i = 0; i < nchunks && !failed; ++i) {
        const size_t b_off = static_cast<size_t>(i) * chunk * d->K * 2;
        check(cudaMemcpyAsync(dev + off_b + b_off, static_cast<const char *>(B_host) + b_off,
                              static_cast<size_t>(chunk) * d->K * 2, cudaMemcpyHostToDevice, hp->h2d),
              "copy a block of B to device");
        check(cudaEventRecord(ev[2 * i], hp->h2d), "record");
        check(cudaStreamWaitEvent(hp->compute, ev[2 * i], 0), "wait for a block of B");
        const size_t c_off = d->out_layout == WAVE_ROW_MAJOR ? static_cast<size_t>(i) * chunk * es
                                                             : static_cast<size_t>(i) * chunk * d->M * es;
        if (!failed && wave_cuda_gemm(&sub, a_dev, dev + off_b + b_off, dev + off_c + c_off, nullptr, hp->compute) != WAVE_OK)
          failed = true; // message already recorded
        check(cudaEventRecord(ev[2 * i + 1], hp->compute), "record");
        check(cudaStreamWaitEvent(hp->d2h, ev[2 * i + 1], 0), "wait for a block of C");
        if (d->out_layout == WAVE_ROW_MAJOR)
          check(cudaMemcpy2DAsync(static_cast<char *>(C_host) + c_off, static_cast<size_t>(d->N) * es,
                                  dev + off_c + c_off, static_cast<size_t>(d->N) * es, static_cast<size_t>(chunk) * es,
                                  static_cast<size_t>(d->M), cudaMemcpyDeviceToHost, hp->d2h),
                "copy a block of C to host");
        else
          check(cudaMemcpyAsync(static_cast<char *>(C_host) + c_off, dev + off_c + c_off,
                                static_cast<size_t>(chunk) * d->M * es, cudaMemcpyDeviceToHost, hp->d2h),
                "copy a block of C to host");
      }
    }
    for (cudaStream_t q : {hp->h2d, hp->compute, hp->d2h})
      check(cudaStreamSynchronize(q), "synchronise the host-call pipeline");
    for (cudaEvent_t e : ev)
      if (e)
        cudaEventDestroy(e);
    return failed ? WAVE_E_CUDA : WAVE_OK;
  }

  // One piece: copy, compute, copy back on the caller's stream.  Whatever
  // fails, the stream is drained before the arena is given up to the next call.
  rc = WAVE_OK;
  auto step = [&](cudaError_t e, const char *what) {
    if (rc == WAVE_OK && e != cudaSuccess)
      rc = cuda_fail(e, what);
    return rc == WAVE_OK;
  };
  void *ws = nullptr;
  if ((a_on_device || step(cudaMemcpyAsync(dev, A_host, a_bytes, cudaMemcpyHostToDevice, s), "copy A to device")) &&
      step(cudaMemcpyAsync(dev + off_b, B_host, b_bytes, cudaMemcpyHostToDevice, s), "copy B to device")) {
    if (scratch + counters > 0) {
      ws = dev + off_ws;
      step(cudaMemsetAsync(dev + off_ws + scratch, 0, counters, s), "clear Stream-K counters");
    }
    if (rc == WAVE_OK)
      rc = wave_cuda_gemm(d, a_dev, dev + off_b, dev + off_c, ws, stream);
    if (rc == WAVE_OK)
      step(cudaMemcpyAsync(C_host, dev + off_c, c_bytes, cudaMemcpyDeviceToHost, s), "copy C to host");
  }
  err = cudaStreamSynchronize(s);
  if (rc == WAVE_OK && err != cudaSuccess)
    rc = cuda_fail(err, "synchronise after GEMM");
  return rc;
}

} // namespace

extern "C" {

int wave_cuda_gemm_host(const wave_gemm_desc *d, const void *A_host, const void *B_host, void *C_host,
                        void *stream) {
  return gemm_host_impl(d, A_host, false, B_host, C_host, stream);
}

int wave_cuda_gemm_host_a_resident(const wave_gemm_desc *d, const void *A_device, const void *B_host, void *C_host,
                                   void *stream) {
  return gemm_host_impl(d, A_device, true, B_host, C_host, stream);
}

// ------------------------------------------------------------ flash attention
// log2(e) * head_dim * scale * qk_max_abs^2: the largest scaled score, in log2
// units, that entries bounded by qk_max_abs can give (amd_fa_wave.py:1599-1601;
// with the default scale this is the log2(e) * sqrt(128) * qk_max_abs^2 of
// wave_flash_attention.py:108-113).
static double fa_log2_score_bound(const wave_fa_desc &d) {
  const double scale = d.scale > 0.0f ? static_cast<double>(d.scale) : 1.0 / std::sqrt(static_cast<double>(d.head_dim));
  return 1.4426950408889634 * d.head_dim * scale * static_cast<double>(d.qk_max_abs) * static_cast<double>(d.qk_max_abs);
}

int wave_cuda_fa_validate(const wave_fa_desc *d) {
  if (!d)
    return fail(WAVE_E_INVALID, "descriptor is null");
  if (d->batch <= 0 || d->heads <= 0)
    return fail(WAVE_E_INVALID, "batch and heads must be positive; got batch=%d, heads=%d", d->batch, d->heads);
  if (d->seq_q <= 0 || d->seq_k <= 0 || d->seq_q % 16 != 0 || d->seq_k % 16 != 0)
    return fail(WAVE_E_INVALID, "sequence lengths must be positive multiples of 16; got seq_q=%d, seq_k=%d",
                d->seq_q, d->seq_k);
  if (d->head_dim < 16 || d->head_dim > 128 || d->head_dim % 16 != 0)
    return fail(WAVE_E_UNSUPPORTED, "head_dim must be a multiple of 16 between 16 and 128; got %d", d->head_dim);
  if (d->io_type != WAVE_BF16 && d->io_type != WAVE_F16)
    return fail(WAVE_E_UNSUPPORTED, "io_type must be bf16 or f16; got %d", d->io_type);
  if (d->causal && d->seq_q != d->seq_k)
    return fail(WAVE_E_UNSUPPORTED, "causal attention requires seq_q == seq_k; got %d and %d", d->seq_q, d->seq_k);
  if (!(d->scale >= 0.0f) || std::isinf(d->scale))
    return fail(WAVE_E_INVALID, "scale must be finite and >= 0 (0 selects 1/sqrt(head_dim))");
  if (d->qk_max_abs != 0.0f) {
    // wave_flash_attention.py:64-75, amd_fa_wave.py:1592-1610
    if (!(d->qk_max_abs > 0.0f) || std::isinf(d->qk_max_abs))
      return fail(WAVE_E_INVALID, "qk_max_abs must be finite and positive; got %g", static_cast<double>(d->qk_max_abs));
    if (2.0 * fa_log2_score_bound(*d) >= 126.0)
      return fail(WAVE_E_INVALID, "qk_max_abs fixed reference exceeds BF16 range; use adaptive reference");
  }
  return WAVE_OK;
}

} // extern "C"

namespace {
int fa_launch(const wave_fa_desc *d, const void *Q, const void *K, const void *V, void *O, float *lse, void *stream,
              void *const *extra_o, int n_extra, bool extra_multimem);
}

extern "C" {

int wave_cuda_flash_attention_fwd(const wave_fa_desc *d, const void *Q, const void *K, const void *V, void *O,
                                  float *lse, void *stream) {
  return fa_launch(d, Q, K, V, O, lse, stream, nullptr, 0, false);
}

int wave_cuda_flash_attention_fwd_multi_output(const wave_fa_desc *d, const void *Q, const void *K, const void *V,
                                               void *const *O_targets, int n_targets, float *lse, void *stream) {
  if (!O_targets || n_targets < 1 || n_targets > 8)
    return fail(WAVE_E_INVALID, "n_targets must be between 1 and 8; got %d", n_targets);
  for (int i = 0; i < n_targets; ++i)
    if (!O_targets[i] || (reinterpret_cast<uintptr_t>(O_targets[i]) & 15))
      return fail(WAVE_E_INVALID, "every output target must be a non-null, 16-byte aligned device pointer");
  return fa_launch(d, Q, K, V, O_targets[0], lse, stream, O_targets + 1, n_targets - 1, false);
}

int wave_cuda_flash_attention_fwd_multicast_output(const wave_fa_desc *d, const void *Q, const void *K, const void *V,
                                                   void *O_local, void *O_multicast, float *lse, void *stream) {
  if (!O_multicast || (reinterpret_cast<uintptr_t>(O_multicast) & 15))
    return fail(WAVE_E_INVALID, "the multicast target must be a non-null, 16-byte aligned address");
  void *const extra[1] = {O_multicast};
  return fa_launch(d, Q, K, V, O_local, lse, stream, extra, 1, true);
}

} // extern "C"

namespace {

int fa_launch(const wave_fa_desc *d, const void *Q, const void *K, const void *V, void *O, float *lse, void *stream,
              void *const *extra_o, int n_extra, bool extra_multimem) {
  int rc = wave_cuda_fa_validate(d);
  if (rc != WAVE_OK)
    return rc;
  if (!Q || !K || !V || !O)
    return fail(WAVE_E_INVALID, "Q, K, V and O must be non-null device pointers");
  if ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V) |
       reinterpret_cast<uintptr_t>(O)) & 15)
    return fail(WAVE_E_INVALID, "Q, K, V and O must be 16-byte aligned");
  wave::FaParams p{};
  p.batch_heads = d->batch * d->heads;
  p.seq_q = d->seq_q;
  p.seq_k = d->seq_k;
  p.head_dim = d->head_dim;
  p.causal = d->causal ? 1 : 0;
  p.is_bf16 = d->io_type == WAVE_BF16;
  p.out_f32 = d->out_f32 ? 1 : 0;
  const double scale = d->scale > 0.0f ? static_cast<double>(d->scale) : 1.0 / std::sqrt(static_cast<double>(d->head_dim));
  p.scale = static_cast<float>(scale);
  p.scale_log2e = static_cast<float>(scale * 1.4426950408889634);
  p.fixed_ref = d->qk_max_abs > 0.0f ? 1 : 0;
  p.ref_log2 = p.fixed_ref ? static_cast<float>(fa_log2_score_bound(*d)) : 0.0f;
  p.O = O;
  p.lse = lse;
  wave::FaExtra extra{};
  extra.n = n_extra;
  extra.multimem = extra_multimem ? 1 : 0;
  for (int i = 0; i < n_extra; ++i)
    extra.o[i] = extra_o[i];
  int sms = 0;
  if ((rc = sm_count(&sms)) != WAVE_OK)
    return rc;
  rc = wave::launch_flash_attention(p, extra, Q, K, V, sms, static_cast<cudaStream_t>(stream));
  return rc;
}

} // namespace

extern "C" {

int wave_cuda_flash_attention_fwd_host(const wave_fa_desc *d, const void *Q_host, const void *K_host,
                                       const void *V_host, void *O_host, void *stream) {
  int rc = wave_cuda_fa_validate(d);
  if (rc != WAVE_OK)
    return rc;
  if (!Q_host || !K_host || !V_host || !O_host)
    return fail(WAVE_E_INVALID, "Q, K, V and O must be non-null host pointers");
  const size_t bh = static_cast<size_t>(d->batch) * d->heads;
  const size_t q_bytes = bh * d->seq_q * d->head_dim * 2, kv_bytes = bh * d->seq_k * d->head_dim * 2;
  const size_t off_k = align_up(q_bytes, 256), off_v = off_k + align_up(kv_bytes, 256);
  const size_t o_bytes = d->out_f32 ? 2 * q_bytes : q_bytes;
  const size_t off_o = off_v + align_up(kv_bytes, 256), total = off_o + align_up(o_bytes, 256);
  DeviceHostState *state = nullptr;
  if ((rc = host_state_for_current_device(&state)) != WAVE_OK)
    return rc;
  std::lock_guard<std::mutex> lock(state->mu);
  void *base = nullptr;
  if ((rc = arena_reserve(*state, total, &base)) != WAVE_OK)
    return rc;
  char *dev = static_cast<char *>(base);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err;

  // Large calls are pipelined by groups of heads (contiguous slabs of Q, K, V
  // and O): the next group's inputs and the previous group's output travel
  // while the current group is computed.
  int parts = 0;
  if (q_bytes + 2 * kv_bytes >= (64u << 20))
    for (int cand : {8, 4, 2})
      if (bh % cand == 0 && bh / cand >= 8) {
        parts = cand;
        break;
      }
  if (parts > 0) {
    HostPipeline *hp = host_pipeline(*state);
    if (!hp)
      return fail(WAVE_E_CUDA, "could not create the streams of the host-call pipeline");
    const size_t group = bh / parts;
    const size_t q_step = q_bytes / parts, kv_step = kv_bytes / parts, o_step = o_bytes / parts;
    std::vector<cudaEvent_t> ev(2 * parts + 1, nullptr);
    bool failed = false;
    auto check = [&](cudaError_t e, const char *what) {
      if (e != cudaSuccess && !failed) {
        failed = true;
        cuda_fail(e, what);
      }
    };
    for (cudaEvent_t &e : ev)
      check(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "create event");
    if (!failed) {
      check(cudaEventRecord(ev[2 * parts], s), "record");
      for (cudaStream_t q : {hp->h2d, hp->compute, hp->d2h})
        check(cudaStreamWaitEvent(q, ev[2 * parts], 0), "order after the caller's stream");
      wave_fa_desc sub = *d;
      sub.batch = 1;
      sub.heads = static_cast<int>(group);
      for (int i = 0; i < parts && !failed; ++i) {
        const char *qh = static_cast<const char *>(Q_host) + i * q_step;
        const char *kh = static_cast<const char *>(K_host) + i * kv_step;
        const char *vh = static_cast<const char *>(V_host) + i * kv_step;
        check(cudaMemcpyAsync(dev + i * q_step, qh, q_step, cudaMemcpyHostToDevice, hp->h2d), "copy Q to device");
        check(cudaMemcpyAsync(dev + off_k + i * kv_step, kh, kv_step, cudaMemcpyHostToDevice, hp->h2d), "copy K to device");
        check(cudaMemcpyAsync(dev + off_v + i * kv_step, vh, kv_step, cudaMemcpyHostToDevice, hp->h2d), "copy V to device");
        check(cudaEventRecord(ev[2 * i], hp->h2d), "record");
        check(cudaStreamWaitEvent(hp->compute, ev[2 * i], 0), "wait for a group of heads");
        if (!failed && wave_cuda_flash_attention_fwd(&sub, dev + i * q_step, dev + off_k + i * kv_step,
                                                     dev + off_v + i * kv_step, dev + off_o + i * o_step, nullptr,
                                                     hp->compute) != WAVE_OK)
          failed = true; // message already recorded
        check(cudaEventRecord(ev[2 * i + 1], hp->compute), "record");
        check(cudaStreamWaitEvent(hp->d2h, ev[2 * i + 1], 0), "wait for a group's output");
        check(cudaMemcpyAsync(static_cast<char *>(O_host) + i * o_step, dev + off_o + i * o_step, o_step,
                              cudaMemcpyDeviceToHost, hp->d2h),
              "copy O to host");
      }
    }
    for (cudaStream_t q : {hp->h2d, hp->compute, hp->d2h})
      check(cudaStreamSynchronize(q), "synchronise the host-call pipeline");
    for (cudaEvent_t e : ev)
      if (e)
        cudaEventDestroy(e);
    return failed ? WAVE_E_CUDA : WAVE_OK;
  }

  rc = WAVE_OK;
  auto step = [&](cudaError_t e, const char *what) {
    if (rc == WAVE_OK && e != cudaSuccess)
      rc = cuda_fail(e, what);
    return rc == WAVE_OK;
  };
  if (step(cudaMemcpyAsync(dev, Q_host, q_bytes, cudaMemcpyHostToDevice, s), "copy Q to device") &&
      step(cudaMemcpyAsync(dev + off_k, K_host, kv_bytes, cudaMemcpyHostToDevice, s), "copy K to device") &&
      step(cudaMemcpyAsync(dev + off_v, V_host, kv_bytes, cudaMemcpyHostToDevice, s), "copy V to device")) {
    rc = wave_cuda_flash_attention_fwd(d, dev, dev + off_k, dev + off_v, dev + off_o, nullptr, stream);
    if (rc == WAVE_OK)
      step(cudaMemcpyAsync(O_host, dev + off_o, o_bytes, cudaMemcpyDeviceToHost, s), "copy O to host");
  }
  err = cudaStreamSynchronize(s); // also on failure: the arena goes to the next call
  if (rc == WAVE_OK && err != cudaSuccess)
    rc = cuda_fail(err, "synchronise after attention");
  return rc;
}

// ------------------------------------------------------- name-based facade
int wave_cuda_module_get_function(const char *kernel_name, const void *desc, void **fn) {
  if (!kernel_name || !desc || !fn)
    return fail(WAVE_E_INVALID, "kernel name, descriptor and result pointer must be non-null");
  FnHandle *h = new FnHandle{};
  if (strcmp(kernel_name, "wmma_f16_matmul_tiled") == 0) {
    h->kind = 0;
    h->gemm = *static_cast<const wave_gemm_desc *>(desc);
    if (h->gemm.streamk_workers != 1)
      h->gemm.streamk_workers = 1; // this ABI carries no workspace
  } else if (strcmp(kernel_name, "gfx950_f16_streamk_gemm") == 0) {
    h->kind = 1;
    h->gemm = *static_cast<const wave_gemm_desc *>(desc);
  } else if (strcmp(kernel_name, "flash_attention_bf16_gfx950") == 0 || strcmp(kernel_name, "flash_attention_f32") == 0) {
    h->kind = 2;
    h->fa = *static_cast<const wave_fa_desc *>(desc);
  } else {
    delete h;
    return fail(WAVE_E_NOT_FOUND, "no kernel named '%s' in this backend", kernel_name);
  }
  int rc = h->kind == 2 ? wave_cuda_fa_validate(&h->fa) : wave_cuda_gemm_validate(&h->gemm);
  if (rc != WAVE_OK) {
    delete h;
    return rc;
  }
  *fn = h;
  return WAVE_OK;
}

int wave_cuda_launch(void *fn, void **args, void *stream) {
  if (!fn || !args)
    return fail(WAVE_E_INVALID, "function handle and argument block must be non-null");
  FnHandle *h = static_cast<FnHandle *>(fn);
  if (h->kind == 0) {
    // {&A, &B, &C, &trip}: trip = K/(k_tile*wave_k_tiles) - 1 (wave_matmul.py:6964)
    const int trip = *static_cast<int *>(args[3]);
    const int expect = h->gemm.K / (16 * h->gemm.wave_k_tiles) - 1;
    if (trip != expect)
      return fail(WAVE_E_INVALID, "trip count %d does not match K/(16*wave_k_tiles)-1 = %d", trip, expect);
    return wave_cuda_gemm(&h->gemm, *static_cast<void **>(args[0]), *static_cast<void **>(args[1]),
                          *static_cast<void **>(args[2]), nullptr, stream);
  }
  if (h->kind == 1) {
    // {&A, &B, &C, &scratch, &counters, &workers}: scratch and counters must be
    // one allocation, counters directly after the scratch.
    wave_gemm_desc d = h->gemm;
    d.streamk_workers = *static_cast<int *>(args[5]);
    size_t scratch = 0, counters = 0;
    int rc = wave_cuda_gemm_workspace_bytes(&d, &scratch, &counters);
    if (rc != WAVE_OK)
      return rc;
    char *ws = *static_cast<char **>(args[3]);
    if (scratch + counters > 0 && *static_cast<char **>(args[4]) != ws + scratch)
      return fail(WAVE_E_INVALID, "counters must directly follow the %zu-byte scratch area", scratch);
    return wave_cuda_gemm(&d, *static_cast<void **>(args[0]), *static_cast<void **>(args[1]),
                          *static_cast<void **>(args[2]), ws, stream);
  }
  return wave_cuda_flash_attention_fwd(&h->fa, *static_cast<void **>(args[0]), *static_cast<void **>(args[1]),
                                       *static_cast<void **>(args[2]), *static_cast<void **>(args[3]), nullptr,
                                       stream);
}

void wave_cuda_function_release(void *fn) { delete static_cast<FnHandle *>(fn); }

int wave_cuda_check_device_status(int *out4) {
  cudaError_t err = cudaDeviceSynchronize();
  if (err != cudaSuccess)
    return cuda_fail(err, "cudaDeviceSynchronize");
  int g[4] = {0, 0, 0, 0}, f[4] = {0, 0, 0, 0}, g2[4] = {0, 0, 0, 0};
  if ((err = wave::gemm_read_status(g, true)) != cudaSuccess)
    return cuda_fail(err, "read GEMM status");
  if ((err = wave::gemm_pair_read_status(g2, true)) != cudaSuccess)
    return cuda_fail(err, "read GEMM (CTA pair) status");
  if (!g[0] && g2[0]) {
    for (int i = 0; i < 4; ++i)
      g[i] = g2[i];
    g[2] += 10; // roles 10.. : CTA-pair kernel
  }
  if ((err = wave::fa_read_status(f, true)) != cudaSuccess)
    return cuda_fail(err, "read attention status");
  const int *bad = g[0] ? g : (f[0] ? f : nullptr);
  if (out4)
    for (int i = 0; i < 4; ++i)
      out4[i] = bad ? bad[i] : 0;
  if (bad)
    return fail(WAVE_E_DEVICE_STATUS, "%s kernel reported status %d (block %d, role %d, detail %d)",
                bad == g ? "GEMM" : "attention", bad[0], bad[1], bad[2], bad[3]);
  return WAVE_OK;
}

} // extern "C"
