// CUDA C++ counterpart of the reference's GEMM calibrate runner
// (tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp): same flags
// for the surface this backend carries (runner.cpp:36-64, 71-102), same
// stdout keys (runner.cpp:1881-1908, 918-954, 1732), same exit codes (1 for a
// CUDA error or failed check, 2 for bad arguments; runner.cpp:66-69, 620-625).
// Where the reference does hipModuleLoad / hipModuleGetFunction /
// hipModuleLaunchKernel with an array of pointers to the argument values
// (runner.cpp:1790-1816, 1846-1879) this runner goes through the name-based
// facade of libwave_cuda.so with the very same argument blocks.
//
// It is a checker: inputs and the f32 CPU reference come from the test
// oracle (oracle/wave_oracle.c), so it lives with the tests, not in the
// product.  Build (see tests/test_native_runner.py):
//   nvcc -std=c++17 -O2 wave_matmul_calibrate_runner.cpp -I<repo>/include \
//        -L<repo>/7_b200 -lwave_cuda -L<repo>/oracle -lwave_oracle -o runner
// Like the reference (runner.cpp:1835) the file can be included with
// WAVE_MATMUL_CALIBRATE_RUNNER_NO_MAIN defined to unit-test its host logic;
// with WAVE_RUNNER_HOST_ONLY it needs neither CUDA headers nor a GPU.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "wave_cuda.h"
#ifndef WAVE_RUNNER_HOST_ONLY
#include <cuda_runtime.h>
#endif

extern "C" {
// oracle/wave_oracle.c (test infrastructure)
int wo_make_input_bits(uint16_t *out, size_t elements, int k, int type, int seed, int stream, int mode);
int wo_gemm_ref(const uint16_t *A, const uint16_t *B, int M, int N, int K, int type, const int *rows, int nrows,
                float *out, int nthreads);
uint16_t wo_f32_to_bf16(float v);
float wo_bf16_to_f32(uint16_t h);
uint16_t wo_f32_to_f16(float v);
float wo_f16_to_f32(uint16_t h);
}

namespace runner {

enum class Abi { Matmul, StreamK };

struct Options {
  std::string kernel;
  int m = 32, n = 32, k = 32;
  int bm = 1, bn = 2, wave_m_tiles = 1, wave_n_tiles = 1, wave_k_tiles = 1;
  int input_type = WAVE_F16, c_type = WAVE_F32, layout = WAVE_ROW_MAJOR;
  Abi abi = Abi::Matmul;
  int streamk_workers = 1, cta_group_m = 1;
  int iters = 1000, warmup = 10, seed = 0;
  bool all_ones = false, rand_int = false, hpl = false, check = true;
  int check_rows = 0; // 0 = every row
};

struct ParseResult {
  bool ok = true;
  std::string error;
};

inline const char *type_name(int t) { return t == WAVE_F16 ? "f16" : t == WAVE_BF16 ? "bf16" : "f32"; }
inline const char *layout_name(int l) {
  return l == WAVE_ROW_MAJOR ? "row-major" : l == WAVE_COL_MAJOR ? "column-major" : "tile-packed";
}
inline const char *mode_name(const Options &o) {
  return o.all_ones ? "all_ones" : o.rand_int ? "rand_int" : o.hpl ? "hpl" : "lcg";
}
inline int input_mode(const Options &o) { return o.all_ones ? 1 : o.rand_int ? 2 : o.hpl ? 3 : 0; }

inline bool parse_int(const std::string &text, int *out) {
  char *end = nullptr;
  long v = std::strtol(text.c_str(), &end, 10);
  if (text.empty() || *end != '\0' || v < INT32_MIN || v > INT32_MAX)
    return false;
  *out = static_cast<int>(v);
  return true;
}

// Flags come as `--name value` or `--name=value`.  AMD-only controls of the
// reference runner are accepted and ignored so that existing command lines run.
inline ParseResult parse(int argc, char **argv, Options *o) {
  ParseResult r;
  auto fail = [&](const std::string &msg) {
    r.ok = false;
    r.error = msg;
    return r;
  };
  for (int i = 1; i < argc; ++i) {
    std::string arg = argv[i], value;
    bool has_value = false;
    size_t eq = arg.find('=');
    if (eq != std::string::npos) {
      value = arg.substr(eq + 1);
      arg = arg.substr(0, eq);
      has_value = true;
    }
    auto need = [&]() -> bool {
      if (has_value)
        return true;
      if (i + 1 >= argc)
        return false;
      value = argv[++i];
      return true;
    };
    struct IntFlag {
      const char *name;
      int *dst;
    } ints[] = {{"--m", &o->m}, {"--n", &o->n}, {"--k", &o->k}, {"--bm", &o->bm}, {"--bn", &o->bn},
                {"--wave-m-tiles", &o->wave_m_tiles}, {"--wave-n-tiles", &o->wave_n_tiles},
                {"--wave-k-tiles", &o->wave_k_tiles}, {"--iters", &o->iters}, {"--warmup", &o->warmup},
                {"--seed", &o->seed}, {"--streamk-workers", &o->streamk_workers}, {"--cta-group-m", &o->cta_group_m},
                {"--check-rows", &o->check_rows}};
    bool done = false;
    for (const IntFlag &f : ints)
      if (arg == f.name) {
        if (!need() || !parse_int(value, f.dst))
          return fail("invalid integer for " + arg);
        done = true;
      }
    if (done)
      continue;
    if (arg == "--kernel") {
      if (!need())
        return fail("missing value for --kernel");
      o->kernel = value;
    } else if (arg == "--input-type") {
      if (!need())
        return fail("missing value for --input-type");
      if (value == "f16")
        o->input_type = WAVE_F16;
      else if (value == "bf16")
        o->input_type = WAVE_BF16;
      else
        return fail("--input-type must be f16 or bf16 on this backend; got " + value);
    } else if (arg == "--c-type") {
      if (!need())
        return fail("missing value for --c-type");
      if (value == "f32")
        o->c_type = WAVE_F32;
      else if (value == "f16")
        o->c_type = WAVE_F16;
      else if (value == "bf16")
        o->c_type = WAVE_BF16;
      else
        return fail("--c-type must be f32, f16 or bf16; got " + value);
    } else if (arg == "--output-layout") {
      if (!need())
        return fail("missing value for --output-layout");
      if (value == "automatic" || value == "row-major")
        o->layout = WAVE_ROW_MAJOR;
      else if (value == "column-major")
        o->layout = WAVE_COL_MAJOR;
      else
        return fail("--output-layout must be automatic, row-major or column-major; got " + value);
    } else if (arg == "--kernel-abi") {
      if (!need())
        return fail("missing value for --kernel-abi");
      if (value == "matmul")
        o->abi = Abi::Matmul;
      else if (value == "streamk")
        o->abi = Abi::StreamK;
      else
        return fail("--kernel-abi must be matmul or streamk on this backend; got " + value);
    } else if (arg == "--all-ones") {
      o->all_ones = true;
    } else if (arg == "--rand-int") {
      o->rand_int = true;
    } else if (arg == "--hpl") {
      o->hpl = true;
    } else if (arg == "--no-check") {
      o->check = false;
    } else if (arg == "--hsaco" || arg == "--wave-size" || arg == "--dynamic-lds-bytes" ||
               arg == "--accumulator-layout" || arg == "--scale-layout" || arg == "--mxfp4-input-layout") {
      if (!need())
        return fail("missing value for " + arg);
    } else {
      return fail("unknown argument: " + arg);
    }
  }
  if (static_cast<int>(o->all_ones) + o->rand_int + o->hpl > 1)
    return fail("--all-ones, --rand-int and --hpl are mutually exclusive");
  if (o->iters <= 0)
    return fail("--iters must be positive");
  if (o->warmup < 0)
    return fail("--warmup must be non-negative");
  if (o->abi == Abi::StreamK && o->streamk_workers < 1)
    return fail("--streamk-workers must be positive");
  if (o->abi == Abi::Matmul && o->streamk_workers != 1)
    return fail("--streamk-workers requires --kernel-abi=streamk");
  if (o->kernel.empty())
    o->kernel = o->abi == Abi::StreamK ? "gfx950_f16_streamk_gemm" : "wmma_f16_matmul_tiled";
  return r;
}

inline wave_gemm_desc make_desc(const Options &o) {
  wave_gemm_desc d;
  wave_cuda_gemm_desc_init(&d, o.m, o.n, o.k);
  d.bm = o.bm;
  d.bn = o.bn;
  d.wave_m_tiles = o.wave_m_tiles;
  d.wave_n_tiles = o.wave_n_tiles;
  d.wave_k_tiles = o.wave_k_tiles;
  d.in_type = o.input_type;
  d.out_type = o.c_type;
  d.out_layout = o.layout;
  d.cta_group_m = o.cta_group_m;
  d.streamk_workers = o.abi == Abi::StreamK ? o.streamk_workers : 1;
  return d;
}

// The i32 kernel argument of the plain ABI: K/(k_tile*wave_k_tiles) - 1
// (python/mlir/dialects/wave_matmul.py:6964, runner.cpp:1114-1133).
inline int trip_count(const Options &o) { return o.k / (16 * o.wave_k_tiles) - 1; }

inline double read_output(const void *c, int type, size_t index) {
  if (type == WAVE_F32)
    return static_cast<const float *>(c)[index];
  uint16_t raw = static_cast<const uint16_t *>(c)[index];
  return type == WAVE_F16 ? wo_f16_to_f32(raw) : wo_bf16_to_f32(raw);
}
inline double round_expected(float v, int type) {
  if (type == WAVE_F16)
    return wo_f16_to_f32(wo_f32_to_f16(v));
  if (type == WAVE_BF16)
    return wo_bf16_to_f32(wo_f32_to_bf16(v));
  return v;
}

struct CheckResult {
  bool ok = true;
  int m = 0, n = 0;
  double expected = 0, got = 0, diff = 0, limit = 0;
  double worst = 0;
  long long worst_index = 0, elements = 0;
};

// |got - exp| <= 1e-2 + 1e-3*|exp| (runner.cpp:907); a bf16 result, which the
// reference never stores, gets one bf16 unit in the last place (2^-7) as the
// relative term.
inline CheckResult check_output(const Options &o, const void *c, const std::vector<int> &rows,
                                const std::vector<float> &expected_rows) {
  CheckResult r;
  const double rel = o.c_type == WAVE_BF16 ? 1.0 / 128.0 : 1.0e-3;
  for (size_t ri = 0; ri < rows.size(); ++ri) {
    const int m = rows[ri];
    for (int n = 0; n < o.n; ++n) {
      const size_t index = o.layout == WAVE_ROW_MAJOR ? static_cast<size_t>(m) * o.n + n
                                                       : static_cast<size_t>(n) * o.m + m;
      const double exp = round_expected(expected_rows[ri * o.n + n], o.c_type);
      const double got = read_output(c, o.c_type, index);
      const double diff = std::fabs(got - exp);
      const double limit = 1.0e-2 + rel * std::fabs(exp);
      ++r.elements;
      if (diff > r.worst) {
        r.worst = diff;
        r.worst_index = static_cast<long long>(index);
      }
      if (!(diff <= limit)) {
        r.ok = false;
        r.m = m;
        r.n = n;
        r.expected = exp;
        r.got = got;
        r.diff = diff;
        r.limit = limit;
        return r;
      }
    }
  }
  return r;
}

inline std::vector<int> rows_to_check(const Options &o) {
  std::vector<int> rows;
  if (o.check_rows <= 0 || o.check_rows >= o.m) {
    for (int m = 0; m < o.m; ++m)
      rows.push_back(m);
    return rows;
  }
  for (int i = 0; i < o.check_rows; ++i) {
    int m = static_cast<int>(static_cast<long long>(i) * (o.m - 1) / (o.check_rows > 1 ? o.check_rows - 1 : 1));
    if (rows.empty() || rows.back() != m)
      rows.push_back(m);
  }
  return rows;
}

#ifndef WAVE_RUNNER_HOST_ONLY
inline void cuda_or_die(cudaError_t err, const char *what) {
  if (err == cudaSuccess)
    return;
  std::fprintf(stderr, "%s failed: %s\n", what, cudaGetErrorString(err));
  std::exit(1);
}
inline void wave_or_die(int rc, int code_for_invalid) {
  if (rc == WAVE_OK)
    return;
  std::fprintf(stderr, "%s\n", wave_cuda_last_error());
  std::exit(rc == WAVE_E_INVALID || rc == WAVE_E_UNSUPPORTED ? code_for_invalid : 1);
}

inline int run(const Options &o) {
  wave_gemm_desc desc = make_desc(o);
  wave_or_die(wave_cuda_gemm_validate(&desc), 2);
  size_t scratch_bytes = 0, counter_bytes = 0;
  wave_or_die(wave_cuda_gemm_workspace_bytes(&desc, &scratch_bytes, &counter_bytes), 2);

  const int otype = o.input_type == WAVE_BF16 ? 1 : 0;
  std::vector<uint16_t> a(static_cast<size_t>(o.m) * o.k), b(static_cast<size_t>(o.n) * o.k);
  wo_make_input_bits(a.data(), a.size(), o.k, otype, o.seed, 0, input_mode(o));
  wo_make_input_bits(b.data(), b.size(), o.k, otype, o.seed, 1, input_mode(o));
  const size_t c_elems = static_cast<size_t>(o.m) * o.n;
  const size_t c_bytes = c_elems * (o.c_type == WAVE_F32 ? 4 : 2);

  void *dA = nullptr, *dB = nullptr, *dC = nullptr, *dW = nullptr;
  cuda_or_die(cudaMalloc(&dA, a.size() * 2), "cudaMalloc A");
  cuda_or_die(cudaMalloc(&dB, b.size() * 2), "cudaMalloc B");
  cuda_or_die(cudaMalloc(&dC, c_bytes), "cudaMalloc C");
  cuda_or_die(cudaMemcpy(dA, a.data(), a.size() * 2, cudaMemcpyHostToDevice), "cudaMemcpy A");
  cuda_or_die(cudaMemcpy(dB, b.data(), b.size() * 2, cudaMemcpyHostToDevice), "cudaMemcpy B");
  cuda_or_die(cudaMemset(dC, 0, c_bytes), "cudaMemset C"); // runner.cpp:1659
  if (scratch_bytes + counter_bytes) {
    cuda_or_die(cudaMalloc(&dW, scratch_bytes + counter_bytes), "cudaMalloc Stream-K workspace");
    cuda_or_die(cudaMemset(dW, 0, scratch_bytes + counter_bytes), "cudaMemset Stream-K workspace");
  }

  void *fn = nullptr;
  wave_or_die(wave_cuda_module_get_function(o.kernel.c_str(), &desc, &fn), 2);
  int trip = trip_count(o), workers = o.streamk_workers;
  void *scratch = dW, *counters = dW ? static_cast<char *>(dW) + scratch_bytes : nullptr;
  void *plain_args[] = {&dA, &dB, &dC, &trip};
  void *streamk_args[] = {&dA, &dB, &dC, &scratch, &counters, &workers};
  void **args = o.abi == Abi::StreamK ? streamk_args : plain_args;

  for (int i = 0; i < o.warmup; ++i)
    wave_or_die(wave_cuda_launch(fn, args, nullptr), 1);
  cuda_or_die(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  cudaEvent_t start, stop;
  cuda_or_die(cudaEventCreate(&start), "cudaEventCreate");
  cuda_or_die(cudaEventCreate(&stop), "cudaEventCreate");
  cuda_or_die(cudaEventRecord(start), "cudaEventRecord");
  for (int i = 0; i < o.iters; ++i)
    wave_or_die(wave_cuda_launch(fn, args, nullptr), 1);
  cuda_or_die(cudaEventRecord(stop), "cudaEventRecord");
  cuda_or_die(cudaEventSynchronize(stop), "cudaEventSynchronize");
  float elapsed_ms = 0;
  cuda_or_die(cudaEventElapsedTime(&elapsed_ms, start, stop), "cudaEventElapsedTime");
  int status[4];
  wave_or_die(wave_cuda_check_device_status(status), 1);

  cudaDeviceProp props;
  cuda_or_die(cudaGetDeviceProperties(&props, 0), "cudaGetDeviceProperties");
  int tile_m = 0, tile_n = 0, grid = 0, sk = 0, swapped = 0;
  wave_or_die(wave_cuda_gemm_plan(&desc, &tile_m, &tile_n, &grid, &sk, &swapped), 2);
  const double per_launch_us = elapsed_ms * 1000.0 / o.iters;
  std::printf("device: %s (sm_%d%da) sms=%d\n", props.name, props.major, props.minor, props.multiProcessorCount);
  std::printf("kernel: %s\n", o.kernel.c_str());
  std::printf("shape: m=%d n=%d k=%d bm=%d bn=%d wave_m_tiles=%d wave_n_tiles=%d wave_k_tiles=%d wave_size=32 "
              "input_type=%s c_type=%s kernel_abi=%s output_layout=%s scale_layout=canonical "
              "mxfp4_input_layout=canonical input_mode=%s\n",
              o.m, o.n, o.k, o.bm, o.bn, o.wave_m_tiles, o.wave_n_tiles, o.wave_k_tiles, type_name(o.input_type),
              type_name(o.c_type), o.abi == Abi::StreamK ? "streamk" : "matmul", layout_name(o.layout), mode_name(o));
  std::printf("output_contract: kernel=%s final=%s conversion=none\n", layout_name(o.layout), layout_name(o.layout));
  std::printf("grid: %d,1,1 block: 192,1,1 tile=%dx%d streamk_workers=%d swapped=%d\n", grid, tile_m, tile_n, sk,
              swapped);
  std::printf("loop_trip_count: %d\n", trip);
  std::printf("iters: %d\n", o.iters);
  std::printf("timing_scope: gemm\n");
  std::printf("total_ms: %.3f\n", elapsed_ms);
  std::printf("per_launch_us: %.3f\n", per_launch_us);
  std::printf("tflops: %.3f\n", 2.0 * o.m * o.n * o.k / per_launch_us * 1e-6);

  int rc = 0;
  if (o.check) {
    std::vector<uint8_t> host_c(c_bytes);
    cuda_or_die(cudaMemcpy(host_c.data(), dC, c_bytes, cudaMemcpyDeviceToHost), "cudaMemcpy C");
    std::vector<int> rows = rows_to_check(o);
    std::vector<float> expected(rows.size() * static_cast<size_t>(o.n));
    wo_gemm_ref(a.data(), b.data(), o.m, o.n, o.k, otype, rows.data(), static_cast<int>(rows.size()),
                expected.data(), 16);
    CheckResult cr = check_output(o, host_c.data(), rows, expected);
    if (!cr.ok) {
      std::fprintf(stderr, "output_check: failed m=%d n=%d expected=%.6f got=%.6f abs_diff=%.6f tolerance=%.6f\n", cr.m,
                   cr.n, cr.expected, cr.got, cr.diff, cr.limit);
      rc = 1;
    } else {
      std::printf("output_check: passed mode=strict layout=%s elements=%lld max_abs_diff=%.6f index=%lld\n",
                  layout_name(o.layout), cr.elements, cr.worst, cr.worst_index);
    }
  }
  if (rc == 0 && counter_bytes) {
    // runner.cpp:1718-1733: every arrival counter must be back at zero.
    std::vector<uint32_t> left(counter_bytes / 4);
    cuda_or_die(cudaMemcpy(left.data(), counters, counter_bytes, cudaMemcpyDeviceToHost), "cudaMemcpy counters");
    for (size_t i = 0; i < left.size(); ++i)
      if (left[i] != 0) {
        std::fprintf(stderr, "Stream-K counter %zu did not reset: %u\n", i, left[i]);
        rc = 2;
        break;
      }
    if (rc == 0)
      std::printf("streamk_counter_check: passed\n");
  }
  wave_cuda_function_release(fn);
  cudaEventDestroy(start);
  cudaEventDestroy(stop);
  cudaFree(dA);
  cudaFree(dB);
  cudaFree(dC);
  cudaFree(dW);
  return rc;
}
#endif // WAVE_RUNNER_HOST_ONLY

} // namespace runner

#ifndef WAVE_MATMUL_CALIBRATE_RUNNER_NO_MAIN
int main(int argc, char **argv) {
  runner::Options options;
  runner::ParseResult parsed = runner::parse(argc, argv, &options);
  if (!parsed.ok) {
    std::fprintf(stderr, "%s\n", parsed.error.c_str());
    return 2;
  }
  return runner::run(options);
}
#endif
