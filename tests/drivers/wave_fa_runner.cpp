// CUDA C++ timed runner for the flash-attention forward through the C ABI's
// name-based launch facade: the sm_100a counterpart of the reference's
// wave-fa-gfx950-runner (tools/wave-fa-calibrate/wave-fa-gfx950-runner.cpp).
//
// Same command line (`--batch --heads --sequence --seed --iters --warmup
// --input-scale --check --zero-qk`, the positional <hsaco> <kernel>; `--threads`
// and `--dynamic-lds` are accepted and ignored), same generator (the LCG of
// :188-202 scaled by 0.125 * input_scale for Q and K, 0.25 for V, rounded to
// bf16), same argument block {&Q, &K, &V, &O} (:446), same stdout lines
// (`shape:`, `grid:`, `per_launch_us:`, `tflops:`, `output_check: passed
// max_abs_diff=... index=...`, :472-481, :392) and exit codes (2 bad
// arguments, 1 failures).  The check is the runner's: f64 softmax rows on the
// sampled heads and rows (:204-232), natural exp, maximum absolute error
// 3e-2 (:388).  Added here: `--causal` (key <= query), `--repeats`.
//
// Build: nvcc -std=c++17 -x cu wave_fa_runner.cpp -I<repo>/include -L<repo>/7_b200 -lwave_cuda
#include "wave_cuda.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

namespace {

constexpr int kHeadDim = 128;
constexpr int kRowsPerWorkgroup = 256; // the reference kernel's BLOCK_M; sequences must be a multiple of it

struct Options {
  std::string kernel = "flash_attention_bf16_gfx950";
  int batch = 1, heads = 1, sequence = 256;
  int seed = 0, iters = 20, warmup = 5, repeats = 1, input_scale = 1;
  bool check = false, zero_qk = false, causal = false;
  float qk_max_abs = 0.0f; // 0: running row maximum; > 0: fixed softmax reference for |Q|,|K| <= this
};

int bad_arguments(const std::string &message) {
  std::fprintf(stderr, "%s\n", message.c_str());
  return 2;
}

bool parse_int(const std::string &text, int *out) {
  char *end = nullptr;
  const long v = std::strtol(text.c_str(), &end, 10);
  if (text.empty() || !end || *end != '\0')
    return false;
  *out = static_cast<int>(v);
  return true;
}

// Returns 0, or the exit code to leave with.
int parse(int argc, char **argv, Options *o) {
  int positional = 0;
  for (int i = 1; i < argc; ++i) {
    std::string arg = argv[i];
    if (arg == "--check") {
      o->check = true;
    } else if (arg == "--zero-qk") {
      o->zero_qk = true;
    } else if (arg == "--causal") {
      o->causal = true;
    } else if (arg.rfind("--", 0) == 0) {
      std::string value;
      const size_t eq = arg.find('=');
      if (eq != std::string::npos) {
        value = arg.substr(eq + 1);
        arg = arg.substr(0, eq);
      } else {
        if (++i == argc)
          return bad_arguments("missing flag value");
        value = argv[i];
      }
      if (arg == "--qk-max-abs") {
        // The reference bakes the bound into the code object (wave-fa-gfx950.py:103-107,
        // 169-176); there is no code object here, so the runner takes it itself.
        char *end = nullptr;
        const double bound = std::strtod(value.c_str(), &end);
        if (value.empty() || !end || *end != '\0' || !std::isfinite(bound) || bound <= 0)
          return bad_arguments("--qk-max-abs must be finite and positive");
        o->qk_max_abs = static_cast<float>(bound);
        continue;
      }
      int ignored = 0;
      int *dst = arg == "--batch"         ? &o->batch
                 : arg == "--heads"       ? &o->heads
                 : arg == "--sequence"    ? &o->sequence
                 : arg == "--seed"        ? &o->seed
                 : arg == "--iters"       ? &o->iters
                 : arg == "--warmup"      ? &o->warmup
                 : arg == "--repeats"     ? &o->repeats
                 : arg == "--input-scale" ? &o->input_scale
                 : (arg == "--threads" || arg == "--dynamic-lds") ? &ignored
                                                                  : nullptr;
      if (!dst)
        return bad_arguments("unknown flag");
      if (!parse_int(value, dst))
        return bad_arguments("bad integer argument");
    } else if (positional++ == 1) {
      o->kernel = arg; // the first positional is the code object's path: there is none here
    } else if (positional > 2) {
      return bad_arguments("unexpected positional argument");
    }
  }
  if (o->batch <= 0 || o->heads <= 0 || o->sequence <= 0 || o->iters <= 0 || o->warmup < 0 || o->repeats <= 0 ||
      o->input_scale <= 0)
    return bad_arguments("invalid non-positive argument");
  if (o->sequence % kRowsPerWorkgroup)
    return bad_arguments("sequence must be a multiple of 256");
  if (o->qk_max_abs > 0.0f && o->qk_max_abs < static_cast<float>(o->input_scale))
    return bad_arguments("--qk-max-abs must cover the generated input range"); // wave-fa-gfx950.py:77-78
  return 0;
}

uint16_t to_bf16(float value) {
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  bits += 0x7fffu + ((bits >> 16) & 1u); // round to nearest even
  return static_cast<uint16_t>(bits >> 16);
}
float from_bf16(uint16_t value) {
  const uint32_t bits = static_cast<uint32_t>(value) << 16;
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}

// 17-bucket LCG of the reference's runners: ((state >> 24) % 17 - 8) * scale.
std::vector<uint16_t> make_input(size_t count, int seed, int stream, float scale) {
  uint32_t state = static_cast<uint32_t>(seed) ^ (static_cast<uint32_t>(stream + 1) * 0x9e3779b9u);
  std::vector<uint16_t> out(count);
  for (uint16_t &v : out) {
    state = 1664525u * state + 1013904223u;
    v = to_bf16(static_cast<float>(static_cast<int>((state >> 24) % 17u) - 8) * scale);
  }
  return out;
}

std::vector<int> sampled_heads(int count) {
  if (count <= 4) {
    std::vector<int> all(count);
    for (int i = 0; i < count; ++i)
      all[i] = i;
    return all;
  }
  return {0, count / 2, count - 1};
}
std::vector<int> sampled_rows(int sequence) {
  std::vector<int> rows;
  if (sequence <= 512) {
    for (int r = 0; r < sequence; ++r)
      rows.push_back(r);
    return rows;
  }
  rows = {0, 31, 32, 127, sequence / 2, sequence - 128, sequence - 1};
  std::sort(rows.begin(), rows.end());
  rows.erase(std::unique(rows.begin(), rows.end()), rows.end());
  return rows;
}

// One output row in f64: softmax(q.k / sqrt(D)) . V over the visible keys.
void reference_row(const Options &o, const uint16_t *q, const uint16_t *k, const uint16_t *v, int head, int row,
                   double *out) {
  const size_t base = static_cast<size_t>(head) * o.sequence * kHeadDim;
  const int keys = o.causal ? row + 1 : o.sequence;
  const double scale = 1.0 / std::sqrt(static_cast<double>(kHeadDim));
  std::vector<double> w(keys);
  double top = -INFINITY;
  for (int key = 0; key < keys; ++key) {
    double dot = 0.0;
    for (int d = 0; d < kHeadDim; ++d)
      dot += static_cast<double>(from_bf16(q[base + static_cast<size_t>(row) * kHeadDim + d])) *
             static_cast<double>(from_bf16(k[base + static_cast<size_t>(key) * kHeadDim + d]));
    w[key] = dot * scale;
    top = std::max(top, w[key]);
  }
  double total = 0.0;
  for (double &x : w) {
    x = std::exp(x - top);
    total += x;
  }
  for (int d = 0; d < kHeadDim; ++d) {
    double acc = 0.0;
    for (int key = 0; key < keys; ++key)
      acc += w[key] * static_cast<double>(from_bf16(v[base + static_cast<size_t>(key) * kHeadDim + d]));
    out[d] = static_cast<double>(static_cast<float>(acc / total));
  }
}

int cuda_failed(cudaError_t err, const char *what) {
  std::fprintf(stderr, "%s: %s\n", what, cudaGetErrorString(err));
  return 1;
}
int wave_failed(const char *what) {
  std::fprintf(stderr, "%s: %s\n", what, wave_cuda_last_error());
  return 1;
}

} // namespace

int main(int argc, char **argv) {
  Options o;
  if (int rc = parse(argc, argv, &o))
    return rc;
  const size_t elements = static_cast<size_t>(o.batch) * o.heads * o.sequence * kHeadDim;
  const float qk_scale = 0.125f * static_cast<float>(o.input_scale);
  std::vector<uint16_t> q = make_input(elements, o.seed, 0, qk_scale);
  std::vector<uint16_t> k = make_input(elements, o.seed, 1, qk_scale);
  std::vector<uint16_t> v = make_input(elements, o.seed, 2, 0.25f);
  if (o.zero_qk) {
    std::fill(q.begin(), q.end(), 0);
    std::fill(k.begin(), k.end(), 0);
  }

  wave_fa_desc desc;
  std::memset(&desc, 0, sizeof(desc));
  desc.batch = o.batch;
  desc.heads = o.heads;
  desc.seq_q = desc.seq_k = o.sequence;
  desc.head_dim = kHeadDim;
  desc.scale = 0.0f; // default 1/sqrt(head_dim)
  desc.causal = o.causal ? 1 : 0;
  desc.io_type = WAVE_BF16;
  desc.out_f32 = 0;
  desc.qk_max_abs = o.qk_max_abs;
  void *fn = nullptr;
  const int found = wave_cuda_module_get_function(o.kernel.c_str(), &desc, &fn);
  if (found == WAVE_E_INVALID || found == WAVE_E_UNSUPPORTED)
    return bad_arguments(wave_cuda_last_error());
  if (found != WAVE_OK)
    return wave_failed("wave_cuda_module_get_function");

  const size_t bytes = elements * sizeof(uint16_t);
  uint16_t *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr;
  cudaError_t err;
  if ((err = cudaMalloc(&dq, bytes)) != cudaSuccess || (err = cudaMalloc(&dk, bytes)) != cudaSuccess ||
      (err = cudaMalloc(&dv, bytes)) != cudaSuccess || (err = cudaMalloc(&dout, bytes)) != cudaSuccess)
    return cuda_failed(err, "cudaMalloc");
  if ((err = cudaMemcpy(dq, q.data(), bytes, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (err = cudaMemcpy(dk, k.data(), bytes, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (err = cudaMemcpy(dv, v.data(), bytes, cudaMemcpyHostToDevice)) != cudaSuccess ||
      (err = cudaMemset(dout, 0, bytes)) != cudaSuccess)
    return cuda_failed(err, "copy inputs");
  void *args[] = {&dq, &dk, &dv, &dout};

  for (int i = 0; i < o.warmup; ++i)
    if (wave_cuda_launch(fn, args, nullptr) != WAVE_OK)
      return wave_failed("wave_cuda_launch");
  if ((err = cudaDeviceSynchronize()) != cudaSuccess)
    return cuda_failed(err, "warmup sync");

  cudaEvent_t start = nullptr, stop = nullptr;
  cudaEventCreate(&start);
  cudaEventCreate(&stop);
  std::vector<double> per_launch_us;
  for (int r = 0; r < o.repeats; ++r) {
    cudaEventRecord(start);
    for (int i = 0; i < o.iters; ++i)
      if (wave_cuda_launch(fn, args, nullptr) != WAVE_OK)
        return wave_failed("wave_cuda_launch");
    cudaEventRecord(stop);
    if ((err = cudaEventSynchronize(stop)) != cudaSuccess)
      return cuda_failed(err, "cudaEventSynchronize");
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, start, stop);
    per_launch_us.push_back(static_cast<double>(ms) * 1000.0 / o.iters);
  }
  int status[4] = {0, 0, 0, 0};
  if (wave_cuda_check_device_status(status) != WAVE_OK)
    return wave_failed("device status");
  std::sort(per_launch_us.begin(), per_launch_us.end());
  const double us = per_launch_us[per_launch_us.size() / 2];
  // The reference counts every query-key pair (4 B H N^2 D); with --causal only the visible ones.
  const long double pairs = o.causal ? static_cast<long double>(o.sequence) * (o.sequence + 1) / 2
                                     : static_cast<long double>(o.sequence) * o.sequence;
  const double tflops = static_cast<double>(4.0L * o.batch * o.heads * pairs * kHeadDim / us * 1.0e-6L);

  std::vector<uint16_t> out(elements);
  if ((err = cudaMemcpy(out.data(), dout, bytes, cudaMemcpyDeviceToHost)) != cudaSuccess)
    return cuda_failed(err, "copy output");
  std::printf("kernel: %s\n", o.kernel.c_str());
  std::printf("shape: B=%d H=%d N=%d D=%d\n", o.batch, o.heads, o.sequence, kHeadDim);
  std::printf("grid: %d,%d,1 block: 384,1,1 dynamic_lds=0 causal=%d\n", o.sequence / kRowsPerWorkgroup,
              o.batch * o.heads, o.causal ? 1 : 0);
  std::printf("iters: %d\n", o.iters);
  std::printf("per_launch_us: %.3f\n", us);
  if (o.repeats > 1) {
    std::printf("median_per_launch_us: %.3f\n", us);
    std::printf("best_per_launch_us: %.3f\n", per_launch_us.front());
  }
  std::printf("tflops: %.3f\n", tflops);

  int exit_code = 0;
  if (o.check) {
    const std::vector<int> heads = sampled_heads(o.batch * o.heads), rows = sampled_rows(o.sequence);
    const size_t n = heads.size() * rows.size();
    std::vector<double> expect(n * kHeadDim);
    unsigned workers = std::max(1u, std::thread::hardware_concurrency());
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < workers; ++t)
      pool.emplace_back([&, t] {
        for (size_t i = t; i < n; i += workers)
          reference_row(o, q.data(), k.data(), v.data(), heads[i / rows.size()], rows[i % rows.size()],
                        &expect[i * kHeadDim]);
      });
    for (std::thread &th : pool)
      th.join();
    double worst = 0.0;
    size_t worst_index = 0, worst_i = 0;
    int worst_d = 0;
    for (size_t i = 0; i < n; ++i) {
      const size_t row_base = (static_cast<size_t>(heads[i / rows.size()]) * o.sequence + rows[i % rows.size()]) * kHeadDim;
      for (int d = 0; d < kHeadDim; ++d) {
        const float got = from_bf16(out[row_base + d]);
        const double diff = std::isfinite(got) ? std::fabs(got - expect[i * kHeadDim + d]) : INFINITY;
        if (diff > worst) {
          worst = diff;
          worst_index = row_base + d;
          worst_i = i;
          worst_d = d;
        }
      }
    }
    if (worst > 3.0e-2) {
      std::fprintf(stderr, "output_check: failed head=%d row=%d d=%d index=%zu expected=%.8f got=%.8f abs_diff=%.8f\n",
                   heads[worst_i / rows.size()], rows[worst_i % rows.size()], worst_d, worst_index,
                   expect[worst_i * kHeadDim + worst_d], from_bf16(out[worst_index]), worst);
      exit_code = 1;
    } else {
      std::printf("output_check: passed max_abs_diff=%.8f index=%zu\n", worst, worst_index);
    }
  }

  cudaEventDestroy(start);
  cudaEventDestroy(stop);
  cudaFree(dq);
  cudaFree(dk);
  cudaFree(dv);
  cudaFree(dout);
  wave_cuda_function_release(fn);
  return exit_code;
}
