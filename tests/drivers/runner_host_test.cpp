// Host-only unit test of the CUDA calibrate runner's host logic, built with
// plain g++ (no CUDA headers, no GPU), the way the reference tests its runner
// (test/Integration/Inputs/wave_matmul_rand_int_test.cpp includes the runner
// with WAVE_MATMUL_CALIBRATE_RUNNER_NO_MAIN; driver
// test/Integration/wave_matmul_rand_int_inputs.mlir).  Checks argument parsing
// and rejection, descriptor construction, the plain ABI's trip count, the
// Stream-K workspace size through the library, and the output comparison.
#define WAVE_MATMUL_CALIBRATE_RUNNER_NO_MAIN
#define WAVE_RUNNER_HOST_ONLY
#include "wave_matmul_calibrate_runner.cpp"

#include <initializer_list>

static int failures = 0;
static void expect(bool cond, const char *what) {
  if (!cond) {
    std::fprintf(stderr, "FAILED: %s\n", what);
    ++failures;
  }
}

static runner::ParseResult parse_args(std::initializer_list<const char *> args, runner::Options *o) {
  std::vector<char *> argv{const_cast<char *>("runner")};
  for (const char *a : args)
    argv.push_back(const_cast<char *>(a));
  return runner::parse(static_cast<int>(argv.size()), argv.data(), o);
}

int main() {
  {
    runner::Options o;
    runner::ParseResult r = parse_args({"--m", "256", "--n=512", "--k", "1024", "--bm=4", "--bn", "4",
                                        "--wave-m-tiles=2", "--wave-n-tiles=4", "--wave-k-tiles=2", "--input-type=bf16",
                                        "--c-type", "f16", "--output-layout=column-major", "--rand-int", "--iters=7",
                                        "--warmup=0", "--seed=91", "--hsaco", "x.hsaco", "--wave-size=64"}, &o);
    expect(r.ok, "well-formed command line parses");
    expect(o.m == 256 && o.n == 512 && o.k == 1024 && o.bm == 4 && o.bn == 4, "shape and wave flags");
    expect(o.input_type == WAVE_BF16 && o.c_type == WAVE_F16 && o.layout == WAVE_COL_MAJOR, "types and layout");
    expect(o.rand_int && !o.hpl && o.iters == 7 && o.warmup == 0 && o.seed == 91, "input mode and timing flags");
    expect(o.kernel == "wmma_f16_matmul_tiled", "default kernel name of the plain ABI");
    expect(runner::trip_count(o) == 1024 / 32 - 1, "trip count = K/(16*wave_k_tiles) - 1");
    wave_gemm_desc d = runner::make_desc(o);
    expect(wave_cuda_gemm_validate(&d) == WAVE_OK, "descriptor validates");
    expect(std::string(runner::mode_name(o)) == "rand_int", "input mode name");
  }
  {
    runner::Options o;
    expect(!parse_args({"--rand-int", "--hpl"}, &o).ok, "rand-int and hpl are exclusive");
    runner::Options o2;
    expect(!parse_args({"--iters=0"}, &o2).ok, "iters must be positive");
    runner::Options o3;
    expect(!parse_args({"--m", "abc"}, &o3).ok, "non-numeric value rejected");
    runner::Options o4;
    expect(!parse_args({"--input-type=mxfp4"}, &o4).ok, "mxfp4 is outside this backend");
    runner::Options o5;
    expect(!parse_args({"--frobnicate"}, &o5).ok, "unknown flag rejected");
    runner::Options o6;
    expect(!parse_args({"--streamk-workers=4"}, &o6).ok, "workers need the streamk ABI");
    runner::Options o7;
    expect(!parse_args({"--kernel-abi=aiter"}, &o7).ok, "AMD-only ABIs rejected");
  }
  {
    runner::Options o;
    expect(parse_args({"--m=512", "--n=768", "--k=1024", "--bm=4", "--bn=4", "--wave-m-tiles=2", "--wave-n-tiles=4",
                       "--kernel-abi=streamk", "--streamk-workers=5"}, &o).ok, "stream-K command line parses");
    expect(o.kernel == "gfx950_f16_streamk_gemm", "default kernel name of the Stream-K ABI");
    wave_gemm_desc d = runner::make_desc(o);
    size_t scratch = 0, counters = 0;
    expect(wave_cuda_gemm_workspace_bytes(&d, &scratch, &counters) == WAVE_OK, "workspace query");
    expect(scratch == size_t(5) * 2 * 128 * 256 * 4 && counters == 4 * 3 * 4, "Stream-K workspace size");
    o.bn = 3;
    wave_gemm_desc bad = runner::make_desc(o);
    expect(wave_cuda_gemm_validate(&bad) == WAVE_E_INVALID, "BN must be a power of two");
    expect(std::strstr(wave_cuda_last_error(), "BN must be a positive power of two") != nullptr, "reference message");
  }
  {
    // output comparison: 2 x 16 f16 outputs, one element moved just past tolerance
    runner::Options o;
    o.m = 2;
    o.n = 16;
    o.c_type = WAVE_F16;
    std::vector<float> expected(32);
    std::vector<uint16_t> c(32);
    for (int i = 0; i < 32; ++i) {
      expected[i] = 0.37f * static_cast<float>(i - 11);
      c[i] = wo_f32_to_f16(expected[i]);
    }
    std::vector<int> rows{0, 1};
    runner::CheckResult ok = runner::check_output(o, c.data(), rows, expected);
    expect(ok.ok && ok.elements == 32 && ok.worst == 0.0, "exactly rounded outputs pass with zero error");
    c[21] = wo_f32_to_f16(expected[21] + 0.05f);
    runner::CheckResult bad = runner::check_output(o, c.data(), rows, expected);
    expect(!bad.ok && bad.m == 1 && bad.n == 5, "an element beyond 1e-2 + 1e-3*|exp| is reported with its coordinates");
    o.layout = WAVE_COL_MAJOR; // element (m, n) lives at n*M + m
    std::vector<uint16_t> cm(32);
    for (int m = 0; m < 2; ++m)
      for (int n = 0; n < 16; ++n)
        cm[n * 2 + m] = wo_f32_to_f16(expected[m * 16 + n]);
    expect(runner::check_output(o, cm.data(), rows, expected).ok, "column-major indexing");
    o.m = 100;
    o.check_rows = 5;
    std::vector<int> sample = runner::rows_to_check(o);
    expect(sample.size() == 5 && sample.front() == 0 && sample.back() == 99, "row sample spans the matrix");
  }
  if (failures == 0)
    std::printf("runner_host_test: ok\n");
  return failures == 0 ? 0 : 1;
}
