/*
 * Exposes the HOST arithmetic of the reference's GEMM calibrate runner
 * (tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp) through a C
 * ABI, by including that source where it lies in the reference checkout with
 * its own WAVE_MATMUL_CALIBRATE_RUNNER_NO_MAIN hook (runner.cpp:1835).  No
 * reference source is copied.  Test infrastructure only: used to validate the
 * restated oracle and, optionally, as the timed CPU baseline.
 */
#define WAVE_MATMUL_CALIBRATE_RUNNER_NO_MAIN
#include WAVE_REF_GEMM_RUNNER

#include <thread>

static InputType shimInputType(int type) {
  return type == 1 ? InputType::BF16 : InputType::F16;
}

extern "C" {

/* makeInputBytes (runner.cpp:1198-...) -> 16-bit patterns.  mode: 0 LCG,
 * 1 all-ones, 2 rand_int, 3 HPL. */
int wave_ref_make_input_bits(uint16_t *out, int rows, int k, int type, int seed,
                             int stream, int mode) {
  std::vector<uint8_t> bytes =
      makeInputBytes(rows, k, shimInputType(type), seed, stream, mode == 1,
                     mode == 2, mode == 3);
  std::memcpy(out, bytes.data(), bytes.size());
  return static_cast<int>(bytes.size() / 2);
}

/* computeExpectedElement (runner.cpp:1586-1595) over selected rows, spread
 * over `nthreads` host threads.  out is [nrows][n] f32. */
int wave_ref_gemm_rows(const uint16_t *a, const uint16_t *b, int m, int n,
                       int k, int type, const int *rows, int nrows, float *out,
                       int nthreads) {
  Args args;
  args.m = m;
  args.n = n;
  args.k = k;
  args.inputType = shimInputType(type);
  HostInputs inputs;
  inputs.a.assign(reinterpret_cast<const uint8_t *>(a),
                  reinterpret_cast<const uint8_t *>(a) +
                      static_cast<size_t>(m) * k * 2);
  inputs.b.assign(reinterpret_cast<const uint8_t *>(b),
                  reinterpret_cast<const uint8_t *>(b) +
                      static_cast<size_t>(n) * k * 2);
  if (!rows)
    nrows = m;
  if (nthreads < 1)
    nthreads = 1;
  std::vector<std::thread> pool;
  for (int t = 0; t < nthreads; ++t)
    pool.emplace_back([&, t] {
      for (int r = t; r < nrows; r += nthreads) {
        int row = rows ? rows[r] : r;
        for (int col = 0; col < n; ++col)
          out[static_cast<size_t>(r) * n + col] =
              computeExpectedElement(inputs, args, row, col);
      }
    });
  for (std::thread &th : pool)
    th.join();
  return 0;
}

/* roundExpectedOutput (runner.cpp:738-744): ctype 0 f32, 1 f16, 2 bf16. */
double wave_ref_round_output(double value, int ctype) {
  return roundExpectedOutput(value, ctype == 1   ? CType::F16
                                    : ctype == 2 ? CType::BF16
                                                 : CType::F32);
}

/* Stream-K workspace sizing (runner.cpp:393-408). */
size_t wave_ref_streamk_scratch_bytes(int workers) {
  Args args;
  args.m = 256;
  args.n = 256;
  args.streamKWorkers = workers;
  return getStreamKWorkspaceSizes(args).scratchBytes;
}
/* getOutputCoordinate (runner.cpp:809-836): packed index -> (m, n) for the
 * fragment layouts.  wmma: 1 WMMA, 0 MFMA accumulator layout. */
int wave_ref_output_coordinate(int m, int n, int bm, int bn, int wave_m_tiles,
                               int wave_n_tiles, int wmma, int wave_size,
                               int index, int *out_mn) {
  Args args;
  args.m = m;
  args.n = n;
  args.bm = bm;
  args.bn = bn;
  args.waveMTiles = wave_m_tiles;
  args.waveNTiles = wave_n_tiles;
  args.accumulatorLayout = wmma ? AccumulatorLayout::Wmma : AccumulatorLayout::Mfma;
  args.waveSize = wave_size;
  OutputCoordinate c = getOutputCoordinate(args, index);
  out_mn[0] = c.m;
  out_mn[1] = c.n;
  return 0;
}
size_t wave_ref_streamk_counter_elements(int m, int n) {
  Args args;
  args.m = m;
  args.n = n;
  return getStreamKWorkspaceSizes(args).counterElements;
}
}
