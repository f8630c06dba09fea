/*
 * Exposes the HOST arithmetic of the reference's gfx950 flash-attention runner
 * (tools/wave-fa-calibrate/wave-fa-gfx950-runner.cpp) through a C ABI by
 * including that source where it lies in the reference checkout; its `main`
 * is renamed away.  No reference source is copied.  Test infrastructure only.
 */
#define main wave_ref_fa_gfx950_unused_main
#include WAVE_REF_FA_RUNNER
#undef main

#include <thread>

extern "C" {

/* makeInput (runner:188-202): bf16 LCG values. */
int wave_ref_fa_input_bits(uint16_t *out, size_t count, int seed, int stream,
                           float scale) {
  std::vector<uint16_t> values = makeInput(count, seed, stream, scale);
  std::memcpy(out, values.data(), count * sizeof(uint16_t));
  return 0;
}

/* computeAttentionRow (runner:247-279) for the given heads x rows, threaded.
 * out is [nheads][nrows][128] f32. */
int wave_ref_fa_rows(const uint16_t *q, const uint16_t *k, const uint16_t *v,
                     int batch, int heads, int sequence, const int *head_list,
                     int nheads, const int *row_list, int nrows, float *out,
                     int nthreads) {
  Args args;
  args.batch = batch;
  args.heads = heads;
  args.sequence = sequence;
  size_t elements = static_cast<size_t>(batch) * heads * sequence * kHeadDim;
  std::vector<uint16_t> qv(q, q + elements), kv(k, k + elements),
      vv(v, v + elements);
  if (nthreads < 1)
    nthreads = 1;
  int tasks = nheads * nrows;
  std::vector<std::thread> pool;
  for (int t = 0; t < nthreads; ++t)
    pool.emplace_back([&, t] {
      for (int task = t; task < tasks; task += nthreads) {
        ReferenceRow row = computeAttentionRow(args, qv, kv, vv,
                                               head_list[task / nrows],
                                               row_list[task % nrows]);
        std::memcpy(out + static_cast<size_t>(task) * kHeadDim,
                    row.values.data(), sizeof(float) * kHeadDim);
      }
    });
  for (std::thread &th : pool)
    th.join();
  return 0;
}

/* referenceHeads / referenceRows (runner:204-232). */
int wave_ref_fa_sample_heads(int batch, int heads, int *out) {
  Args args;
  args.batch = batch;
  args.heads = heads;
  std::vector<int> list = referenceHeads(args);
  std::memcpy(out, list.data(), list.size() * sizeof(int));
  return static_cast<int>(list.size());
}
int wave_ref_fa_sample_rows(int sequence, int *out) {
  Args args;
  args.sequence = sequence;
  std::vector<int> list = referenceRows(args);
  std::memcpy(out, list.data(), list.size() * sizeof(int));
  return static_cast<int>(list.size());
}
}
