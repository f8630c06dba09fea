/*
 * wave_oracle.c -- CPU restatement of the reference's deterministic references
 * for the tiled f16/bf16 GEMM and the flash-attention forward.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the parity tests,
 * the smoke test and the benchmark's cpu_baseline leg compare the CUDA path
 * against.  Nothing in the product path (the wave_cuda library or the Python
 * host mirror) may call it: the CUDA path has no CPU fallback.
 *
 * Parity status: PINNED.  Every function below is checked in the test suite
 * against (a) the known-answer vectors held by the reference's own tests and
 * (b) golden vectors produced by running the reference's Python references,
 * and (where the reference checkout is present) against the reference's C++
 * runner code compiled as a shared object.
 *
 * Reference functions restated here (paths relative to the reference tree):
 *   python/mlir/dialects/wave_matmul.py:828-852   LCG values, f16/bf16 rounding
 *   python/mlir/dialects/wave_matmul.py:966-994   generate_wmma_f16_matmul_inputs
 *   python/mlir/dialects/wave_matmul.py:997-1022  _reference_tile (k ascending)
 *   tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp:633-744
 *                                                  half/bf16 conversion, LCG,
 *                                                  rand_int / HPL generators
 *   tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp:1156-1196
 *                                                  make16BitInputBytes
 *   tools/wave-matmul-calibrate/wave-matmul-calibrate-runner.cpp:1586-1595
 *                                                  computeExpectedElement (f32)
 *   python/mlir/dialects/wave_attention.py:210-278 toy FA inputs + exp2 reference
 *   tools/wave-fa-calibrate/wave-fa-gfx950-runner.cpp:178-279
 *                                                  bf16 inputs, f64 attention row
 *
 * Extensions that the reference does not have (labelled where they appear):
 * a causal mask (key <= row), a caller-supplied softmax scale, f16 inputs for
 * the f64 attention row, and multi-threading over independent outputs.  None
 * changes the arithmetic of any single output element.
 */
#define _GNU_SOURCE
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define WO_F16 0
#define WO_BF16 1

#define WO_MODE_LCG 0      /* seed/stream LCG, 17 buckets of 0.25        */
#define WO_MODE_ALL_ONES 1 /* every element 1.0                          */
#define WO_MODE_RAND_INT 2 /* index hash, ints in {-2..2}, B sign flips  */
#define WO_MODE_HPL 3      /* index hash, uniform in (-0.5, 0.5)         */
#define WO_MODE_HALVES 4   /* first half 1.0, second half 2.0 (Python)   */

/* ------------------------------------------------------------------ */
/* 16-bit float conversions                                            */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float v) {
  uint32_t b;
  memcpy(&b, &v, sizeof b);
  return b;
}
static inline float bits_f32(uint32_t b) {
  float v;
  memcpy(&v, &b, sizeof v);
  return v;
}

/* runner.cpp:672-677 / wave_matmul.py:843-846: add 0x7FFF + lsb, truncate. */
uint16_t wo_f32_to_bf16(float v) {
  uint32_t b = f32_bits(v);
  b += 0x7FFFu + ((b >> 16) & 1u);
  return (uint16_t)(b >> 16);
}
float wo_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* Round-to-nearest-even f32 -> IEEE binary16, written out by hand so the
 * result does not depend on compiler half-float support.  The reference uses
 * struct.pack("<e") (wave_matmul.py:839-840) and a _Float16 cast
 * (runner.cpp:665-670); both are RNE. */
uint16_t wo_f32_to_f16(float v) {
  uint32_t b = f32_bits(v);
  uint32_t sign = (b >> 16) & 0x8000u;
  uint32_t absb = b & 0x7FFFFFFFu;
  if (absb >= 0x7F800000u) /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | (absb > 0x7F800000u ? 0x200u : 0u));
  if (absb >= 0x477FF000u) /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7C00u);
  if (absb < 0x38800000u) { /* result is subnormal or zero */
    if (absb < 0x33000000u) /* below half of the smallest subnormal */
      return (uint16_t)sign;
    int exp = (int)(absb >> 23);
    uint32_t mant = (absb & 0x7FFFFFu) | 0x800000u;
    int shift = 126 - exp; /* 14..24 */
    uint32_t half = mant >> shift;
    uint32_t rem = mant & ((1u << shift) - 1u);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1u)))
      half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((absb >> 13) & 0x3FFu) | ((((absb >> 23) - 112u)) << 10);
  uint32_t rem = absb & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u)))
    half++;
  return (uint16_t)(sign | half);
}

/* runner.cpp:633-663 (halfToFloat). */
float wo_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t mant = h & 0x3FFu;
  if (exp == 0) {
    if (mant == 0)
      return bits_f32(sign);
    int e = 1;
    while ((mant & 0x400u) == 0) {
      mant <<= 1;
      --e;
    }
    mant &= 0x3FFu;
    return bits_f32(sign | ((uint32_t)(e + 112) << 23) | (mant << 13));
  }
  if (exp == 0x1F)
    return bits_f32(sign | 0x7F800000u | (mant << 13));
  return bits_f32(sign | ((exp + 112u) << 23) | (mant << 13));
}

static inline uint16_t to_bits(int type, float v) {
  return type == WO_BF16 ? wo_f32_to_bf16(v) : wo_f32_to_f16(v);
}
static inline float from_bits(int type, uint16_t h) {
  return type == WO_BF16 ? wo_bf16_to_f32(h) : wo_f16_to_f32(h);
}

void wo_round_array(const float *in, uint16_t *out, size_t count, int type) {
  for (size_t i = 0; i < count; ++i)
    out[i] = to_bits(type, in[i]);
}
void wo_widen_array(const uint16_t *in, float *out, size_t count, int type) {
  for (size_t i = 0; i < count; ++i)
    out[i] = from_bits(type, in[i]);
}

/* ------------------------------------------------------------------ */
/* Input generators                                                    */
/* ------------------------------------------------------------------ */

/* wave_matmul.py:828-836, wave_attention.py:210-218, runner.cpp:681-694:
 * state = seed ^ ((stream+1) * 0x9E3779B9); state = 1664525*state+1013904223;
 * value = (((state >> 24) % 17) - 8) * scale.  */
void wo_lcg_values(float *out, size_t count, int seed, int stream,
                   float scale) {
  uint32_t state = (uint32_t)seed ^ ((uint32_t)(stream + 1) * 0x9E3779B9u);
  for (size_t i = 0; i < count; ++i) {
    state = 1664525u * state + 1013904223u;
    int bucket = (int)((state >> 24) % 17u) - 8;
    out[i] = (float)bucket * scale;
  }
}

/* runner.cpp:696-716. */
static uint64_t xorshift_mix(uint64_t s) {
  return s ^ (s << 13) ^ (s >> 17) ^ (s << 5);
}
static uint32_t index_hash(size_t index) {
  uint64_t s = (uint64_t)index * 1664525u + 1013904223u;
  s = xorshift_mix(s);
  s = xorshift_mix(s);
  s = xorshift_mix(s);
  return (uint32_t)s;
}
float wo_rand_int_value(size_t index) {
  return (float)(index_hash(index) % 5u) - 2.0f;
}
float wo_hpl_value(size_t index) {
  return (float)((double)index_hash(index) / (double)UINT32_MAX - 0.5);
}

/* runner.cpp:1156-1196 (make16BitInputBytes) plus the Python non-random fill
 * of wave_matmul.py:985-989 (mode WO_MODE_HALVES).  `k` is the row length and
 * only matters for the rand_int sign flip of stream 1. */
int wo_make_input_bits(uint16_t *out, size_t elements, int k, int type,
                       int seed, int stream, int mode) {
  if (type != WO_F16 && type != WO_BF16)
    return -1;
  switch (mode) {
  case WO_MODE_ALL_ONES:
    for (size_t i = 0; i < elements; ++i)
      out[i] = to_bits(type, 1.0f);
    return 0;
  case WO_MODE_HALVES: {
    size_t half = elements / 2;
    for (size_t i = 0; i < elements; ++i)
      out[i] = to_bits(type, i < half ? 1.0f : 2.0f);
    return 0;
  }
  case WO_MODE_HPL:
    for (size_t i = 0; i < elements; ++i)
      out[i] = to_bits(type, wo_hpl_value(i));
    return 0;
  case WO_MODE_RAND_INT:
    if (k <= 0)
      return -1;
    for (size_t i = 0; i < elements; ++i) {
      float v = wo_rand_int_value(i);
      size_t row = i / (size_t)k, col = i % (size_t)k;
      if (stream == 1 && ((row ^ col) & 1u) == 0)
        v = -v;
      out[i] = to_bits(type, v);
    }
    return 0;
  case WO_MODE_LCG: {
    uint32_t state = (uint32_t)seed ^ ((uint32_t)(stream + 1) * 0x9E3779B9u);
    for (size_t i = 0; i < elements; ++i) {
      state = 1664525u * state + 1013904223u;
      int bucket = (int)((state >> 24) % 17u);
      out[i] = to_bits(type, (float)((bucket - 8) * 0.25f));
    }
    return 0;
  }
  default:
    return -1;
  }
}

/* wave-fa-gfx950-runner.cpp:188-202 (makeInput): bf16 LCG values, Q/K scale
 * 0.125*inputScale, V scale 0.25; streams 0,1,2.  Also serves the toy kernel's
 * f16 inputs (wave_attention.py:225-245) through `type`. */
void wo_fa_input_bits(uint16_t *out, size_t count, int type, int seed,
                      int stream, float scale) {
  uint32_t state = (uint32_t)seed ^ ((uint32_t)(stream + 1) * 0x9E3779B9u);
  for (size_t i = 0; i < count; ++i) {
    state = 1664525u * state + 1013904223u;
    int bucket = (int)((state >> 24) % 17u) - 8;
    out[i] = to_bits(type, (float)bucket * scale);
  }
}

/* ------------------------------------------------------------------ */
/* Thread helper                                                       */
/* ------------------------------------------------------------------ */

typedef void (*wo_task_fn)(void *ctx, size_t task);
typedef struct {
  wo_task_fn fn;
  void *ctx;
  size_t ntasks;
  size_t next;
  pthread_mutex_t mu;
} wo_pool;

static void *wo_pool_worker(void *p) {
  wo_pool *pool = (wo_pool *)p;
  for (;;) {
    pthread_mutex_lock(&pool->mu);
    size_t t = pool->next++;
    pthread_mutex_unlock(&pool->mu);
    if (t >= pool->ntasks)
      return NULL;
    pool->fn(pool->ctx, t);
  }
}

static void wo_parallel_for(wo_task_fn fn, void *ctx, size_t ntasks,
                            int nthreads) {
  if (nthreads < 1)
    nthreads = 1;
  if ((size_t)nthreads > ntasks)
    nthreads = (int)(ntasks ? ntasks : 1);
  wo_pool pool = {fn, ctx, ntasks, 0, PTHREAD_MUTEX_INITIALIZER};
  if (nthreads == 1) {
    wo_pool_worker(&pool);
    return;
  }
  pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)nthreads);
  int started = 0;
  for (int i = 0; i < nthreads; ++i)
    if (pthread_create(&th[i], NULL, wo_pool_worker, &pool) == 0)
      th[started++] = th[i];
  if (started == 0)
    wo_pool_worker(&pool);
  for (int i = 0; i < started; ++i)
    pthread_join(th[i], NULL);
  free(th);
}

/* ------------------------------------------------------------------ */
/* GEMM reference                                                      */
/* ------------------------------------------------------------------ */

/* One output element exactly as runner.cpp:1586-1595 writes it: f32
 * accumulator starting at zero, k ascending, acc += lhs * rhs.  Products of
 * two f16 or two bf16 values are exact in f32, so a fused multiply-add gives
 * the same bits as a separate multiply and add. */
float wo_gemm_element(const uint16_t *A, const uint16_t *B, int K, int type,
                      int m, int n) {
  const uint16_t *a = A + (size_t)m * (size_t)K;
  const uint16_t *b = B + (size_t)n * (size_t)K;
  float acc = 0.0f;
  for (int k = 0; k < K; ++k)
    acc += from_bits(type, a[k]) * from_bits(type, b[k]);
  return acc;
}

/* The same arithmetic for many outputs at once.  A is M x K row-major, B is
 * N x K row-major (the reference stores B as its transpose:
 * wave_matmul.py:328-332).  Eight columns are carried side by side in one
 * vector, each lane keeping its own k-ascending f32 chain, so every output has
 * the bits wo_gemm_element() would give.  `rows` selects the output rows to
 * compute (NULL = all M rows); out is [nrows][N] f32 row-major. */
typedef float wo_v8 __attribute__((vector_size(32)));

typedef struct {
  const float *Af; /* [M][K] widened */
  const float *Bf; /* [N][K] widened */
  const int *rows;
  int nrows, N, K;
  float *out;
} wo_gemm_ctx;

#define WO_NB 16 /* columns per task panel */

static void wo_gemm_panel(void *vctx, size_t task) {
  wo_gemm_ctx *c = (wo_gemm_ctx *)vctx;
  const int K = c->K, N = c->N;
  int n0 = (int)task * WO_NB;
  int nb = N - n0 < WO_NB ? N - n0 : WO_NB;
  /* Transposed panel Bt[k][16], zero padded. */
  float *Bt = (float *)aligned_alloc(64, (size_t)K * WO_NB * sizeof(float));
  for (int k = 0; k < K; ++k)
    for (int j = 0; j < WO_NB; ++j)
      Bt[(size_t)k * WO_NB + j] =
          j < nb ? c->Bf[(size_t)(n0 + j) * (size_t)K + k] : 0.0f;
  int r = 0;
  for (; r + 4 <= c->nrows; r += 4) {
    const float *a0 = c->Af + (size_t)(c->rows ? c->rows[r + 0] : r + 0) * K;
    const float *a1 = c->Af + (size_t)(c->rows ? c->rows[r + 1] : r + 1) * K;
    const float *a2 = c->Af + (size_t)(c->rows ? c->rows[r + 2] : r + 2) * K;
    const float *a3 = c->Af + (size_t)(c->rows ? c->rows[r + 3] : r + 3) * K;
    wo_v8 c00 = {0}, c01 = {0}, c10 = {0}, c11 = {0};
    wo_v8 c20 = {0}, c21 = {0}, c30 = {0}, c31 = {0};
    for (int k = 0; k < K; ++k) {
      const wo_v8 *bt = (const wo_v8 *)(Bt + (size_t)k * WO_NB);
      wo_v8 b0 = bt[0], b1 = bt[1];
      c00 += a0[k] * b0;
      c01 += a0[k] * b1;
      c10 += a1[k] * b0;
      c11 += a1[k] * b1;
      c20 += a2[k] * b0;
      c21 += a2[k] * b1;
      c30 += a3[k] * b0;
      c31 += a3[k] * b1;
    }
    wo_v8 acc[4][2] = {{c00, c01}, {c10, c11}, {c20, c21}, {c30, c31}};
    for (int i = 0; i < 4; ++i)
      for (int j = 0; j < nb; ++j)
        c->out[(size_t)(r + i) * N + n0 + j] = acc[i][j / 8][j % 8];
  }
  for (; r < c->nrows; ++r) {
    const float *a0 = c->Af + (size_t)(c->rows ? c->rows[r] : r) * K;
    wo_v8 c00 = {0}, c01 = {0};
    for (int k = 0; k < K; ++k) {
      const wo_v8 *bt = (const wo_v8 *)(Bt + (size_t)k * WO_NB);
      c00 += a0[k] * bt[0];
      c01 += a0[k] * bt[1];
    }
    wo_v8 acc[2] = {c00, c01};
    for (int j = 0; j < nb; ++j)
      c->out[(size_t)r * N + n0 + j] = acc[j / 8][j % 8];
  }
  free(Bt);
}

int wo_gemm_ref(const uint16_t *A, const uint16_t *B, int M, int N, int K,
                int type, const int *rows, int nrows, float *out,
                int nthreads) {
  if (M <= 0 || N <= 0 || K <= 0 || (type != WO_F16 && type != WO_BF16))
    return -1;
  if (!rows)
    nrows = M;
  float *Af = (float *)malloc((size_t)M * K * sizeof(float));
  float *Bf = (float *)malloc((size_t)N * K * sizeof(float));
  if (!Af || !Bf) {
    free(Af);
    free(Bf);
    return -2;
  }
  wo_widen_array(A, Af, (size_t)M * K, type);
  wo_widen_array(B, Bf, (size_t)N * K, type);
  wo_gemm_ctx ctx = {Af, Bf, rows, nrows, N, K, out};
  wo_parallel_for(wo_gemm_panel, &ctx, (size_t)((N + WO_NB - 1) / WO_NB),
                  nthreads);
  free(Af);
  free(Bf);
  return 0;
}

/* ------------------------------------------------------------------ */
/* Flash-attention references                                          */
/* ------------------------------------------------------------------ */

typedef struct {
  const uint16_t *Q, *K, *V;
  int type, seq_q, seq_k, D;
  double scale;
  int causal, exp2_mode;
  const int *heads, *rows;
  int nheads, nrows;
  float *out;  /* [nheads][nrows][D] */
  double *lse; /* [nheads][nrows] natural-log sum-exp of scaled scores, or NULL */
} wo_fa_ctx;

/* One output row.  Non-causal, exp2_mode == 0 is computeAttentionRow of
 * wave-fa-gfx950-runner.cpp:247-279: scores = (q.k) * scale in f64, subtract
 * the row maximum, exp, normalise, weighted sum of V in key order, final cast
 * to f32.  exp2_mode == 1 is compute_flash_attention_f32_reference of
 * wave_attention.py:248-278, which uses 2**(s - max) on unscaled scores (its
 * caller pre-multiplies Q).  causal != 0 (an extension: the reference has no
 * causal Wave kernel) keeps only keys with index <= row, the top-left-aligned
 * mask used by integrations/tlx/workloads/amd-fa-pipelined_test.py:173-177. */
static void wo_fa_row(void *vctx, size_t task) {
  wo_fa_ctx *c = (wo_fa_ctx *)vctx;
  int hi = (int)(task / (size_t)c->nrows), ri = (int)(task % (size_t)c->nrows);
  int head = c->heads ? c->heads[hi] : hi;
  int row = c->rows ? c->rows[ri] : ri;
  const int D = c->D;
  const uint16_t *q = c->Q + ((size_t)head * c->seq_q + row) * D;
  const uint16_t *kb = c->K + (size_t)head * c->seq_k * D;
  const uint16_t *vb = c->V + (size_t)head * c->seq_k * D;
  int nkeys = c->seq_k;
  if (c->causal && row + 1 < nkeys)
    nkeys = row + 1;
  double *scores = (double *)malloc(sizeof(double) * (size_t)nkeys);
  double *qd = (double *)malloc(sizeof(double) * (size_t)D);
  for (int d = 0; d < D; ++d)
    qd[d] = (double)from_bits(c->type, q[d]);
  double row_max = -INFINITY;
  for (int key = 0; key < nkeys; ++key) {
    const uint16_t *kr = kb + (size_t)key * D;
    double s = 0.0;
    for (int d = 0; d < D; ++d)
      s += qd[d] * (double)from_bits(c->type, kr[d]);
    s *= c->scale;
    scores[key] = s;
    if (s > row_max)
      row_max = s;
  }
  double denom = 0.0;
  for (int key = 0; key < nkeys; ++key) {
    double w = c->exp2_mode ? exp2(scores[key] - row_max)
                            : exp(scores[key] - row_max);
    scores[key] = w;
    denom += w;
  }
  float *o = c->out + ((size_t)hi * c->nrows + ri) * D;
  for (int d = 0; d < D; ++d) {
    double sum = 0.0;
    for (int key = 0; key < nkeys; ++key)
      sum += scores[key] * (double)from_bits(c->type, vb[(size_t)key * D + d]);
    o[d] = (float)(sum / denom);
  }
  if (c->lse)
    c->lse[(size_t)hi * c->nrows + ri] =
        c->exp2_mode ? (row_max + log2(denom)) : (row_max + log(denom));
  free(scores);
  free(qd);
}

int wo_fa_ref(const uint16_t *Q, const uint16_t *K, const uint16_t *V, int type,
              int n_heads_total, int seq_q, int seq_k, int D, double scale,
              int causal, int exp2_mode, const int *heads, int nheads,
              const int *rows, int nrows, float *out, double *lse,
              int nthreads) {
  if (n_heads_total <= 0 || seq_q <= 0 || seq_k <= 0 || D <= 0)
    return -1;
  if (type != WO_F16 && type != WO_BF16)
    return -1;
  if (!heads)
    nheads = n_heads_total;
  if (!rows)
    nrows = seq_q;
  wo_fa_ctx ctx = {Q,      K,      V,    type,  seq_q,  seq_k, D,   scale,
                   causal, exp2_mode, heads, rows, nheads, nrows, out, lse};
  wo_parallel_for(wo_fa_row, &ctx, (size_t)nheads * (size_t)nrows, nthreads);
  return 0;
}

/* Sampling rule of wave-fa-gfx950-runner.cpp:204-232: all heads when there are
 * at most four, else {0, mid, last}; all rows when sequence <= 512, else
 * {0, 31, 32, 127, S/2, S-128, S-1} sorted and de-duplicated.  Returns the
 * count written (heads: <= 4, rows: <= max(512, 7) -- the caller sizes it). */
int wo_fa_sample_heads(int total_heads, int *out) {
  if (total_heads <= 4) {
    for (int i = 0; i < total_heads; ++i)
      out[i] = i;
    return total_heads;
  }
  out[0] = 0;
  out[1] = total_heads / 2;
  out[2] = total_heads - 1;
  return 3;
}
static int cmp_int(const void *a, const void *b) {
  return *(const int *)a - *(const int *)b;
}
int wo_fa_sample_rows(int sequence, int *out) {
  if (sequence <= 512) {
    for (int i = 0; i < sequence; ++i)
      out[i] = i;
    return sequence;
  }
  int rows[7] = {0, 31, 32, 127, sequence / 2, sequence - 128, sequence - 1};
  qsort(rows, 7, sizeof(int), cmp_int);
  int n = 0;
  for (int i = 0; i < 7; ++i)
    if (n == 0 || out[n - 1] != rows[i])
      out[n++] = rows[i];
  return n;
}
