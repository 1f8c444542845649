/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the Matmul -> row-Softmax chain.
 *
 * This file is the checker for the CUDA path: it is loaded by the test-suite,
 * by the smoke check and by the benchmark's CPU-baseline leg, and by nothing
 * else.  The product never calls into it and has no CPU fallback.
 *
 * What is restated (reference project paths):
 *   - operator order and initial values: mlir/matmul_softmax_chain.mlir:15-80
 *       C = A.B (fill 0 + matmul), max (init -3.4028235e38), exp(C-max),
 *       sum (init 0), divide.
 *   - where the f16 casts sit:           mlir/matmul_softmax_chain_f16_native.mlir:13-31
 *   - named softmax == the decomposed form: compiler/ir/ChainCanonicalize.cpp:62-71,145-159
 *   - checker math (f64 accumulate, max-subtracted softmax):
 *       backend/welder/bench/verify_matmul_softmax.py:242-265
 *   - loop structure of the timed baseline (scalar i,j,k nest, then four
 *     separate row passes): bench/baselines/default/fused/04c.after_linalg_to_loops.mlir
 *   - input generators: backend/welder/compiler/solver/WelderProfilerRuntime.h:128-168,193-231
 *   - f32->f16 conversions: round-to-nearest-even as
 *       backend/welder/bench/verify_matmul_softmax.py:66-107, and the profiler's
 *       add-half-then-truncate as backend/welder/compiler/solver/WelderProfilerEval.h:50-100.
 *
 * Parity pin: the generators and both f16 conversions are checked bit-for-bit
 * against vectors produced by importing the reference's Python checker and by
 * compiling the reference's profiler headers (tests/golden); the chain math is
 * checked by running the reference's unmodified checker on dumps of this
 * oracle's output.  The reference ships no numeric golden outputs of its own.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define WTC_DT_F32 0
#define WTC_DT_F16 1

/* accumulate modes for the contraction */
#define WTC_ACC_F64 0      /* checker: Python-float accumulate            */
#define WTC_ACC_F32_SEQ 1  /* loop lowering with outs(f32): k-sequential  */
#define WTC_ACC_F16_SEQ 2  /* loop lowering with outs(f16): round per add */

/* ---------- f16 <-> f32 ---------- */

/* round-to-nearest-even, verify_matmul_softmax.py:66-107 */
uint16_t wtc_oracle_f32_to_f16_rne(float x) {
  uint32_t u; memcpy(&u, &x, 4);
  uint32_t sign = (u >> 31) & 1u, exp = (u >> 23) & 0xFFu, mant = u & 0x7FFFFFu;
  if (exp == 0xFF) {
    if (mant == 0) return (uint16_t)((sign << 15) | 0x7C00u);
    return (uint16_t)((sign << 15) | 0x7C00u | ((mant >> 13) & 0x3FFu) | 1u);
  }
  int e16 = (int)exp - 127 + 15;
  if (e16 >= 31) return (uint16_t)((sign << 15) | 0x7C00u);
  if (e16 <= 0) {
    if (e16 < -10) return (uint16_t)(sign << 15);
    mant |= 0x800000u;
    int shift = 1 - e16;
    uint32_t m16 = mant >> (shift + 13);
    uint32_t rem = mant & ((1u << (shift + 13)) - 1u);
    uint32_t half = 1u << (shift + 12);
    if (rem > half || (rem == half && (m16 & 1u))) m16 += 1;
    return (uint16_t)((sign << 15) | (m16 & 0x3FFu));
  }
  uint32_t m16 = mant >> 13, rem = mant & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (m16 & 1u))) {
    m16 += 1;
    if (m16 == 0x400u) { m16 = 0; e16 += 1; if (e16 >= 31) return (uint16_t)((sign << 15) | 0x7C00u); }
  }
  return (uint16_t)((sign << 15) | ((uint32_t)(e16 & 0x1F) << 10) | (m16 & 0x3FFu));
}

/* add-half-then-truncate, WelderProfilerEval.h:50-100 (ties go up, not to even) */
uint16_t wtc_oracle_f32_to_f16_profiler(float x) {
  uint32_t u; memcpy(&u, &x, 4);
  uint32_t sign = (u >> 31) & 1u; int exp = (int)((u >> 23) & 0xFFu); uint32_t mant = u & 0x7FFFFFu;
  uint16_t s = (uint16_t)(sign << 15);
  if (exp == 0xFF) return (uint16_t)(s | (mant == 0 ? 0x7C00u : 0x7E00u));
  int he = exp - 127 + 15;
  if (he >= 31) return (uint16_t)(s | 0x7C00u);
  if (he <= 0) {
    if (he < -10) return s;
    mant |= 0x800000u;
    int shift = 14 - he;
    uint32_t r = mant + (1u << (shift - 1));
    return (uint16_t)(s | (uint16_t)(r >> shift));
  }
  uint32_t r = mant + 0x1000u;
  if (r & 0x800000u) { r = 0; ++he; if (he >= 31) return (uint16_t)(s | 0x7C00u); }
  return (uint16_t)(s | (uint16_t)(he << 10) | (uint16_t)((r >> 13) & 0x3FFu));
}

float wtc_oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
  float v;
  if (exp == 0) v = ldexpf((float)mant, -24);
  else if (exp == 31) v = mant ? NAN : INFINITY;
  else v = ldexpf((float)(mant | 0x400u), (int)exp - 25);
  return sign ? -v : v;
}

/* ---------- input generators, WelderProfilerRuntime.h:128-168 ---------- */

static inline float linear_val(int64_t flat) { return (float)(flat % 1024) * 0.001f - 0.5f; }

static inline float xorshift_next(uint32_t *rng) {
  uint32_t r = *rng;
  r ^= r << 13; r ^= r >> 17; r ^= r << 5;
  *rng = r;
  return (float)r * (1.0f / 4294967296.0f) * 2.0f - 1.0f;
}

/* mode: 0 zero, 1 linear, 2 random.  Dense row-major buffer of `count` elements. */
void wtc_oracle_fill_f32(float *dst, int64_t count, int mode, uint64_t seed) {
  uint32_t rng = (uint32_t)(seed == 0 ? 1 : seed);
  for (int64_t i = 0; i < count; ++i)
    dst[i] = mode == 0 ? 0.0f : (mode == 2 ? xorshift_next(&rng) : linear_val(i));
}

/* f16 buffers: same streams, converted with the profiler's own conversion
 * (conv = 0) or with round-to-nearest-even (conv = 1). */
void wtc_oracle_fill_f16(uint16_t *dst, int64_t count, int mode, uint64_t seed, int conv) {
  uint32_t rng = (uint32_t)(seed == 0 ? 1 : seed);
  for (int64_t i = 0; i < count; ++i) {
    float v = mode == 0 ? 0.0f : (mode == 2 ? xorshift_next(&rng) : linear_val(i));
    dst[i] = conv ? wtc_oracle_f32_to_f16_rne(v) : wtc_oracle_f32_to_f16_profiler(v);
  }
}

/* ---------- the chain ---------- */

static inline double load_elem(const void *p, int dt, int64_t idx) {
  return dt == WTC_DT_F16 ? (double)wtc_oracle_f16_to_f32(((const uint16_t *)p)[idx])
                          : (double)((const float *)p)[idx];
}

/*
 * probs[b,i,j] = softmax_j(scale * sum_k A[b,i,k] * B[b,k,j]) as f64.
 * A: [batch,M,K] row-major (lda = K), B: [batch,K,N] row-major (ldb = N),
 * b_batch_stride may be 0 to share one B across batches.
 * Optional outputs: logits (f64, scaled), row_max, row_sum (of exp(s-max)).
 * threads <= 0 means "all".  Returns 0, or 1 on bad arguments.
 */
int wtc_oracle_chain(const void *A, const void *B, double *probs, double *logits_out,
                     int64_t batch, int64_t M, int64_t N, int64_t K,
                     int in_dtype, double scale, int acc_mode, int64_t b_batch_stride,
                     int threads) {
  if (!A || !B || !probs || batch <= 0 || M < 0 || N < 0 || K < 0) return 1;
  if (in_dtype != WTC_DT_F32 && in_dtype != WTC_DT_F16) return 1;
  if (M == 0 || N == 0) return 0;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  /* widen B once so the inner loop is a plain fma stream */
  int64_t b_elems = (b_batch_stride == 0 ? 1 : batch) * K * N;
  double *Bd = (double *)malloc(sizeof(double) * (size_t)(b_elems > 0 ? b_elems : 1));
  if (!Bd) return 1;
  for (int64_t i = 0; i < b_elems; ++i) Bd[i] = load_elem(B, in_dtype, i);

  int64_t rows = batch * M;
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)N);
    double *arow = (double *)malloc(sizeof(double) * (size_t)(K > 0 ? K : 1));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      int64_t b = r / M;
      const double *Bb = Bd + (b_batch_stride == 0 ? 0 : b * K * N);
      for (int64_t k = 0; k < K; ++k) arow[k] = load_elem(A, in_dtype, r * K + k);
      if (acc_mode == WTC_ACC_F64) {
        for (int64_t j = 0; j < N; ++j) acc[j] = 0.0;
        for (int64_t k = 0; k < K; ++k) {
          double a = arow[k]; const double *brow = Bb + k * N;
          for (int64_t j = 0; j < N; ++j) acc[j] += a * brow[j];
        }
      } else if (acc_mode == WTC_ACC_F32_SEQ) {
        for (int64_t j = 0; j < N; ++j) {
          float s = 0.0f;
          for (int64_t k = 0; k < K; ++k) s = s + (float)arow[k] * (float)Bb[k * N + j];
          acc[j] = (double)s;
        }
      } else {
        for (int64_t j = 0; j < N; ++j) {
          float s = 0.0f;  /* value always representable in f16 */
          for (int64_t k = 0; k < K; ++k) {
            float p = wtc_oracle_f16_to_f32(wtc_oracle_f32_to_f16_rne((float)arow[k] * (float)Bb[k * N + j]));
            s = wtc_oracle_f16_to_f32(wtc_oracle_f32_to_f16_rne(s + p));
          }
          acc[j] = (double)s;
        }
      }
      double mx = -3.4028234663852886e38;
      for (int64_t j = 0; j < N; ++j) { acc[j] *= scale; if (acc[j] > mx) mx = acc[j]; }
      if (logits_out) memcpy(logits_out + r * N, acc, sizeof(double) * (size_t)N);
      double sum = 0.0;
      double *prow = probs + r * N;
      for (int64_t j = 0; j < N; ++j) { prow[j] = exp(acc[j] - mx); sum += prow[j]; }
      double inv = 1.0 / sum;
      for (int64_t j = 0; j < N; ++j) prow[j] *= inv;
    }
    free(acc); free(arow);
  }
  free(Bd);
  return 0;
}

/*
 * The timed CPU baseline: the loop nest that convert-linalg-to-loops gives for
 * this chain -- scalar i,j,k matmul accumulating in f32, then separate max /
 * exp / sum / divide passes over the rows -- parallelised over rows only.
 * Inputs f32 or f16 (widened on load), output f32 [rows, N].
 */
int wtc_oracle_chain_loops_f32(const void *A, const void *B, float *out,
                               int64_t batch, int64_t M, int64_t N, int64_t K,
                               int in_dtype, float scale, int64_t b_batch_stride, int threads) {
  if (!A || !B || !out || batch <= 0 || M <= 0 || N <= 0 || K < 0) return 1;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  int64_t b_elems = (b_batch_stride == 0 ? 1 : batch) * K * N;
  float *Bf = (float *)malloc(sizeof(float) * (size_t)(b_elems > 0 ? b_elems : 1));
  if (!Bf) return 1;
  for (int64_t i = 0; i < b_elems; ++i) Bf[i] = (float)load_elem(B, in_dtype, i);
  int64_t rows = batch * M;
#pragma omp parallel
  {
    float *arow = (float *)malloc(sizeof(float) * (size_t)(K > 0 ? K : 1));
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      int64_t b = r / M;
      const float *Bb = Bf + (b_batch_stride == 0 ? 0 : b * K * N);
      float *c = out + r * N;
      for (int64_t k = 0; k < K; ++k) arow[k] = (float)load_elem(A, in_dtype, r * K + k);
      for (int64_t j = 0; j < N; ++j) c[j] = 0.0f;
      for (int64_t k = 0; k < K; ++k) {        /* i,k,j order: same sums per (i,j), k ascending */
        float a = arow[k]; const float *brow = Bb + k * N;
        for (int64_t j = 0; j < N; ++j) c[j] += a * brow[j];
      }
      float mx = -3.4028235e38f;
      for (int64_t j = 0; j < N; ++j) { c[j] *= scale; mx = c[j] > mx ? c[j] : mx; }
      for (int64_t j = 0; j < N; ++j) c[j] = expf(c[j] - mx);
      float sum = 0.0f;
      for (int64_t j = 0; j < N; ++j) sum += c[j];
      for (int64_t j = 0; j < N; ++j) c[j] = c[j] / sum;
    }
    free(arow);
  }
  free(Bf);
  return 0;
}

int wtc_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
