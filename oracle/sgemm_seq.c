/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference FP32 GEMM arithmetic.
 * Only tests, the smoke check and the benchmark's CPU-baseline leg may use this file; the
 * library itself never does.
 *
 * Follows the reference kernels' arithmetic exactly:
 *   naive/naive_1.cu:9-13              float acc = 0; for k ascending: acc += A[i*K+k] * B[k*N+j]
 *   shared/shared_2.cu:20,45-47,55     same accumulator walked tile by tile, k still ascending
 *   blocktile_1d/blocktile_1d.cu:17,52-59,65   same, TM accumulators per thread
 * All three are compiled with --use_fast_math (naive/test.py:8), i.e. the multiply-add is
 * contracted into one fused multiply-add (-fmad=true) with denormal inputs and results
 * flushed to zero (-ftz=true).  `ftz` selects that flushing here.
 *
 * Loop order is i, k, j so the j loop vectorises; every C[i][j] still receives its terms in
 * ascending k through a single accumulator, which is all that determines the result bits.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float flush(float x) {
  return (fabsf(x) < FLT_MIN) ? copysignf(0.0f, x) : x;
}

void oracle_sgemm_seq(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                      int64_t lda, int64_t ldb, int64_t ldc, int ftz) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i) {
    float* c = C + i * ldc;
    for (int64_t j = 0; j < N; ++j) c[j] = 0.0f;
    for (int64_t k = 0; k < K; ++k) {
      float a = A[i * lda + k];
      const float* b = B + k * ldb;
      if (ftz) {
        a = flush(a);
        for (int64_t j = 0; j < N; ++j) c[j] = flush(fmaf(a, flush(b[j]), c[j]));
      } else {
        for (int64_t j = 0; j < N; ++j) c[j] = fmaf(a, b[j], c[j]);
      }
    }
  }
}

/* Plain FP32 GEMM with an FP32 accumulator per element and operands given as FP32 (used for
 * the BF16 / MXFP8 operand oracles on small shapes; the tensor cores add in a different order,
 * so those comparisons carry a tolerance). */
void oracle_sgemm_f64acc(const float* A, const float* B, double* C, int64_t M, int64_t N, int64_t K,
                         int64_t lda, int64_t ldb, int64_t ldc) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < M; ++i) {
    double* c = C + i * ldc;
    for (int64_t j = 0; j < N; ++j) c[j] = 0.0;
    for (int64_t k = 0; k < K; ++k) {
      const double a = (double)A[i * lda + k];
      const float* b = B + k * ldb;
      for (int64_t j = 0; j < N; ++j) c[j] += a * (double)b[j];
    }
  }
}
