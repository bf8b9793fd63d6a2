/* A caller of the C-ABI that knows nothing of Python, torch or CUDA headers: plain C, host arrays,
 * include/gemm_b200.h and -lgemm_b200.  It multiplies seeded FP32 matrices through
 * gemm_b200_sgemm_f32_host (the entry point that replaces the reference's wrapper + launcher,
 * naive/naive.cpp:6-22 and naive/naive_1.cu:17-24, for callers that hold host arrays), recomputes
 * the product with the reference kernels' arithmetic (one FP32 accumulator per element, fused
 * multiply-adds in ascending k, naive/naive_1.cu:9-12) and requires bit equality.
 * Usage: host_caller M K N   -> prints "ok <checksum>" and exits 0, or a message and a non-zero code. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "gemm_b200.h"

static uint32_t lcg(uint32_t* s) { *s = *s * 1664525u + 1013904223u; return *s; }

int main(int argc, char** argv) {
  if (argc != 4) { fprintf(stderr, "usage: %s M K N\n", argv[0]); return 2; }
  const int64_t M = atoll(argv[1]), K = atoll(argv[2]), N = atoll(argv[3]);
  if (!gemm_b200_device_supported(0)) { fprintf(stderr, "device 0 is not supported\n"); return 3; }
  float* A = (float*)malloc(sizeof(float) * (size_t)(M * K));
  float* B = (float*)malloc(sizeof(float) * (size_t)(K * N));
  float* C = (float*)malloc(sizeof(float) * (size_t)(M * N));
  if (!A || !B || !C) return 4;
  uint32_t seed = 12345u;
  for (int64_t i = 0; i < M * K; ++i) A[i] = (float)(lcg(&seed) >> 8) / 8388608.0f - 1.0f;   /* uniform [-1, 1) */
  for (int64_t i = 0; i < K * N; ++i) B[i] = (float)(lcg(&seed) >> 8) / 8388608.0f - 1.0f;
  memset(C, 0xff, sizeof(float) * (size_t)(M * N));
  const int rc = gemm_b200_sgemm_f32_host(A, B, C, M, N, K);
  if (rc != GEMM_B200_OK) { fprintf(stderr, "gemm_b200_sgemm_f32_host: %d: %s\n", rc, gemm_b200_last_error()); return 5; }
  uint64_t checksum = 0;
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) acc = fmaf(A[i * K + k], B[k * N + j], acc);
      uint32_t want, got;
      memcpy(&want, &acc, 4);
      memcpy(&got, &C[i * N + j], 4);
      if (want != got) { fprintf(stderr, "C[%lld][%lld]: got %08x, want %08x\n", (long long)i, (long long)j, got, want); return 6; }
      checksum = checksum * 1099511628211ull + got;
    }
  }
  /* a refused call reports through the same channel */
  if (gemm_b200_sgemm_f32_host(A, B, C, -1, N, K) != GEMM_B200_ERR_INVALID_ARG || !strstr(gemm_b200_last_error(), "negative")) return 7;
  printf("ok %016llx version %d launches %lld\n", (unsigned long long)checksum, gemm_b200_version(), (long long)gemm_b200_launch_count());
  free(A); free(B); free(C);
  return 0;
}
