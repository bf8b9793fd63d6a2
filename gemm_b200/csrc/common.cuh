// Shared host-side plumbing of the gemm_b200 library: the per-thread error
// string, the launch counter and the CUDA error check used by every entry point.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <atomic>

#include "../../include/gemm_b200.h"

namespace gemm_b200 {

struct ErrorSlot { char msg[512]; };

inline ErrorSlot& error_slot() {
  static thread_local ErrorSlot slot = {{0}};
  return slot;
}

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_slot().msg, sizeof(error_slot().msg), fmt, ap);
  va_end(ap);
  return code;
}

inline std::atomic<int64_t>& launch_counter() {
  static std::atomic<int64_t> n{0};
  return n;
}

inline int cuda_fail(cudaError_t e, const char* what) {
  return fail(GEMM_B200_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define GEMM_B200_CUDA_TRY(expr)                                   \
  do {                                                             \
    cudaError_t e__ = (expr);                                      \
    if (e__ != cudaSuccess) return ::gemm_b200::cuda_fail(e__, #expr); \
  } while (0)

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace gemm_b200
