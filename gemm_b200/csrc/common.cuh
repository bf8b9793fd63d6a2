// Shared host-side plumbing of the gemm_b200 library: the per-thread error
// string, the launch counter and the CUDA error check used by every entry point.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <stdlib.h>
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

// Environment knobs (read once):
//   GEMM_B200_LOG=1                 one line on stderr per launch with the kernel variant chosen
//   GEMM_B200_F32_CONFIG / GEMM_B200_BF16_CONFIG / GEMM_B200_MXFP8_CONFIG = <index>
//                                   force a variant wherever the caller asked for the heuristic
inline int env_int(const char* name, int fallback) {
  const char* e = getenv(name);
  return (e && *e) ? atoi(e) : fallback;
}
inline bool log_enabled() {
  static const bool on = env_int("GEMM_B200_LOG", 0) != 0;
  return on;
}

}  // namespace gemm_b200
