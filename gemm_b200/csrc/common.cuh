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

// ---------------------------------------------------------------------------------------
// Bounds-checking build (-DGEMM_B200_DEBUG, `python -m gemm_b200.build --debug`): every global
// access that the kernels address themselves (TMA transfers are clipped by the tensor map in
// hardware) is first checked against the extent of its matrix.  An access that falls outside is
// NOT made: the thread records {GEMM_B200_ERR_BOUNDS, block, site, byte offset} in a status word
// of its translation unit and goes on, so a wrong index shows up as an error code on the host, never
// as a fault.  gemm_b200_debug_bounds_f32 / _tc read and clear the word.  Release builds compile
// the checks away.
// ---------------------------------------------------------------------------------------
#ifdef GEMM_B200_DEBUG
namespace dbg {
static __device__ __attribute__((unused)) int32_t g_bounds[4];
// test knob: every checked extent is understated by this many bytes, so that accesses near the end
// of a matrix are refused (and skipped) without any access ever leaving the matrix
static __device__ __attribute__((unused)) long long g_shrink;
__device__ __forceinline__ bool in_bounds(const void* p, const void* base, long long bytes, int access, int site) {
  const long long off = static_cast<const char*>(p) - static_cast<const char*>(base);
  if (off >= 0 && off + access <= bytes - g_shrink) return true;
  if (atomicCAS(&g_bounds[0], 0, GEMM_B200_ERR_BOUNDS) == 0) {
    g_bounds[1] = (int32_t)blockIdx.x;
    g_bounds[2] = site;
    g_bounds[3] = (int32_t)(off < 0 ? -1 : (off > 0x7fffffffLL ? 0x7fffffffLL : off));
  }
  return false;
}
// host side of the two debug entry points: read and clear the word, set the test knob
static inline int read_bounds(int32_t out[4], long long shrink) {
  GEMM_B200_CUDA_TRY(cudaDeviceSynchronize());
  int32_t h[4] = {0, 0, 0, 0};
  GEMM_B200_CUDA_TRY(cudaMemcpyFromSymbol(h, g_bounds, sizeof(h)));
  const int32_t z[4] = {0, 0, 0, 0};
  GEMM_B200_CUDA_TRY(cudaMemcpyToSymbol(g_bounds, z, sizeof(z)));
  GEMM_B200_CUDA_TRY(cudaMemcpyToSymbol(g_shrink, &shrink, sizeof(shrink)));
  if (out)
    for (int i = 0; i < 4; ++i) out[i] = h[i];
  return h[0];
}
}  // namespace dbg
#define GEMM_B200_IN_BOUNDS(p, base, bytes, access, site) ::gemm_b200::dbg::in_bounds(p, base, (long long)(bytes), access, site)
#else
#define GEMM_B200_IN_BOUNDS(p, base, bytes, access, site) true
#endif

}  // namespace gemm_b200
