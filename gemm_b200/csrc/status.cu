// Library-state entry points of the C-ABI that every build of the library carries
// (the full shared library and the per-variant extension modules alike).
#include "common.cuh"

extern "C" const char* gemm_b200_last_error(void) { return gemm_b200::error_slot().msg; }

extern "C" int gemm_b200_version(void) { return GEMM_B200_VERSION; }

extern "C" int64_t gemm_b200_launch_count(void) {
  return gemm_b200::launch_counter().load(std::memory_order_relaxed);
}

extern "C" int gemm_b200_device_supported(int dev) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return major == 10 ? 1 : 0;
}
