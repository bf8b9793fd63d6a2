// TMA streaming probe, a measurement helper in a shared library of its own
// (libgemm_b200_probe.so): the time a grid needs just to pull a [rows, cols] byte matrix through
// TMA into shared memory, tiled the way the skinny GEMMs stream their B operand.  It is the floor
// a bandwidth-bound GEMM call can be held against (same launch, same cold caches).  Not part of
// the GEMM library and not on any of its call paths.
#include "../csrc/common.cuh"
#include "../csrc/tc_common.cuh"

namespace gemm_b200 {
namespace tc {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// byte matrix [rows, cols], box = box_cols x box_rows, 128-byte swizzle
static int make_byte_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int box_cols, int box_rows) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || !p)
    return fail(GEMM_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = reinterpret_cast<EncodeTiledFn>(p)(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides,
                                                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(GEMM_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return GEMM_B200_OK;
}

}  // namespace tc
}  // namespace gemm_b200

namespace gemm_b200 {
namespace tc {

// Every CTA streams `rows_per_cta` rows: in passes of ROWS rows, SEG adjacent 128-byte column
// segments per stage.  One producer warp, one consumer warp that only frees the stage.
template <int ROWS, int SEG, int STAGES>
__global__ void __launch_bounds__(64, 1)
tma_stream_probe_kernel(const __grid_constant__ CUtensorMap tm, int cols, int rows_per_cta) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int STAGE_BYTES = ROWS * 128 * SEG;
  const uint32_t bar0 = base + STAGES * STAGE_BYTES;
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (STAGES + s); };
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    fence_mbar_init();
  }
  __syncthreads();
  const int row0 = blockIdx.x * rows_per_cta, passes = rows_per_cta / ROWS, ksteps = cols / (128 * SEG);
  const bool issuer = elect_one();
  uint32_t it = 0;
  for (int p = 0; p < passes; ++p) {
    for (int ks = 0; ks < ksteps; ++ks, ++it) {
      const int s = it % STAGES;
      const uint32_t ph = (it / STAGES) & 1u;
      if (threadIdx.x < 32) {
        if (!mbar_wait_warp(empty(s), ph ^ 1u, kRoleProducer, s)) return;
        if (issuer) {
          mbar_arrive_expect_tx(full(s), STAGE_BYTES);
#pragma unroll
          for (int g = 0; g < SEG; ++g)
            tma_load_2d(base + s * STAGE_BYTES + g * ROWS * 128, &tm, (ks * SEG + g) * 128, row0 + p * ROWS, full(s));
        }
      } else {
        if (!mbar_wait_warp(full(s), ph, kRoleMma, s)) return;
        if (issuer) mbar_arrive(empty(s));
      }
      __syncwarp();
    }
  }
}

template <int ROWS, int SEG, int STAGES>
static int launch_stream_probe(const void* X, int64_t rows, int64_t cols, int64_t rows_per_cta, cudaStream_t st) {
  if (rows % rows_per_cta != 0 || rows_per_cta % ROWS != 0 || cols % (128 * SEG) != 0)
    return fail(GEMM_B200_ERR_INVALID_ARG, "tma_stream_probe: rows %% rows_per_cta, rows_per_cta %% %d and cols %% %d must be 0",
                ROWS, 128 * SEG);
  CUtensorMap tm;
  if (int rc = make_byte_map(&tm, X, rows, cols, 128, ROWS)) return rc;
  auto kern = tma_stream_probe_kernel<ROWS, SEG, STAGES>;
  constexpr int smem = 1024 + STAGES * ROWS * 128 * SEG + 2 * STAGES * 8 + 64;
  GEMM_B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  kern<<<(unsigned)(rows / rows_per_cta), 64, smem, st>>>(tm, (int)cols, (int)rows_per_cta);
  GEMM_B200_CUDA_TRY(cudaGetLastError());
  return GEMM_B200_OK;
}

}  // namespace tc
}  // namespace gemm_b200

extern "C" int gemm_b200_probe_tma_stream(const void* X, int64_t rows, int64_t cols, int64_t rows_per_cta, int pattern,
                                             void* stream) {
  using namespace gemm_b200;
  if (!X || rows <= 0 || cols <= 0 || rows_per_cta <= 0 || rows > 0x7fffffff || cols > 0x7fffffff)
    return fail(GEMM_B200_ERR_INVALID_ARG, "tma_stream_probe: bad arguments");
  if (reinterpret_cast<uintptr_t>(X) % 16 != 0 || cols % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "tma_stream_probe: X and cols must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (pattern) {
    case 0: return tc::launch_stream_probe<256, 1, 4>(X, rows, cols, rows_per_cta, st);
    case 1: return tc::launch_stream_probe<256, 1, 6>(X, rows, cols, rows_per_cta, st);
    case 2: return tc::launch_stream_probe<64, 4, 6>(X, rows, cols, rows_per_cta, st);
    case 3: return tc::launch_stream_probe<32, 8, 6>(X, rows, cols, rows_per_cta, st);
    default: return fail(GEMM_B200_ERR_INVALID_ARG, "tma_stream_probe: pattern %d (0..3)", pattern);
  }
}

// Reads and clears this library's own copy of the bounded-wait status word.
extern "C" int gemm_b200_probe_check_status(void* stream) {
  using namespace gemm_b200;
  GEMM_B200_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int32_t h[4] = {0, 0, 0, 0};
  GEMM_B200_CUDA_TRY(cudaMemcpyFromSymbol(h, tc::g_status, sizeof(h)));
  if (h[0] != 0) {
    const int32_t z[4] = {0, 0, 0, 0};
    GEMM_B200_CUDA_TRY(cudaMemcpyToSymbol(tc::g_status, z, sizeof(z)));
    return fail(GEMM_B200_ERR_TIMEOUT, "a device-side wait gave up: block %d role %d stage %d", h[1], h[2], h[3]);
  }
  return GEMM_B200_OK;
}
extern "C" const char* gemm_b200_probe_last_error(void) { return gemm_b200::error_slot().msg; }
