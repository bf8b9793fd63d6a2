// MXFP8 quantiser: bf16 -> e4m3 data + one UE8M0 scale per 32 consecutive K elements.
//
// No counterpart in the reference (its kernels are FP32 only: naive/naive_1.cu:5-15); this is
// the operand format of the block-scaled tensor-core GEMM in this library.
//
// Recipe per block of 32:  amax = max |x|;  scale byte = max(biased_exponent(amax) - 8, 0),
// i.e. scale = 2^(floor(log2 amax) - 8) clamped at 2^-127;  q = e4m3(x * 2^(127 - byte)) with
// round-to-nearest-even and saturation at +-448.  A zero block gets byte 0 and zero data.
//
// Scales are written in the layout the GEMM copies straight into tensor memory: 512-byte chunks
// holding 128 rows x 4 K-blocks as 32 x 16 bytes,
//     offset(r, kb) = ((r / 128) * ceil(KB / 4) + kb / 4) * 512 + (r % 32) * 16 + ((r / 32) % 4) * 4 + kb % 4,
// chunks ordered [row block][K chunk]; padding bytes (rows >= rows, kb >= KB) are written as 0.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "common.cuh"

namespace gemm_b200 {
namespace mx {

__host__ __device__ inline size_t scale_offset(int64_t kchunks, int64_t r, int64_t kb) {
  return (size_t)((r / 128) * kchunks + kb / 4) * 512 + (size_t)((r % 32) * 16 + ((r / 32) % 4) * 4 + (kb % 4));
}

__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
  // cvt.rn.satfinite.e4m3x2.f32 d, hi, lo : low byte = lo
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b16) { return __uint_as_float(b16 << 16); }

// quantise 32 values held as 16 packed bf16x2 words; returns the scale byte, writes 8 words of e4m3
__device__ __forceinline__ uint32_t quantise_block(const uint32_t (&w)[16], uint32_t (&q)[8]) {
  uint32_t amax_bits = 0;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    // |x| as FP32 bits compares like an unsigned integer
    const uint32_t lo = (w[i] << 16) & 0x7fffffffu, hi = w[i] & 0x7fff0000u;
    amax_bits = max(amax_bits, max(lo, hi));
  }
  const int eb = (int)(amax_bits >> 23);                 // biased exponent of amax (0 for 0 / denormals)
  const uint32_t byte = (uint32_t)max(eb - 8, 0);
  const float inv = __uint_as_float((uint32_t)(254 - (int)byte) << 23);   // 2^(127 - byte)
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = bf16_bits_to_float(w[2 * i] & 0xffffu) * inv, b = bf16_bits_to_float(w[2 * i] >> 16) * inv;
    const float c = bf16_bits_to_float(w[2 * i + 1] & 0xffffu) * inv, d = bf16_bits_to_float(w[2 * i + 1] >> 16) * inv;
    q[i] = pack4_e4m3(a, b, c, d);
  }
  return byte;
}

// X [rows, K] row-major (ldx).  One thread per (row, K-block) over the PADDED scale grid
// (rows up to a multiple of 128, K-blocks up to a multiple of 4) so padding scales become 0.
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __nv_bfloat16* __restrict__ X, int64_t rows, int64_t K, int64_t ldx,
                     uint8_t* __restrict__ Xq, uint8_t* __restrict__ SF, int64_t kb_pad, int64_t rows_pad) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t kb = idx % kb_pad, r = idx / kb_pad;
  if (r >= rows_pad) return;
  const int64_t KB = K / 32, kchunks = kb_pad / 4;
  uint32_t byte = 0;
  if (r < rows && kb < KB && GEMM_B200_IN_BOUNDS(X + r * ldx + kb * 32, X, ((rows - 1) * ldx + K) * 2, 64, 40) &&
      GEMM_B200_IN_BOUNDS(Xq + r * K + kb * 32, Xq, rows * K, 32, 41)) {
    const uint4* src = reinterpret_cast<const uint4*>(X + r * ldx + kb * 32);
    uint32_t w[16], q[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(src + i);
      w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
    byte = quantise_block(w, q);
    uint4* dst = reinterpret_cast<uint4*>(Xq + r * K + kb * 32);
    dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
    dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
  }
  if (GEMM_B200_IN_BOUNDS(SF + scale_offset(kchunks, r, kb), SF, (rows_pad / 128) * kchunks * 512, 1, 42))
    SF[scale_offset(kchunks, r, kb)] = (uint8_t)byte;
}

// X [K, rows] row-major (ldx): quantise every column along K, write Xq [rows, K] K-contiguous.
// A CTA of 256 threads owns 128 k (one 4-block scale chunk) x 64 columns:
//   1. the bf16 tile is staged with 16-byte loads, 8 threads per 128-byte row segment;
//   2. thread (column c = t % 64, block kb = t / 64) reads its 32 values down the tile, quantises
//      them and parks the 32 e4m3 bytes in a [64][128] byte tile, the scale byte in a [64][4] one;
//   3. the byte tile leaves as whole 128-byte lines of Xq (8 threads x 16 bytes per row) and the
//      four scale bytes of a row as one 32-bit word of the packed layout.
// Every global access is a full line; rows of the shared tiles are padded by 16 bytes so that the
// 16-byte accesses of a quarter warp and the 2-byte column walks fall in distinct banks.
constexpr int kQcK = 128, kQcCols = 64;
template <int COLS>
__global__ void __launch_bounds__(COLS * 4)
quantize_cols_kernel(const __nv_bfloat16* __restrict__ X, int64_t rows, int64_t K, int64_t ldx,
                     uint8_t* __restrict__ Xq, uint8_t* __restrict__ SF, int64_t kb_pad, int vec_ok) {
  constexpr int kThreads = COLS * 4;
  // the byte tile reuses the bf16 tile's storage once every thread holds its 32 values in registers
  __shared__ __align__(16) uint16_t tile[kQcK][COLS + 8];
  uint8_t (*qtile)[kQcK + 16] = reinterpret_cast<uint8_t (*)[kQcK + 16]>(&tile[0][0]);
  __shared__ __align__(4) uint8_t sft[COLS][4];
  const int64_t c0 = (int64_t)blockIdx.x * COLS, kc = blockIdx.y, k0 = kc * kQcK;
  const int64_t KB = K / 32, kchunks = kb_pad / 4;
  const int t = threadIdx.x;
  const uint16_t* Xu = reinterpret_cast<const uint16_t*>(X);
  if (vec_ok) {
    constexpr int kPerRow = COLS / 8;          // threads per k row, 8 columns each; 32 k rows per pass
    const int cg = (t % kPerRow) * 8, kr = t / kPerRow;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int k = kr + 32 * p;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (k0 + k < K && c0 + cg < rows) v = __ldg(reinterpret_cast<const uint4*>(Xu + (k0 + k) * ldx + c0 + cg));   // rows % 8 == 0
      *reinterpret_cast<uint4*>(&tile[k][cg]) = v;
    }
  } else {
    const int c = t % COLS, kr = t / COLS;  // one thread per column, 4 k rows per pass
#pragma unroll 4
    for (int p = 0; p < 32; ++p) {
      const int k = kr + 4 * p;
      tile[k][c] = (k0 + k < K && c0 + c < rows) ? Xu[(k0 + k) * ldx + c0 + c] : (uint16_t)0;
    }
  }
  __syncthreads();
  {
    const int c = t % COLS, kb = t / COLS;
    uint32_t w[16], q[8];
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] = (uint32_t)tile[32 * kb + 2 * i][c] | ((uint32_t)tile[32 * kb + 2 * i + 1][c] << 16);
    __syncthreads();
    // columns / K-blocks past the end hold zeros: they quantise to byte 0, the padding value
    const uint32_t byte = quantise_block(w, q);
    uint4* dst = reinterpret_cast<uint4*>(&qtile[c][32 * kb]);
    dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
    dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
    sft[c][kb] = (uint8_t)byte;
  }
  __syncthreads();
  {
    const int j = t & 7, cr = t >> 3;             // 16-byte piece j of the row; half of the rows per pass
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      const int c = cr + (kThreads / 8) * p;
      if (c0 + c < rows && kc * 4 + j / 2 < KB)
        *reinterpret_cast<uint4*>(Xq + (c0 + c) * K + k0 + 16 * j) = *reinterpret_cast<const uint4*>(&qtile[c][16 * j]);
    }
  }
  if (t < COLS)   // the launch covers rows up to a multiple of 128: padding rows get zero scales
    *reinterpret_cast<uint32_t*>(SF + scale_offset(kchunks, c0 + t, kc * 4)) = *reinterpret_cast<const uint32_t*>(&sft[t][0]);
}

}  // namespace mx
}  // namespace gemm_b200
