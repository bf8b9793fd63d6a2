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
  // the GEMM that consumes this operand is a programmatic dependent launch: let it be scheduled and set
  // itself up now; it waits for this grid to complete before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
//   1. the bf16 tile is staged in shared memory as it lies in X ([k][column], 16-byte cp.async, 8
//      threads per 128-byte row segment; 2-byte loads for unaligned operands);
//   2. warp w owns columns 8 w .. 8 w + 7 and walks the four K blocks.  One ldmatrix.x4.trans per
//      block transposes 32 k x 8 columns: the row addresses are chosen so that lane 4 c + j
//      receives, as four ready-packed bf16 pairs, k = 8 j .. 8 j + 7 of column c.  The block
//      maximum is two shuffles away (the four lanes of a column); each lane converts its eight
//      values and stores eight e4m3 bytes, so a column's block leaves as one 32-byte sector;
//   3. lane 4 c keeps the four scale bytes of its column and stores them as one 32-bit word of
//      the packed layout.
// Rows of the shared tile are padded by 16 bytes so that the eight row addresses of an ldmatrix
// fall in distinct 16-byte bank groups.
constexpr int kQcK = 128, kQcCols = 64, kQcMaxTiles = 8;
template <int COLS>
__global__ void __launch_bounds__(COLS * 4)
quantize_cols_kernel(const __nv_bfloat16* __restrict__ X, int64_t rows, int64_t K, int64_t ldx,
                     uint8_t* __restrict__ Xq, uint8_t* __restrict__ SF, int64_t kb_pad, int vec_ok, int tiles_per_cta) {
  static_assert(COLS * 4 == 32 * (COLS / 8), "one warp per eight columns");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // as in quantize_rows_kernel
  // two tiles: the CTA walks tiles_per_cta consecutive K chunks of its columns and fetches chunk i + 1
  // (cp.async, straight into shared memory) while it quantises chunk i, so loads are in flight
  // all the time
  __shared__ __align__(16) uint16_t tile[2][kQcK][COLS + 8];
  const int64_t c0 = (int64_t)blockIdx.x * COLS;
  const int64_t KB = K / 32, kchunks = kb_pad / 4;
  const int64_t kc_first = (int64_t)blockIdx.y * tiles_per_cta;
  const int n_tiles = (int)((kchunks - kc_first < tiles_per_cta) ? (kchunks - kc_first) : tiles_per_cta);
  const int t = threadIdx.x;
  const uint16_t* Xu = reinterpret_cast<const uint16_t*>(X);
  const int warp = t >> 5, lane = t & 31;
  const int j = lane & 3, c = warp * 8 + (lane >> 2);       // this lane's k octet and column
  // row address this lane hands to ldmatrix: matrix m = lane / 8, row slot r = lane % 8  ->  k = 8 (r / 2) + 2 m + r % 2
  const int lm = lane >> 3, lr = lane & 7;
  const int k_addr = 8 * (lr >> 1) + 2 * lm + (lr & 1);
  const uint32_t row_addr0 = (uint32_t)__cvta_generic_to_shared(&tile[0][k_addr][warp * 8]);
  constexpr uint32_t kTileBytes = kQcK * (COLS + 8) * 2;
  const bool col_ok = c0 + c < rows;

  auto fetch = [&](int i) {       // chunk i of this CTA into buffer i % 2 (16-byte path)
    constexpr int kPerRow = COLS / 8;          // threads per k row, 8 columns each; 32 k rows per pass
    const int cg = (t % kPerRow) * 8, kr = t / kPerRow;
    const int64_t k0 = (kc_first + i) * kQcK;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int k = kr + 32 * p;
      const bool ok = k0 + k < K && c0 + cg < rows;       // rows % 8 == 0: a chunk of 8 columns is all in or all out
      const uint16_t* src = ok ? Xu + (k0 + k) * ldx + c0 + cg : Xu;
      const uint32_t dst = (uint32_t)__cvta_generic_to_shared(&tile[i & 1][k][cg]);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0));
    }
  };

  if (vec_ok && n_tiles > 0) fetch(0);
  asm volatile("cp.async.commit_group;\n" ::);
  for (int i = 0; i < n_tiles; ++i) {
    const int64_t kc = kc_first + i, k0 = kc * kQcK;
    if (vec_ok) {
      if (i + 1 < n_tiles) fetch(i + 1);
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      const int cc = t % COLS, kr = t / COLS;  // one thread per column, 4 k rows per pass
#pragma unroll 4
      for (int p = 0; p < 32; ++p) {
        const int k = kr + 4 * p;
        tile[i & 1][k][cc] = (k0 + k < K && c0 + cc < rows) ? Xu[(k0 + k) * ldx + c0 + cc] : (uint16_t)0;
      }
    }
    __syncthreads();
    const uint32_t row_addr = row_addr0 + (uint32_t)(i & 1) * kTileBytes;
    uint32_t scale_word = 0;
#pragma unroll
    for (int kb = 0; kb < 4; ++kb) {
      uint32_t w[4];
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                   : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3])
                   : "r"(row_addr + (uint32_t)(32 * kb * (COLS + 8) * 2)));
      uint32_t amax_bits = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t lo = (w[e] << 16) & 0x7fffffffu, hi = w[e] & 0x7fff0000u;
        amax_bits = max(amax_bits, max(lo, hi));
      }
      amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 1));
      amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 2));
      // columns / K blocks past the end hold zeros: they quantise to byte 0, the padding value
      const int eb = (int)(amax_bits >> 23);
      const uint32_t byte = (uint32_t)max(eb - 8, 0);
      const float inv = __uint_as_float((uint32_t)(254 - (int)byte) << 23);   // 2^(127 - byte)
      uint32_t q[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float a = bf16_bits_to_float(w[2 * e] & 0xffffu) * inv, b = bf16_bits_to_float(w[2 * e] >> 16) * inv;
        const float cc = bf16_bits_to_float(w[2 * e + 1] & 0xffffu) * inv, d = bf16_bits_to_float(w[2 * e + 1] >> 16) * inv;
        q[e] = pack4_e4m3(a, b, cc, d);
      }
      if (col_ok && kc * 4 + kb < KB)
        *reinterpret_cast<uint2*>(Xq + (c0 + c) * K + k0 + 32 * kb + 8 * j) = make_uint2(q[0], q[1]);
      scale_word |= byte << (8 * kb);
    }
    if (j == 0)   // the launch covers rows up to a multiple of 128: padding rows get zero scales
      *reinterpret_cast<uint32_t*>(SF + scale_offset(kchunks, c0 + c, kc * 4)) = scale_word;
    __syncthreads();   // every warp is done with this buffer before chunk i + 2 is fetched into it
  }
}

}  // namespace mx
}  // namespace gemm_b200
