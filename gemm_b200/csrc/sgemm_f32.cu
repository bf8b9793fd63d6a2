// FP32 CUDA-core GEMM for sm_100: C[M,N] = A[M,K] @ B[K,N], row-major, beta = 0.
//
// One kernel family replaces the three reference kernels
//   naive_gemm            naive/naive_1.cu:5-15
//   sgemm                 shared/shared_2.cu:4-57
//   gemm<64,64,16,4>      blocktile_1d/blocktile_1d.cu:5-68
// and keeps their arithmetic: every element of C has ONE FP32 accumulator that
// starts at zero and takes fused multiply-adds in strictly ascending k, with
// denormals flushed (the reference is compiled with --use_fast_math).  The
// result is therefore bit-identical to all three reference kernels.
//
// Design (per CTA):
//   * BM x BN tile of C, register-blocked TM x TN per thread;
//   * A and B tiles staged in shared memory by 16-byte cp.async, STAGES deep,
//     one __syncthreads per K tile;
//   * A is kept K-contiguous in shared memory with rows padded to BK+4 floats:
//     a thread reads two consecutive k of one row with one LDS.64 (AK = 2; AK = 4
//     reads four with one LDS.128) and the four row addresses of a warp fall into
//     different bank groups (the row stride is an odd multiple of 16 bytes); B
//     fragments are LDS.128 along N, 128 contiguous bytes per warp;
//   * optionally the multiply-adds are issued as packed fma.rn.f32x2 (two
//     columns of C per instruction), which halves the issue slots the FMA
//     stream needs.
// Tiles on the M/N/K edges are zero-filled by the cp.async source-size operand.
// A 4-byte cp.async variant of the same kernel serves operands whose pointers
// or leading dimensions are not 16-byte aligned.
#include <string.h>

#include "common.cuh"

namespace gemm_b200 {
namespace f32 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

template <int BM_, int BN_, int BK_, int WMW_, int WNW_, int STAGES_, int MINB_, bool X2_, int AK_ = 2>
struct Cfg {
  static constexpr int AK = AK_;              // k-width of one A fragment load (2: LDS.64, 4: LDS.128)
  static constexpr int BM = BM_, BN = BN_, BK = BK_, WMW = WMW_, WNW = WNW_;
  static constexpr int STAGES = STAGES_, MINB = MINB_;
  static constexpr bool X2 = X2_;
  static constexpr int THREADS = WMW * WNW * 32;
  static constexpr int TM = BM / (WMW * 4);   // rows per thread (interleaved by 4)
  static constexpr int TN = BN / (WNW * 8);   // columns per thread (float4 groups, 32 apart)
  static constexpr int LDA_S = BK + 4;        // padded row of the A tile, in floats
  static constexpr int A_STAGE = BM * LDA_S;
  static constexpr int B_STAGE = BK * BN;
  static constexpr int SMEM_BYTES = STAGES * (A_STAGE + B_STAGE) * 4;
  static_assert(TM >= 1 && TN >= 4 && TN % 4 == 0, "thread tile");
  static_assert(BK % 4 == 0, "BK");
  static_assert(((LDA_S / 4) & 1) == 1, "A row stride must be an odd number of 16-byte units");
};

// VEC = 4: 16-byte cp.async and float4 stores (needs aligned pointers, lda/ldb/ldc % 4 == 0,
//          which also makes every 4-wide chunk entirely inside or outside the matrix).
// VEC = 1: 4-byte cp.async, scalar stores; any alignment.
template <class C, int VEC>
__global__ void __launch_bounds__(C::THREADS, C::MINB)
sgemm_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ Cm,
             int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int tiles_m, int tiles_n,
             int64_t batch_a, int64_t batch_b, int64_t batch_c) {
  // Programmatic dependent launch: the grid may have been scheduled while the kernel before it in the
  // stream still runs (when that kernel is one of this library's); wait for it before touching
  // memory, then let the kernel behind this one be scheduled early in turn.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // blockIdx.y = problem of a strided batch (strides in elements; 0 shares the operand)
  A += (int64_t)blockIdx.y * batch_a;
  B += (int64_t)blockIdx.y * batch_b;
  Cm += (int64_t)blockIdx.y * batch_c;
  constexpr int BM = C::BM, BN = C::BN, BK = C::BK, TM = C::TM, TN = C::TN, TNC = C::TN / 4;
  constexpr int STAGES = C::STAGES, THREADS = C::THREADS, LDA_S = C::LDA_S, AK = C::AK;
  extern __shared__ __align__(16) float smem[];
  float* sA = smem;
  float* sB = smem + STAGES * C::A_STAGE;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp / C::WNW, wn = warp % C::WNW;
  const int ty = lane >> 3, tx = lane & 7;

  // Grouped raster: consecutive CTAs walk down a band of 8 row tiles before moving to the
  // next column tile, so the CTAs resident at one time share A and B tiles in L2.
  constexpr int GROUP = 8;
  const int pid = blockIdx.x;
  const int width = GROUP * tiles_n;
  const int first_m = (pid / width) * GROUP;
  const int gsz = min(tiles_m - first_m, GROUP);
  const int bm = first_m + (pid % width) % gsz;
  const int bn = (pid % width) / gsz;
  const int row0 = bm * BM, col0 = bn * BN;

  const int num_kt = (K + BK - 1) / BK;

  // Per-thread loader state for the 16-byte path: chunk `it` of a thread is RPI rows below chunk
  // `it - 1`, so one base pointer per operand (advanced by BK columns / BK rows per K tile) suffices.
  constexpr int KC = BK / 4, NC = BN / 4;
  constexpr int A_IT = (BM * KC + THREADS - 1) / THREADS, A_RPI = THREADS / KC;   // A: rows per pass
  constexpr int B_IT = BK * NC / THREADS, B_RPI = THREADS / NC;                   // B: k rows per pass
  constexpr bool A_EVEN = (BM * KC) % THREADS == 0;   // else the last pass is guarded (tile heights such as 28)
  static_assert(THREADS % KC == 0, "a pass over the A tile must cover whole rows");
  static_assert(BK * NC % THREADS == 0 && THREADS % NC == 0, "B tile must split evenly over the threads");
  const int a_r = tid / KC, a_kc = (tid % KC) * 4;
  const int b_r = tid / NC, b_nc = (tid % NC) * 4;
  const float* a_src = A + (int64_t)(row0 + a_r) * lda + a_kc;
  const float* b_src = B + (int64_t)b_r * ldb + (col0 + b_nc);
  const uint32_t a_sdst = smem_u32(sA) + (a_r * LDA_S + a_kc) * 4;
  const uint32_t b_sdst = smem_u32(sB) + (b_r * BN + b_nc) * 4;
  const bool b_col_ok = (col0 + b_nc) < N;

  auto load_tile = [&](int kt, int slot) {
    const int k0 = kt * BK;
    if constexpr (VEC == 4) {
      const bool a_k_ok = (k0 + a_kc) < K;
#pragma unroll
      for (int it = 0; it < A_IT; ++it) {
        if (!A_EVEN && a_r + it * A_RPI >= BM) break;
        const float* src = a_src + (int64_t)(it * A_RPI) * lda + k0;
        const bool ok = a_k_ok && (row0 + a_r + it * A_RPI < M) &&
                        GEMM_B200_IN_BOUNDS(src, A, ((long long)(M - 1) * lda + K) * 4, 16, 3);
        cp_async16(a_sdst + (slot * C::A_STAGE + it * A_RPI * LDA_S) * 4, ok ? src : A, ok ? 16 : 0);
      }
#pragma unroll
      for (int it = 0; it < B_IT; ++it) {
        const float* src = b_src + (int64_t)(k0 + it * B_RPI) * ldb;
        const bool ok = b_col_ok && (k0 + b_r + it * B_RPI < K) &&
                        GEMM_B200_IN_BOUNDS(src, B, ((long long)(K - 1) * ldb + N) * 4, 16, 4);
        cp_async16(b_sdst + (slot * C::B_STAGE + it * B_RPI * BN) * 4, ok ? src : B, ok ? 16 : 0);
      }
    } else {
      float* a_dst = sA + slot * C::A_STAGE;
      float* b_dst = sB + slot * C::B_STAGE;
#pragma unroll 4
      for (int it = 0; it < (BM * BK + THREADS - 1) / THREADS; ++it) {
        const int c = tid + it * THREADS;
        if ((BM * BK) % THREADS != 0 && c >= BM * BK) break;
        const int r = c / BK, kc = c % BK;
        const int gr = row0 + r, gk = k0 + kc;
        const bool ok = (gr < M) && (gk < K);
        const float* src = ok ? (A + (int64_t)gr * lda + gk) : A;
        cp_async4(smem_u32(a_dst + r * LDA_S + kc), src, ok ? 4 : 0);
      }
#pragma unroll 4
      for (int it = 0; it < BK * BN / THREADS; ++it) {
        const int c = tid + it * THREADS;
        const int r = c / BN, nc = c % BN;
        const int gk = k0 + r, gc = col0 + nc;
        const bool ok = (gk < K) && (gc < N);
        const float* src = ok ? (B + (int64_t)gk * ldb + gc) : B;
        cp_async4(smem_u32(b_dst + r * BN + nc), src, ok ? 4 : 0);
      }
    }
  };

  // accumulators: acc2[i][j] holds columns (2j, 2j+1) of the thread tile for row (ty + 4 i)
  float2 acc2[TM][TN / 2];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN / 2; ++j) acc2[i][j] = make_float2(0.0f, 0.0f);

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_kt) load_tile(s, s);
    cp_async_commit();
  }

  const int a_off = (wm * (BM / C::WMW) + ty) * LDA_S;
  const int b_off = wn * (BN / C::WNW) + tx * 4;

#pragma unroll 1
  for (int kt = 0; kt < num_kt; ++kt) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();
    {
      const int nk = kt + STAGES - 1;
      if (nk < num_kt) load_tile(nk, nk % STAGES);
      cp_async_commit();
    }
    const int slot = kt % STAGES;
    const float* a_s = sA + slot * C::A_STAGE + a_off;
    const float* b_s = sB + slot * C::B_STAGE + b_off;
#pragma unroll
    for (int kq = 0; kq < BK / AK; ++kq) {
      float af[TM][AK];
#pragma unroll
      for (int i = 0; i < TM; ++i) {
        if constexpr (AK == 4) {
          const float4 v = *reinterpret_cast<const float4*>(a_s + (4 * i) * LDA_S + kq * 4);
          af[i][0] = v.x; af[i][1] = v.y; af[i][2] = v.z; af[i][3] = v.w;
        } else {
          const float2 v = *reinterpret_cast<const float2*>(a_s + (4 * i) * LDA_S + kq * 2);
          af[i][0] = v.x; af[i][1] = v.y;
        }
      }
#pragma unroll
      for (int kk = 0; kk < AK; ++kk) {
        float4 bf[TNC];
#pragma unroll
        for (int c = 0; c < TNC; ++c)
          bf[c] = *reinterpret_cast<const float4*>(b_s + (kq * AK + kk) * BN + c * 32);
#pragma unroll
        for (int i = 0; i < TM; ++i) {
          const float a = af[i][kk];
          if constexpr (C::X2) {
            const float2 a2 = make_float2(a, a);
#pragma unroll
            for (int c = 0; c < TNC; ++c) {
              acc2[i][2 * c + 0] = __ffma2_rn(a2, make_float2(bf[c].x, bf[c].y), acc2[i][2 * c + 0]);
              acc2[i][2 * c + 1] = __ffma2_rn(a2, make_float2(bf[c].z, bf[c].w), acc2[i][2 * c + 1]);
            }
          } else {
#pragma unroll
            for (int c = 0; c < TNC; ++c) {
              acc2[i][2 * c + 0].x = fmaf(a, bf[c].x, acc2[i][2 * c + 0].x);
              acc2[i][2 * c + 0].y = fmaf(a, bf[c].y, acc2[i][2 * c + 0].y);
              acc2[i][2 * c + 1].x = fmaf(a, bf[c].z, acc2[i][2 * c + 1].x);
              acc2[i][2 * c + 1].y = fmaf(a, bf[c].w, acc2[i][2 * c + 1].y);
            }
          }
        }
      }
    }
  }
  cp_async_wait<0>();

  // store
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gr = row0 + wm * (BM / C::WMW) + ty + 4 * i;
    if (gr >= M) continue;
    float* crow = Cm + (int64_t)gr * ldc;
    const long long c_bytes = ((long long)(M - 1) * ldc + N) * 4;   // extent of C (bounds-checking build)
    (void)c_bytes;
#pragma unroll
    for (int c = 0; c < TNC; ++c) {
      const int gc = col0 + wn * (BN / C::WNW) + c * 32 + tx * 4;
      if constexpr (VEC == 4) {
        if (gc < N && GEMM_B200_IN_BOUNDS(crow + gc, Cm, c_bytes, 16, 1))
          *reinterpret_cast<float4*>(crow + gc) =
              make_float4(acc2[i][2 * c].x, acc2[i][2 * c].y, acc2[i][2 * c + 1].x, acc2[i][2 * c + 1].y);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (gc + e < N && GEMM_B200_IN_BOUNDS(crow + gc + e, Cm, c_bytes, 4, 2)) crow[gc + e] = (e & 1) ? acc2[i][2 * c + e / 2].y : acc2[i][2 * c + e / 2].x;
      }
    }
  }
}

struct ConfigEntry {
  const char* name;
  int bm, bn;
  int (*launch)(const float*, const float*, float*, int, int, int, int64_t, int64_t, int64_t, bool,
                cudaStream_t, int, int64_t, int64_t, int64_t);
};

// Internal linkage on purpose: this source is compiled into several modules of one process (the
// shared library and the three extension modules), each with its own copy of the kernels; the
// "attribute already set" cache below must not be merged across them by the dynamic linker.
template <class C>
static int launch_cfg(const float* A, const float* B, float* Cm, int M, int N, int K, int64_t lda,
                      int64_t ldb, int64_t ldc, bool vec, cudaStream_t stream, int batch, int64_t batch_a,
                      int64_t batch_b, int64_t batch_c) {
  const int tiles_m = (M + C::BM - 1) / C::BM, tiles_n = (N + C::BN - 1) / C::BN;
  const int64_t tiles = (int64_t)tiles_m * tiles_n;
  if (tiles == 0) return GEMM_B200_OK;
  if (tiles > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "sgemm_f32: %lld tiles", (long long)tiles);
  auto kv = sgemm_kernel<C, 4>;
  auto ks = sgemm_kernel<C, 1>;
  auto kern = vec ? kv : ks;
  if (C::SMEM_BYTES > 48 * 1024) {
    // opt in to more than 48 KB of dynamic shared memory, once per (device, kernel)
    static thread_local int done_dev[2] = {-1, -1};
    static thread_local const void* done_fn[2] = {nullptr, nullptr};
    int dev = 0;
    GEMM_B200_CUDA_TRY(cudaGetDevice(&dev));
    const int slot = vec ? 0 : 1;
    if (done_dev[slot] != dev || done_fn[slot] != reinterpret_cast<const void*>(kern)) {
      GEMM_B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
      done_dev[slot] = dev;
      done_fn[slot] = reinterpret_cast<const void*>(kern);
    }
  }
  // at most 65535 problems per launch (grid.y)
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = batch - b0 < 65535 ? batch - b0 : 65535;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)tiles, (unsigned)nb);
    cfg.blockDim = dim3((unsigned)C::THREADS);
    cfg.dynamicSmemBytes = (size_t)C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    static const bool pdl = env_int("GEMM_B200_PDL", 1) != 0;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    GEMM_B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, A + b0 * batch_a, B + b0 * batch_b, Cm + b0 * batch_c, M, N, K, lda, ldb, ldc, tiles_m,
                                          tiles_n, batch_a, batch_b, batch_c));
    launch_counter().fetch_add(1, std::memory_order_relaxed);
  }
  return GEMM_B200_OK;
}

//                        BM   BN  BK WMW WNW ST MINB X2  AK
using C64x128k32p3     = Cfg<64, 128, 32, 2, 2, 3, 2, true>;
using C64x64k32p       = Cfg<64, 64, 32, 2, 2, 4, 4, true>;
using C32x64k32p       = Cfg<32, 64, 32, 2, 2, 4, 6, true>;
// Tile heights of 28 and 56 rows: 148 SMs = 4 x 37, and 37 tiles of 28 rows cover 1024 rows (74 of
// 28 or 37 of 56 cover 2048, ...), so power-of-two problems split into a whole number of tiles per
// SM instead of leaving a third of the SMs one tile short.  7 rows x 8 (or 4) columns per thread.
using C28x128k32p      = Cfg<28, 128, 32, 1, 4, 4, 2, true>;
using C56x128k32p      = Cfg<56, 128, 32, 2, 2, 3, 3, true>;
#ifdef GEMM_B200_TUNING
// tile shapes the heuristic never picks; built only for tuning sweeps
using C128x128k16      = Cfg<128, 128, 16, 4, 2, 3, 2, false>;
using C128x128k16p     = Cfg<128, 128, 16, 4, 2, 3, 2, true>;
using C128x128k32p     = Cfg<128, 128, 32, 4, 2, 3, 2, true>;
using C128x128k32pa4   = Cfg<128, 128, 32, 4, 2, 3, 2, true, 4>;
using C128x256k16p     = Cfg<128, 256, 16, 4, 2, 3, 1, true>;
using C128x256k32p     = Cfg<128, 256, 32, 4, 2, 3, 1, true>;
using C256x128k32p     = Cfg<256, 128, 32, 8, 1, 3, 1, true>;
using C128x64k32p      = Cfg<128, 64, 32, 4, 2, 3, 2, true>;
using C64x64k16p       = Cfg<64, 64, 16, 2, 2, 4, 4, true>;
using C64x64k16        = Cfg<64, 64, 16, 2, 2, 4, 4, false>;
using C32x64k16p       = Cfg<32, 64, 16, 2, 2, 4, 6, true>;
using C128x128k32      = Cfg<128, 128, 32, 4, 2, 3, 2, false>;
using C28x256k32p      = Cfg<28, 256, 32, 1, 4, 3, 1, true>;
using C28x256k32pw8    = Cfg<28, 256, 32, 1, 8, 3, 1, true>;
using C56x256k16p      = Cfg<56, 256, 16, 2, 4, 4, 2, true>;
using C56x256k32p      = Cfg<56, 256, 32, 2, 4, 3, 1, true>;
using C28x64k32p       = Cfg<28, 64, 32, 1, 2, 4, 4, true>;
using C28x128k32ps3    = Cfg<28, 128, 32, 1, 4, 3, 2, true>;
using C28x128k16ps6    = Cfg<28, 128, 16, 1, 4, 6, 2, true>;
using C28x128k32pa4    = Cfg<28, 128, 32, 1, 4, 4, 2, true, 4>;
using C28x128k32       = Cfg<28, 128, 32, 1, 4, 4, 2, false>;
// 16 x 8 accumulators per thread (64 x 64 per warp, 240 registers): three quarters of the shared-memory
// reads per multiply-add of the 8 x 8 tile, yet within 1 % of it (57.9 against 57.5 TFLOP/s at 8192^3):
// the loop is bound by the issue of the multiply-add stream, not by shared memory
using C128x128k32w4    = Cfg<128, 128, 32, 2, 2, 3, 2, true>;
#endif

static const ConfigEntry kConfigs[] = {
    {"64x128x32_s3_f32x2", 64, 128, launch_cfg<C64x128k32p3>},
    {"64x64x32_s4_f32x2", 64, 64, launch_cfg<C64x64k32p>},
    {"32x64x32_s4_f32x2", 32, 64, launch_cfg<C32x64k32p>},
    {"28x128x32_s4_f32x2", 28, 128, launch_cfg<C28x128k32p>},
    {"56x128x32_s3_f32x2", 56, 128, launch_cfg<C56x128k32p>},
#ifdef GEMM_B200_TUNING
    {"128x128x16_s3", 128, 128, launch_cfg<C128x128k16>},
    {"128x128x16_s3_f32x2", 128, 128, launch_cfg<C128x128k16p>},
    {"128x128x32_s3_f32x2", 128, 128, launch_cfg<C128x128k32p>},
    {"128x128x32_s3_f32x2_a4", 128, 128, launch_cfg<C128x128k32pa4>},
    {"128x256x16_s3_f32x2", 128, 256, launch_cfg<C128x256k16p>},
    {"128x256x32_s3_f32x2", 128, 256, launch_cfg<C128x256k32p>},
    {"256x128x32_s3_f32x2", 256, 128, launch_cfg<C256x128k32p>},
    {"128x64x32_s3_f32x2", 128, 64, launch_cfg<C128x64k32p>},
    {"64x64x16_s4_f32x2", 64, 64, launch_cfg<C64x64k16p>},
    {"64x64x16_s4", 64, 64, launch_cfg<C64x64k16>},
    {"32x64x16_s4_f32x2", 32, 64, launch_cfg<C32x64k16p>},
    {"128x128x32_s3", 128, 128, launch_cfg<C128x128k32>},
    {"28x256x32_s3_f32x2", 28, 256, launch_cfg<C28x256k32p>},
    {"28x256x32_s3_f32x2_w8", 28, 256, launch_cfg<C28x256k32pw8>},
    {"56x256x16_s4_f32x2", 56, 256, launch_cfg<C56x256k16p>},
    {"56x256x32_s3_f32x2", 56, 256, launch_cfg<C56x256k32p>},
    {"28x64x32_s4_f32x2", 28, 64, launch_cfg<C28x64k32p>},
    {"28x128x32_s3_f32x2", 28, 128, launch_cfg<C28x128k32ps3>},
    {"28x128x16_s6_f32x2", 28, 128, launch_cfg<C28x128k16ps6>},
    {"28x128x32_s4_f32x2_a4", 28, 128, launch_cfg<C28x128k32pa4>},
    {"28x128x32_s4", 28, 128, launch_cfg<C28x128k32>},
    {"128x128x32_s3_f32x2_w4", 128, 128, launch_cfg<C128x128k32w4>},
#endif
};
constexpr int kNumConfigs = sizeof(kConfigs) / sizeof(kConfigs[0]);

inline int config_index(const char* name) {
  for (int i = 0; i < kNumConfigs; ++i)
    if (strcmp(kConfigs[i].name, name) == 0) return i;
  return 0;
}

// Tile choice: the CTAs of a launch spread evenly over the SMs, so the launch takes
//   ceil(tiles / SMs) x (time of one tile),   time of one tile ~ BM x BN / (rate of that tile shape),
// with the rates measured at 8192^3 on a B200 (TFLOP/s): 64x128 57.3, 56x128 56.5, 64x64 55.5,
// 28x128 51.5, 32x64 44.5.  The estimate ranks the five shapes as the measurements do at 512^3 ...
// 8192^3 (n = 1024: 28x128 53 us, 64x128 / 64x64 59, 32x64 68, 56x128 90; n = 2048: 56x128 329 us,
// 64x64 339, 28x128 356, 64x128 363, 32x64 410).  28- and 56-row tiles exist because 148 SMs =
// 4 x 37 and 37 x 28 covers 1024 rows: power-of-two problems then split into whole tiles per SM.
inline int pick_config(int64_t M, int64_t N, int num_sms, int64_t batch = 1) {
  struct Cand { const char* name; int bm, bn; double rate; };
  static const Cand cands[] = {{"64x128x32_s3_f32x2", 64, 128, 57.3}, {"56x128x32_s3_f32x2", 56, 128, 56.5},
                               {"64x64x32_s4_f32x2", 64, 64, 55.5},  {"28x128x32_s4_f32x2", 28, 128, 51.5},
                               {"32x64x32_s4_f32x2", 32, 64, 44.5}};
  static const int index[5] = {config_index(cands[0].name), config_index(cands[1].name), config_index(cands[2].name),
                               config_index(cands[3].name), config_index(cands[4].name)};
  int best = 0;
  double best_t = 0.0;
  for (int i = 0; i < 5; ++i) {
    const int64_t tiles = batch * ceil_div64(M, cands[i].bm) * ceil_div64(N, cands[i].bn);
    const double t = (double)ceil_div64(tiles, num_sms) * cands[i].bm * cands[i].bn / cands[i].rate;
    if (i == 0 || t < best_t * 0.999) { best = i; best_t = t; }
  }
  return index[best];
}

}  // namespace f32
}  // namespace gemm_b200

namespace gemm_b200 {
namespace f32 {

// Shared body of the plain and the strided-batched entry points (batch == 1, strides 0: plain).
static int entry(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda,
                 int64_t ldb, int64_t ldc, int64_t stride_a, int64_t stride_b, int64_t stride_c, int config, void* stream) {
  if (M < 0 || N < 0 || K < 0 || batch < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "sgemm_f32: negative size");
  if (M == 0 || N == 0 || batch == 0) return GEMM_B200_OK;
  if (!C || (K > 0 && (!A || !B))) return fail(GEMM_B200_ERR_INVALID_ARG, "sgemm_f32: null pointer");
  if (lda < K || ldb < N || ldc < N)
    return fail(GEMM_B200_ERR_INVALID_ARG, "sgemm_f32: leading dimension smaller than the row (lda=%lld ldb=%lld ldc=%lld)",
                (long long)lda, (long long)ldb, (long long)ldc);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff || batch > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "sgemm_f32: a dimension exceeds 2^31-1");
  if (batch > 1) {
    // matrices of one operand must not interleave; 0 shares A or B between the problems
    if (stride_a < 0 || stride_b < 0 || (stride_a != 0 && stride_a < (M - 1) * lda + K) ||
        (stride_b != 0 && stride_b < (K - 1) * ldb + N) || stride_c < (M - 1) * ldc + N)
      return fail(GEMM_B200_ERR_INVALID_ARG,
                  "sgemm_f32_batched: a batch stride is smaller than its matrix (stride_a=%lld stride_b=%lld stride_c=%lld)",
                  (long long)stride_a, (long long)stride_b, (long long)stride_c);
  } else {
    stride_a = stride_b = stride_c = 0;
  }
  if (config >= kNumConfigs) return fail(GEMM_B200_ERR_INVALID_ARG, "sgemm_f32: config %d out of range", config);
  if (config < 0) {
    static thread_local int cached_dev = -1, cached_sms = 148;
    int dev = 0;
    GEMM_B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev != cached_dev) {
      GEMM_B200_CUDA_TRY(cudaDeviceGetAttribute(&cached_sms, cudaDevAttrMultiProcessorCount, dev));
      cached_dev = dev;
    }
    static const int forced = env_int("GEMM_B200_F32_CONFIG", -1);
    config = (forced >= 0 && forced < kNumConfigs) ? forced : pick_config(M, N, cached_sms, batch);
  }
  const bool vec = (lda % 4 == 0) && (ldb % 4 == 0) && (ldc % 4 == 0) && (K % 4 == 0) && (N % 4 == 0) &&
                   (stride_a % 4 == 0) && (stride_b % 4 == 0) && (stride_c % 4 == 0) &&
                   ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
                     reinterpret_cast<uintptr_t>(C)) % 16 == 0);
  if (log_enabled())
    fprintf(stderr, "[gemm_b200] sgemm_f32 %lldx%lldx%lld -> %s%s\n", (long long)M, (long long)K, (long long)N,
            kConfigs[config].name, vec ? "" : " (4-byte loads)");
  return kConfigs[config].launch(A, B, C, (int)M, (int)N, (int)K, lda, ldb, ldc, vec, static_cast<cudaStream_t>(stream),
                                 (int)batch, stride_a, stride_b, stride_c);
}

}  // namespace f32
}  // namespace gemm_b200

extern "C" int gemm_b200_sgemm_f32_cfg(const float* A, const float* B, float* C, int64_t M, int64_t N,
                                       int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int config,
                                       void* stream) {
  return gemm_b200::f32::entry(A, B, C, 1, M, N, K, lda, ldb, ldc, 0, 0, 0, config, stream);
}

extern "C" int gemm_b200_sgemm_f32(const float* A, const float* B, float* C, int64_t M, int64_t N, int64_t K,
                                   int64_t lda, int64_t ldb, int64_t ldc, void* stream) {
  return gemm_b200::f32::entry(A, B, C, 1, M, N, K, lda, ldb, ldc, 0, 0, 0, -1, stream);
}

extern "C" int gemm_b200_sgemm_f32_batched(const float* A, const float* B, float* C, int64_t batch, int64_t M, int64_t N,
                                           int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t stride_a,
                                           int64_t stride_b, int64_t stride_c, void* stream) {
  return gemm_b200::f32::entry(A, B, C, batch, M, N, K, lda, ldb, ldc, stride_a, stride_b, stride_c, -1, stream);
}

extern "C" int gemm_b200_sgemm_f32_num_configs(void) { return gemm_b200::f32::kNumConfigs; }
extern "C" const char* gemm_b200_sgemm_f32_config_name(int config) {
  if (config < 0 || config >= gemm_b200::f32::kNumConfigs) return "";
  return gemm_b200::f32::kConfigs[config].name;
}

#ifdef GEMM_B200_DEBUG
// Bounds-checking build only: reads and clears the status word of the FP32 kernels' checks
// ({code, block, site, byte offset}; code 0 = clean) and sets the test knob `shrink`.
extern "C" int gemm_b200_debug_bounds_f32(int32_t out[4], long long shrink) { return gemm_b200::dbg::read_bounds(out, shrink); }
#endif
