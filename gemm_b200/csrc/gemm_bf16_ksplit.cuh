// BF16 GEMM for problems with few output tiles: K is split across the CTAs of a thread-block
// cluster and the partial sums are combined through distributed shared memory, in one launch and
// without scratch in global memory.
//
// Same operator as gemm_bf16_kernel (C[M,N] = A[M,K] @ B, FP32 accumulation; the reference computes
// it in FP32 on CUDA cores: naive/naive_1.cu:5-15, shared/shared_2.cu:4-57,
// blocktile_1d/blocktile_1d.cu:5-68).
//
// A cluster of S = 2, 4 or 8 CTAs owns one 128 x 128 tile of C.  CTA r multiplies the r-th range of
// K into its own TMEM accumulator (single-CTA tcgen05.mma, TMA ring, one producer warp, one MMA
// warp, as in the main kernel).  Then the four epilogue warps of every CTA
//   1. stage, for every other CTA d, the 128 / S accumulator columns that d will finish in their
//      own shared memory (the operand ring is free by then) and send them to d's landing zone
//      with one bulk shared-memory-to-shared-memory copy per warp and destination, which
//      completes on d's barrier by byte count (element-wise remote stores of a lane-per-row
//      layout took 5 us here, the bulk copies take well under one);
//   2. wait until all S - 1 pieces for their own columns have landed, add the S partial sums in
//      ascending CTA order (their own comes from TMEM at its place in that order) and store the
//      128 x (128 / S) piece of C.
// Every CTA therefore reduces and stores an equal share, the order of the additions is fixed, and
// the result does not depend on timing.  A CTA leaves only after everything addressed to it has
// arrived, so no peer writes into the shared memory of a CTA that has exited.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"
#include "tc_common.cuh"
#include "gemm_bf16.cuh"

namespace gemm_b200 {
namespace tc {

constexpr int kKsBN = 128;                // tile width
constexpr int kKsStages = 4;
constexpr int kKsThreads = 192;           // producer warp, MMA warp, 4 epilogue warps
constexpr int kKsABytes = kBlockM * kBlockK * 2;          // 16 KB
constexpr int kKsBBytes = kKsBN * kBlockK * 2;            // 16 KB
constexpr int kKsStageBytes = kKsABytes + kKsBBytes;
// landing zone: (S - 1) pieces of 128 rows x (128 / S) columns of FP32, rows padded by 16 bytes
// (the 16-byte stores of a quarter warp then fall in distinct banks): at most 7/8 x 64 KB + padding
constexpr int kKsLandBytes = 7 * 128 * (16 + 4) * 4;      // S = 8 is the largest: 71680 bytes
constexpr int kKsBarBytes = (2 * kKsStages + 2) * 8 + 16;
constexpr int kKsSmemBytes = 1024 + kKsStages * kKsStageBytes + kKsLandBytes + kKsBarBytes;
static_assert(kKsSmemBytes <= 232448, "shared memory budget");

// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// bulk copy from this CTA's shared memory into a peer's; completes `bytes` on the peer's barrier
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, uint32_t src_addr, uint32_t bytes, uint32_t cluster_bar) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster_addr), "r"(src_addr), "r"(bytes), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}

struct KsShape {
  int M, N, K;
  int tiles_n;        // column tiles of kKsBN; the grid has tiles_m * tiles_n clusters
  int kb_per_split;   // K blocks (of kBlockK) per CTA of the cluster; no CTA's range is empty
};

template <bool B_MN, bool OUT_F32>
__global__ void __launch_bounds__(kKsThreads, 1)
gemm_bf16_cluster_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                void* __restrict__ Cptr, int64_t ldc, const KsShape shape) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA0 = smem_base;
  const uint32_t sB0 = smem_base + kKsStages * kKsABytes;
  const uint32_t land0 = smem_base + kKsStages * kKsStageBytes;
  const uint32_t bar0 = land0 + kKsLandBytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kKsStages + s); };
  const uint32_t tfull_bar = bar0 + 8u * (2 * kKsStages);
  const uint32_t landed_bar = bar0 + 8u * (2 * kKsStages + 1);
  const uint32_t tmem_slot = bar0 + 8u * (2 * kKsStages + 2);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t S = cluster_nctarank();
  const uint32_t rank = cluster_ctarank();
  const int tile = blockIdx.x / (int)S;
  const int tm = tile / shape.tiles_n, tn = tile % shape.tiles_n;
  const int m0 = tm * kBlockM, n0 = tn * kKsBN;
  const int num_kb = (shape.K + kBlockK - 1) / kBlockK;
  const int kb0 = (int)rank * shape.kb_per_split;
  const int kb1 = min(num_kb, kb0 + shape.kb_per_split);
  const int W = kKsBN / (int)S;                 // columns of C this CTA finishes
  const uint32_t land_pitch = (uint32_t)(W + 4) * 4u;   // bytes per padded row of a landed piece

  if (threadIdx.x == 0) {
    trace_stamp(0);
    for (int s = 0; s < kKsStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(landed_bar, 1);
    fence_mbar_init();
    // everything addressed to this CTA: S - 1 pieces of 128 padded rows
    mbar_arrive_expect_tx(landed_bar, (S - 1) * 128u * land_pitch);
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, kKsBN);
    tmem_relinquish<1>();
    tc_fence_before_sync();
  }
  __syncthreads();
  cluster_arrive();      // every CTA's barriers exist before any peer arrives on them
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = ld_shared_u32(tmem_slot);
  if (threadIdx.x == 0) trace_stamp(1);
  // programmatic dependent launch: wait for the kernel before this one, let the one behind it be scheduled
  pdl_wait();
  pdl_launch_dependents();

  bool failed = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    const bool issuer = elect_one();
    uint32_t it = 0;
    for (int kb = kb0; kb < kb1; ++kb, ++it) {
      const int s = it % kKsStages;
      const uint32_t ph = (it / kKsStages) & 1u;
      if (!mbar_wait_warp(empty_bar(s), ph ^ 1u, kRoleProducer, s)) { failed = true; break; }
      if (issuer) {
        if (it == 0) trace_stamp(2);
        mbar_arrive_expect_tx(full_bar(s), kKsStageBytes);
        tma_load_3d(sA0 + s * kKsABytes, &tmA, kb * kBlockK, m0, 0, full_bar(s));
        const uint32_t b_dst = sB0 + s * kKsBBytes;
        if constexpr (B_MN) {
#pragma unroll
          for (int j = 0; j < kKsBN / 64; ++j) tma_load_3d(b_dst + j * 8192, &tmB, n0 + j * 64, kb * kBlockK, 0, full_bar(s));
        } else {
          tma_load_3d(b_dst, &tmB, kb * kBlockK, n0, 0, full_bar(s));
        }
      }
      __syncwarp();
    }
    if (issuer) trace_stamp(3);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const bool issuer = elect_one();
    constexpr uint32_t idesc = make_idesc_bf16(kBlockM, kKsBN, 0, B_MN ? 1 : 0);
    constexpr uint64_t a_hi = make_smem_desc_hi(16, 1024, kLayoutSw128);
    constexpr uint64_t b_hi = B_MN ? make_smem_desc_hi(8192, 1024, kLayoutSw128) : make_smem_desc_hi(16, 1024, kLayoutSw128);
    constexpr uint32_t b_kstep = B_MN ? (kUmmaK * 128) : (kUmmaK * 2);
    uint32_t it = 0;
    for (int kb = kb0; kb < kb1; ++kb, ++it) {
      const int s = it % kKsStages;
      const uint32_t ph = (it / kKsStages) & 1u;
      if (!mbar_wait_warp(full_bar(s), ph, kRoleMma, s)) { failed = true; break; }
      tc_fence_after_sync();
      if (it == 0 && issuer) trace_stamp(4);
      const uint32_t a_addr = sA0 + s * kKsABytes, b_addr = sB0 + s * kKsBBytes;
      if (issuer) {
#pragma unroll
        for (int k = 0; k < kBlockK / kUmmaK; ++k)
          mma_f16<1>(tmem_base, smem_desc(a_hi, a_addr + k * (kUmmaK * 2)), smem_desc(b_hi, b_addr + k * b_kstep), idesc,
                     (k != 0 || kb != kb0) ? 1u : 0u);
        mma_commit_local(empty_bar(s));
      }
      __syncwarp();
    }
    if (!failed) {
      if (issuer) { trace_stamp(5); mma_commit_local(tfull_bar); }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..5
    const int quad = warp & 3;                       // TMEM lanes [32 quad, 32 quad + 32)
    const int row_in_tile = quad * 32 + lane;
    const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
    const bool ready = mbar_wait(tfull_bar, 0, kRoleEpilogue, 200);
    if (!__all_sync(0xffffffffu, ready)) {
      failed = true;
    } else {
      tc_fence_after_sync();
      if (warp == 2 && lane == 0) trace_stamp(6);
      // 1. hand every other CTA its columns of this CTA's partial sums: staged in the operand ring
      //    (every MMA that read it has completed: the accumulator barrier says so), then one bulk
      //    copy of this warp's 32 padded rows per destination
      for (uint32_t d = 0; d < S; ++d) {
        if (d == rank) continue;
        const uint32_t stage_rows = smem_base + (d * 128u + (uint32_t)(quad * 32)) * land_pitch;
        const uint32_t my_row = stage_rows + (uint32_t)lane * land_pitch;
        for (int c = 0; c < W; c += 16) {
          uint32_t v[16];
          tmem_ld_32x32b_x16(t_addr + d * W + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 4; ++j)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + (uint32_t)(c + 4 * j) * 4u), "r"(v[4 * j]),
                         "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3]) : "memory");
        }
        fence_proxy_async_smem();      // the bulk copy reads through the async proxy
        __syncwarp();
        if (lane == 0) {
          // pieces land in the order of their source, skipping the destination itself
          const uint32_t piece = rank < d ? rank : rank - 1;
          bulk_copy_to_peer(map_to_cta(land0 + (piece * 128u + (uint32_t)(quad * 32)) * land_pitch, d), stage_rows,
                            32u * land_pitch, map_to_cta(landed_bar, d));
        }
      }
      // 2. finish this CTA's own columns
      if (warp == 2 && lane == 0) trace_stamp(7);
      const bool landed = mbar_wait_cluster(landed_bar, 0, kRoleEpilogue, 210);
      if (warp == 2 && lane == 0) trace_stamp(8);
      if (!__all_sync(0xffffffffu, landed)) {
        failed = true;
      } else {
        const int row = m0 + row_in_tile;
        for (int c = 0; c < W; c += 16) {
          uint32_t own[16];
          tmem_ld_32x32b_x16(t_addr + rank * W + c, own);
          tmem_ld_wait();
          float acc[16];
          bool first = true;
          for (uint32_t s = 0; s < S; ++s) {
            float part[16];
            if (s == rank) {
#pragma unroll
              for (int j = 0; j < 16; ++j) part[j] = __uint_as_float(own[j]);
            } else {
              const uint32_t piece = s < rank ? s : s - 1;
              const uint32_t src = land0 + (piece * 128u + (uint32_t)row_in_tile) * land_pitch + (uint32_t)c * 4u;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t a, b, cc, dd;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(cc), "=r"(dd) : "r"(src + 16u * j) : "memory");
                part[4 * j] = __uint_as_float(a); part[4 * j + 1] = __uint_as_float(b);
                part[4 * j + 2] = __uint_as_float(cc); part[4 * j + 3] = __uint_as_float(dd);
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = first ? part[j] : acc[j] + part[j];
            first = false;
          }
          const int col = n0 + (int)rank * W + c;
          if (row < shape.M) {
            if constexpr (OUT_F32) {
              float* dst = reinterpret_cast<float*>(Cptr) + (int64_t)row * ldc + col;
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (col + 4 * j < shape.N)
                  *reinterpret_cast<float4*>(dst + 4 * j) = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cptr) + (int64_t)row * ldc + col;
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                if (col + 8 * j < shape.N) {
                  uint32_t p[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(acc[8 * j + 2 * e], acc[8 * j + 2 * e + 1]);
                    p[e] = *reinterpret_cast<uint32_t*>(&h);
                  }
                  *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(p[0], p[1], p[2], p[3]);
                }
              }
            }
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (failed || aborted()) {
    // give copies and MMAs still in flight time to land before shared memory and TMEM go away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (threadIdx.x == 64) trace_stamp(9);
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();      // nobody leaves while a peer may still be writing into its landing zone
  cluster_wait();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, kKsBN);
    if (lane == 0) trace_stamp(10);
  }
}

}  // namespace tc
}  // namespace gemm_b200
