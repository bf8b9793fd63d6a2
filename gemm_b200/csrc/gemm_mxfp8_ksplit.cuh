// MXFP8 block-scaled GEMM for problems with few output tiles: K is split across the CTAs of a
// thread-block cluster and the partial sums are combined through distributed shared memory, in one
// launch and without scratch in global memory.  The scheme is the one of gemm_bf16_ksplit.cuh
// (reduce-scatter of the FP32 accumulators with bulk shared-memory-to-shared-memory copies, sums
// in ascending CTA order); the main loop is the single-CTA one of gemm_mxfp8.cuh (128-byte K
// blocks, packed UE8M0 scale chunks copied smem -> TMEM by tcgen05.cp, four block-scaled MMAs of
// K = 32 per block).  Same operator as the reference's C = A @ B (naive/naive_1.cu:5-15) on
// microscaled operands, which the reference does not have.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"
#include "tc_common.cuh"
#include "gemm_bf16.cuh"
#include "gemm_bf16_ksplit.cuh"
#include "gemm_mxfp8.cuh"

namespace gemm_b200 {
namespace tc {

constexpr int kMxKsStages = 4;
constexpr int kMxKsABytes = kBlockM * kMxBlockK;          // 16 KB: 128 rows x 128 e4m3
constexpr int kMxKsBBytes = kKsBN * kMxBlockK;            // 16 KB
constexpr int kMxKsSfBytes = 512;                         // one packed scale chunk: 128 rows x 4 blocks of 32 k
constexpr int kMxKsStageBytes = kMxKsABytes + kMxKsBBytes + 2 * kMxKsSfBytes;
constexpr int kMxKsBarBytes = (2 * kMxKsStages + 2) * 8 + 16;
constexpr int kMxKsSmemBytes = 1024 + kMxKsStages * kMxKsStageBytes + kKsLandBytes + kMxKsBarBytes;
static_assert(kMxKsSmemBytes <= 232448, "shared memory budget");
static_assert(kMxKsStages * (kMxKsABytes + kMxKsBBytes) >= 8 * 128 * (16 + 4) * 4, "the operand ring must hold the staged pieces");
constexpr int kMxKsTmemCols = 256;                        // 128 accumulator columns + 4 + 4 scale columns
constexpr int kMxKsSfaCol = 128, kMxKsSfbCol = 132;       // even columns (a scale operand at an odd column faults)

// K blocks here are 128 e4m3 elements; KsShape::kb_per_split counts those.
template <bool OUT_F32>
__global__ void __launch_bounds__(kKsThreads, 1)
gemm_mxfp8_cluster_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                 const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                                 void* __restrict__ Cptr, int64_t ldc, const KsShape shape) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA0 = smem_base;
  const uint32_t sB0 = smem_base + kMxKsStages * kMxKsABytes;
  const uint32_t sSFA0 = sB0 + kMxKsStages * kMxKsBBytes;
  const uint32_t sSFB0 = sSFA0 + kMxKsStages * kMxKsSfBytes;
  const uint32_t land0 = smem_base + kMxKsStages * kMxKsStageBytes;
  const uint32_t bar0 = land0 + kKsLandBytes;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kMxKsStages + s); };
  const uint32_t tfull_bar = bar0 + 8u * (2 * kMxKsStages);
  const uint32_t landed_bar = bar0 + 8u * (2 * kMxKsStages + 1);
  const uint32_t tmem_slot = bar0 + 8u * (2 * kMxKsStages + 2);

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t S = cluster_nctarank();
  const uint32_t rank = cluster_ctarank();
  const int tile = blockIdx.x / (int)S;
  const int tm = tile / shape.tiles_n, tn = tile % shape.tiles_n;
  const int m0 = tm * kBlockM, n0 = tn * kKsBN;
  const int mblk = tm;                                   // 128-row block of A: row of the packed scale buffer
  const int num_kb = (shape.K + kMxBlockK - 1) / kMxBlockK;
  const int kb0 = (int)rank * shape.kb_per_split;
  const int kb1 = min(num_kb, kb0 + shape.kb_per_split);
  const int W = kKsBN / (int)S;                 // columns of C this CTA finishes
  const uint32_t land_pitch = (uint32_t)(W + 4) * 4u;   // bytes per padded row of a landed piece

  if (threadIdx.x == 0) {
    trace_stamp(0);
    for (int s = 0; s < kMxKsStages; ++s) {
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
    prefetch_tensormap(&tmSFA);
    prefetch_tensormap(&tmSFB);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, kMxKsTmemCols);
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
      const int s = it % kMxKsStages;
      const uint32_t ph = (it / kMxKsStages) & 1u;
      if (!mbar_wait_warp(empty_bar(s), ph ^ 1u, kRoleProducer, s)) { failed = true; break; }
      if (issuer) {
        if (it == 0) trace_stamp(2);
        mbar_arrive_expect_tx(full_bar(s), kMxKsStageBytes);
        tma_load_2d(sA0 + s * kMxKsABytes, &tmA, kb * kMxBlockK, m0, full_bar(s));
        tma_load_2d(sB0 + s * kMxKsBBytes, &tmB, kb * kMxBlockK, n0, full_bar(s));
        // scale maps: 32-bit elements, row = 128-row block, 128 elements (512 bytes) per K chunk
        tma_load_2d(sSFA0 + s * kMxKsSfBytes, &tmSFA, kb * 128, mblk, full_bar(s));
        tma_load_2d(sSFB0 + s * kMxKsSfBytes, &tmSFB, kb * 128, tn, full_bar(s));
      }
      __syncwarp();
    }
    if (issuer) trace_stamp(3);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const bool issuer = elect_one();
    constexpr uint64_t ab_hi = make_smem_desc_hi(16, 1024, kLayoutSw128);
    constexpr uint64_t sf_hi = make_smem_desc_hi(16, 128, kLayoutNone);   // 32 rows x 16 bytes, 8-row groups 128 bytes apart
    const uint32_t sfa_tmem = tmem_base + kMxKsSfaCol, sfb_tmem = tmem_base + kMxKsSfbCol;
    uint32_t it = 0;
    for (int kb = kb0; kb < kb1; ++kb, ++it) {
      const int s = it % kMxKsStages;
      const uint32_t ph = (it / kMxKsStages) & 1u;
      if (!mbar_wait_warp(full_bar(s), ph, kRoleMma, s)) { failed = true; break; }
      tc_fence_after_sync();
      if (it == 0 && issuer) trace_stamp(4);
      const uint32_t a_addr = sA0 + s * kMxKsABytes, b_addr = sB0 + s * kMxKsBBytes;
      if (issuer) {
        // tcgen05.cp and tcgen05.mma of one thread execute in issue order: these copies land after
        // the previous block's MMAs have read the scale columns and before the next ones do
        tmem_cp_32x128b_warpx4<1>(sfa_tmem, smem_desc(sf_hi, sSFA0 + s * kMxKsSfBytes));
        tmem_cp_32x128b_warpx4<1>(sfb_tmem, smem_desc(sf_hi, sSFB0 + s * kMxKsSfBytes));
#pragma unroll
        for (int k = 0; k < kMxBlockK / kMxUmmaK; ++k) {
          const uint32_t idesc = make_idesc_mxf8(kBlockM, kKsBN, k, k);   // byte k of every scale column
          mma_mxf8<1>(tmem_base, smem_desc(ab_hi, a_addr + k * kMxUmmaK), smem_desc(ab_hi, b_addr + k * kMxUmmaK), idesc,
                      sfa_tmem + ((uint32_t)k << 30), sfb_tmem + ((uint32_t)k << 30), (k != 0 || kb != kb0) ? 1u : 0u);
        }
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
    tmem_dealloc<1>(tmem_base, kMxKsTmemCols);
    if (lane == 0) trace_stamp(10);
  }
}

}  // namespace tc
}  // namespace gemm_b200
