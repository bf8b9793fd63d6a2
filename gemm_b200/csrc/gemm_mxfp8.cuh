// MXFP8 block-scaled GEMM on the sm_100a tensor cores:
//   C[M,N] = (Aq * SFA)[M,K] @ (Bq * SFB)[N,K]^T,  e4m3 data, one UE8M0 scale per 32 k,
//   FP32 accumulation in TMEM, bf16 or f32 output.
//
// Same operator as the reference's C = A @ B (naive/naive.cpp:6-22, kernels
// naive/naive_1.cu:5-15, shared/shared_2.cu:4-57, blocktile_1d/blocktile_1d.cu:5-68) on
// microscaled operands, which the reference does not have.
//
// Persistent, warp-specialised, 320 threads:
//   warp 0      TMA producer: A and B tiles (128 rows x 128 bytes, 128B swizzle) and the packed
//               scale chunks of the same K range (512 bytes per 128 rows) into a smem ring;
//   warp 1      owns TMEM; copies the scales smem -> TMEM (tcgen05.cp) and issues
//               tcgen05.mma kind::mxf8f6f4.block_scale (K = 32 per instruction).  Warps 0 and 1
//               run their loops as whole warps (warp-uniform addresses and descriptors) and
//               one elect.sync-elected lane executes the issuing instructions;
//   warps 2-9   epilogue: each warp pulls 32 rows x 128 columns of the accumulator into
//               registers, releases the accumulator at once, then converts and stores (swizzled
//               staging + TMA store, or direct 16-byte stores for split-K partial sums).
// The 256-column accumulator plus the scale columns do not fit twice in the 512 TMEM columns,
// so the accumulator is single-buffered; draining it to registers first keeps the tensor pipe
// idle only for the TMEM read, not for the global stores.
// With CG = 2 a CTA pair shares a 256 x 256 tile; every CTA loads the scales of all 256 columns
// of B because each SM applies them locally.  No load uses cluster multicast.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"
#include "tc_common.cuh"
#include "gemm_bf16.cuh"
#include "quant_mxfp8.cuh"

namespace gemm_b200 {
namespace tc {

constexpr int kMxBlockK = 128;     // e4m3 elements per 128-byte swizzled row = 4 scale blocks
constexpr int kMxUmmaK = 32;
constexpr int kMxThreads = 320;
constexpr int kMxSfaCol = 256;     // TMEM columns [256, 260): scales of A
constexpr int kMxSfbCol = 260;     // TMEM columns [260, 268): scales of B (256 columns of C)

// EPI: 0 = direct 16-byte global stores (also the split-K partial sums);
//      1 = per-warp swizzled staging in shared memory + TMA store (full 128-byte lines).
// A_ROWS: rows of A a stage loads (the TMA box).  128 = the whole row block.  Fewer (skinny
//      problems, M <= A_ROWS): the MMA still reads 128 rows of shared memory, but only the first
//      A_ROWS are loaded; consecutive stages sit A_ROWS rows apart, so the rows above a stage's
//      own are another stage's bytes or stale ones.  They only reach accumulator rows >= M, which
//      are never stored, and the shared memory saved buys more stages of B in flight.
// BN:  columns of C per tile (per CTA for CG = 1, per CTA pair for CG = 2): 256, or 128 for problems
//      whose 256-column tiles would not fill one round of the persistent grid.
// DYN: work units handed out at run time (see SchedRing) instead of unit = cluster + i * clusters.
template <int CG_, int STAGES_, bool COMMIT_MASK_, int EPI_ = 0, int A_ROWS_ = kBlockM, int BN_ = kBlockN, bool DYN_ = false>
struct MxCfg {
  static constexpr int CG = CG_, STAGES = STAGES_, EPI = EPI_, A_ROWS = A_ROWS_, BN = BN_;
  static constexpr bool COMMIT_MASK = COMMIT_MASK_, DYN = DYN_;
  static constexpr int NCH = BN / 64;                       // 32-column accumulator chunks per epilogue warp
  static constexpr int BN_CTA = BN / CG;
  static constexpr int A_BYTES = A_ROWS * kMxBlockK;        // bytes a stage loads and the stage pitch (16 KB for 128 rows)
  static constexpr int A_RING_BYTES = STAGES * A_BYTES + (kBlockM - A_ROWS) * kMxBlockK;
  static constexpr int B_BYTES = BN_CTA * kMxBlockK;        // 32 KB / 16 KB
  static constexpr int SFA_BYTES = 512;
  static constexpr int SFB_BYTES = (BN / 128) * 512;        // one scale chunk per 128 columns of C
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
  static constexpr int EPI_WARP_BUF = 32 * 128;             // 32 rows x 128 bytes per epilogue warp
  static constexpr int EPI_BYTES = EPI == 1 ? 8 * EPI_WARP_BUF : 0;
  static constexpr int BAR_BYTES = (2 * STAGES + 2) * 8 + 16 + (DYN ? kSchedBytes : 0);
  static_assert(STAGES + 5 <= kSchedSlots, "the unit ring must outlast the producer's lead over the epilogue");
  static constexpr int SMEM_BYTES = 1024 + A_RING_BYTES + STAGES * (B_BYTES + SFA_BYTES + SFB_BYTES) + EPI_BYTES + BAR_BYTES;
  static_assert(A_ROWS % 8 == 0 && A_ROWS >= 8 && A_ROWS <= kBlockM, "A rows per stage: whole 8-row swizzle atoms");
  static_assert(A_ROWS == kBlockM || CG == 1, "narrow A stages are a single-CTA variant");
  static_assert(BN == 256 || BN == 128, "tile width");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

// Grouped problems: group g multiplies the 128-row blocks [first_block[g], first_block[g + 1]) of one
// tall A (and its packed scales) by its own B_g into the same rows of one tall C.  The B matrices
// and their scale buffers follow one another, so B_g starts N rows (and ceil(N / 128) scale blocks)
// after B_{g-1}; only the producer warp needs to know the group.  Every group is a whole number of
// row tiles (256 rows for CTA pairs), so no tile spans two groups.  count == 0: not grouped.
struct MxGroups {
  int count;
  int first_block[kMaxGroups + 1];
};

// OUT: 0 = bf16, 1 = f32, 2 = MXFP8 (C quantised along its columns: e4m3 data to Cptr, one UE8M0
// scale per 32 columns to SFC in the packed layout, exactly what quantising the bf16 result gives)
template <class Cfg, int OUT>
__global__ void __launch_bounds__(kMxThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                  const __grid_constant__ CUtensorMap tmC, void* __restrict__ Cptr, int64_t ldc,
                  uint8_t* __restrict__ SFC, const GemmShape shape, const __grid_constant__ MxGroups groups) {
  constexpr int CG = Cfg::CG, STAGES = Cfg::STAGES;
  constexpr bool OUT_F32 = (OUT == 1);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA0 = smem_base;
  const uint32_t sB0 = sA0 + Cfg::A_RING_BYTES;
  // epilogue staging right after the A/B ring keeps it 1024-byte aligned (128B-swizzled TMA store);
  // the scale ring (512 / 1024 bytes per stage) and the barriers follow
  const uint32_t sEpi0 = sB0 + STAGES * Cfg::B_BYTES;
  const uint32_t sSFA0 = sEpi0 + Cfg::EPI_BYTES;
  const uint32_t sSFB0 = sSFA0 + STAGES * Cfg::SFA_BYTES;
  const uint32_t bar0 = sSFB0 + STAGES * Cfg::SFB_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t tfull_bar = bar0 + 8u * (2 * STAGES);
  const uint32_t tempty_bar = bar0 + 8u * (2 * STAGES + 1);
  const uint32_t tmem_slot = bar0 + 8u * (2 * STAGES + 2);
  const SchedRing ring{bar0 + 8u * (2 * STAGES + 2) + 16u};   // only with Cfg::DYN
  constexpr bool DYN = Cfg::DYN;

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / CG;
  const int num_clusters = gridDim.x / CG;
  const int num_kb = (shape.K + kMxBlockK - 1) / kMxBlockK;
  // work units: (tile, K split), consecutive units share the tile
  const int num_units = shape.tiles_m * shape.tiles_n * shape.k_splits;
  auto unit_range = [&](int u, int& tile, int& split, int& kb0, int& kb1) {
    tile = u / shape.k_splits;
    split = u - tile * shape.k_splits;
    kb0 = split * shape.kb_per_split;
    kb1 = min(num_kb, kb0 + shape.kb_per_split);
  };

  if (threadIdx.x == 0) {
    trace_stamp(0);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 8 * CG);   // one arrival per epilogue warp of every CTA of the pair
    if constexpr (DYN) ring.init();
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    prefetch_tensormap(&tmSFA);
    prefetch_tensormap(&tmSFB);
    if (Cfg::EPI == 1) prefetch_tensormap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc<CG>(tmem_slot, kTmemCols);
    tmem_relinquish<CG>();
    tc_fence_before_sync();
  }
  __syncthreads();
  if (CG == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after_sync();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");
  // split-K: lets the reduce kernel behind this one be scheduled early; it waits for this grid
  // programmatic dependent launch: wait for the kernel before this one, let the one behind it be scheduled
  // (see gemm_bf16_kernel)
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) trace_stamp(1);

  bool failed = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the schedule; one elected lane issues the copies.
    const bool issuer = elect_one();
    const bool stream_b = (CG == 1) && shape.l2_stream_a_keep_b != 0;   // set by the host for single-row-tile problems
    const uint64_t pol_b = stream_b ? l2_policy_evict_first() : 0ull;
    uint32_t it = 0, n = 0;   // n: how many units this cluster has started
    int u = cluster_id;
    while (u >= 0 && u < num_units && !failed) {
      int t, split, kb0, kb1, tm, tn;
      unit_range(u, t, split, kb0, kb1);
      tile_coord(t, shape, tm, tn);
      const int mblk = tm * CG + (int)cta_rank;            // 128-row block of A / C
      const int m0 = mblk * kBlockM;
      int n0 = tn * Cfg::BN + (int)cta_rank * Cfg::BN_CTA;    // row of the (stacked) B matrices
      int sfb_blk = tn * (Cfg::BN / 128);                      // 128-row block of their scales
      if (groups.count > 0) {
        int lo = 0, hi = groups.count - 1;                    // the last group that starts at or before this row block
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (groups.first_block[mid] <= mblk) lo = mid; else hi = mid - 1;
        }
        n0 += lo * shape.N;
        sfb_blk += lo * ((shape.N + 127) / 128);
      }
      if constexpr (DYN) {
        if (cta_rank == 0 && issuer) ring.request(n + 1);   // the answer arrives while this unit loads
      }
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        if (!mbar_wait_warp(empty_bar(s), ph ^ 1u, kRoleProducer, s)) { failed = true; break; }
        const uint32_t a_dst = sA0 + s * Cfg::A_BYTES, b_dst = sB0 + s * Cfg::B_BYTES;
        const uint32_t sfa_dst = sSFA0 + s * Cfg::SFA_BYTES, sfb_dst = sSFB0 + s * Cfg::SFB_BYTES;
        if (it == 0 && issuer) trace_stamp(2);
        // scale maps: 32-bit elements, row = 128-row block, 128 elements (512 bytes) per K chunk
        if constexpr (CG == 1) {
          if (issuer) {
            mbar_arrive_expect_tx(full_bar(s), Cfg::STAGE_BYTES);
            tma_load_2d(a_dst, &tmA, kb * kMxBlockK, m0, full_bar(s));
            // one row tile: every byte of B is read once, by this CTA.  Evict-first keeps the stream
            // from pushing other data (the caller's, or dirty lines that would have to be written
            // back while this kernel reads) out of the L2
            if (stream_b) tma_load_2d_hint(b_dst, &tmB, kb * kMxBlockK, n0, full_bar(s), pol_b);
            else tma_load_2d(b_dst, &tmB, kb * kMxBlockK, n0, full_bar(s));
            tma_load_2d(sfa_dst, &tmSFA, kb * 128, mblk, full_bar(s));
            tma_load_2d(sfb_dst, &tmSFB, kb * 128, sfb_blk, full_bar(s));
          }
        } else {
          const uint32_t lead_full = map_to_cta(full_bar(s), 0);
          if (issuer) {
            if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * Cfg::STAGE_BYTES);
            tma_load_2d_pair(a_dst, &tmA, kb * kMxBlockK, m0, lead_full);
            tma_load_2d_pair(b_dst, &tmB, kb * kMxBlockK, n0, lead_full);
            tma_load_2d_pair(sfa_dst, &tmSFA, kb * 128, mblk, lead_full);
            tma_load_2d_pair(sfb_dst, &tmSFB, kb * 128, sfb_blk, lead_full);
          }
        }
        __syncwarp();
      }
      if (failed) break;
      if (issuer) trace_stamp(3);
      ++n;
      if constexpr (DYN) {
        u = (cta_rank == 0) ? ring.template fetch_and_publish<CG>(n, issuer) : ring.wait_unit(n, kRoleProducer);
        if (u == -2) failed = true;
      } else {
        u += num_clusters;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    // The whole warp runs the loop, so shared-memory addresses, descriptors and TMEM addresses
    // are warp-uniform; one elected lane issues the tcgen05 instructions.
    if (cta_rank == 0) {
      const bool issuer = elect_one();
      constexpr uint64_t ab_hi = make_smem_desc_hi(16, 1024, kLayoutSw128);
      // scale chunk: 32 rows x 16 bytes, unswizzled, 8-row groups 128 bytes apart
      constexpr uint64_t sf_hi = make_smem_desc_hi(16, 128, kLayoutNone);
      auto commit = [&](uint32_t bar) {
        if constexpr (CG == 1) {
          mma_commit_local(bar);
        } else if constexpr (Cfg::COMMIT_MASK) {
          mma_commit_pair_mask(bar, (uint16_t)3);
        } else {
          mma_commit_pair(map_to_cta(bar, 0));
          mma_commit_pair(map_to_cta(bar, 1));
        }
      };
      const uint32_t d_tmem = tmem_base;
      const uint32_t sfa_tmem = tmem_base + kMxSfaCol, sfb_tmem = tmem_base + kMxSfbCol;
      uint32_t it = 0, acc_it = 0;
      int u = cluster_id;
      while (u >= 0 && u < num_units && !failed) {
        int t, split, kb0, kb1;
        unit_range(u, t, split, kb0, kb1);
        if (!mbar_wait_warp(tempty_bar, (acc_it & 1u) ^ 1u, kRoleMma, 100)) { failed = true; break; }
        tc_fence_after_sync();
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_warp(full_bar(s), ph, kRoleMma, s)) { failed = true; break; }
          tc_fence_after_sync();
          if (it == 0 && issuer) trace_stamp(4);
          const uint32_t a_addr = sA0 + s * Cfg::A_BYTES, b_addr = sB0 + s * Cfg::B_BYTES;
          const uint32_t sfa_addr = sSFA0 + s * Cfg::SFA_BYTES, sfb_addr = sSFB0 + s * Cfg::SFB_BYTES;
          const uint32_t first = (kb != kb0) ? 1u : 0u;
          if (issuer) {
            // tcgen05.cp and tcgen05.mma of one thread execute in issue order: these copies land
            // after the previous block's MMAs have read the scale columns and before the next ones do
            tmem_cp_32x128b_warpx4<CG>(sfa_tmem, smem_desc(sf_hi, sfa_addr));
#pragma unroll
            for (int c = 0; c < Cfg::BN / 128; ++c)
              tmem_cp_32x128b_warpx4<CG>(sfb_tmem + 4 * c, smem_desc(sf_hi, sfb_addr + 512 * c));
#pragma unroll
            for (int k = 0; k < kMxBlockK / kMxUmmaK; ++k) {
              // byte k of every 32-bit scale column belongs to this 32-wide K slice
              const uint32_t idesc = make_idesc_mxf8(kBlockM * CG, Cfg::BN, k, k);
              mma_mxf8<CG>(d_tmem, smem_desc(ab_hi, a_addr + k * kMxUmmaK), smem_desc(ab_hi, b_addr + k * kMxUmmaK), idesc,
                           sfa_tmem + ((uint32_t)k << 30), sfb_tmem + ((uint32_t)k << 30), k != 0 ? 1u : first);
            }
            commit(empty_bar(s));
          }
          __syncwarp();
        }
        if (failed) break;
        if (issuer) { trace_stamp(5); commit(tfull_bar); }
        __syncwarp();
        ++acc_it;
        if constexpr (DYN) {
          u = ring.wait_unit(acc_it, kRoleMma);
          if (u == -2) failed = true;
        } else {
          u += num_clusters;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps 2..9
    const int quad = warp & 3;             // TMEM lanes [32 quad, 32 quad + 32)
    constexpr int NCH = Cfg::NCH;
    const int half = (warp - 2) >> 2;      // columns [BN/2 half, BN/2 half + BN/2) of the tile
    const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(half * (Cfg::BN / 2));
    uint32_t acc_it = 0;
    int u = cluster_id;
    while (u >= 0 && u < num_units && !failed) {
      int t, split, kb0, kb1, tm, tn;
      unit_range(u, t, split, kb0, kb1);
      tile_coord(t, shape, tm, tn);
      const int row = (tm * CG + (int)cta_rank) * kBlockM + quad * 32 + lane;
      const int col0 = tn * Cfg::BN + half * (Cfg::BN / 2);
      const bool ready = mbar_wait(tfull_bar, acc_it & 1u, kRoleEpilogue, 200);
      if (!__all_sync(0xffffffffu, ready)) { failed = true; break; }
      tc_fence_after_sync();
      if (warp == 2 && lane == 0) trace_stamp(6);
      uint32_t v[NCH][32];
#pragma unroll
      for (int c = 0; c < NCH; ++c) tmem_ld_32x32b_x32(t_addr + c * 32, v[c]);
      tmem_ld_wait();
      // accumulator is in registers: the next tile's MMAs may overwrite it
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CG == 1) mbar_arrive(tempty_bar);
        else mbar_arrive_cluster(map_to_cta(tempty_bar, 0));
      }
      if constexpr (Cfg::EPI == 1 && OUT != 2) {
        // 128-byte-wide slabs (64 bf16 or 32 f32 columns) of this warp's 32 rows: swizzled staging,
        // then one TMA store per slab; rows / columns outside C are clipped by the tensor map
        const uint32_t buf = sEpi0 + (uint32_t)(warp - 2) * Cfg::EPI_WARP_BUF;
        const uint32_t row_addr = buf + (uint32_t)lane * 128u;
        const uint32_t sw = (uint32_t)(lane & 7);
        const int row0 = (tm * CG + (int)cta_rank) * kBlockM + quad * 32;
        constexpr int SLABS = OUT_F32 ? NCH : NCH / 2;
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          if (lane == 0) tma_store_wait_read<0>();   // the previous slab's store has read the buffer
          __syncwarp();
          if constexpr (OUT_F32) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)j ^ sw) << 4)),
                           "r"(v[sl][4 * j]), "r"(v[sl][4 * j + 1]), "r"(v[sl][4 * j + 2]), "r"(v[sl][4 * j + 3]) : "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              uint32_t p[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int idx = (j & 3) * 8 + 2 * e;     // column within the 32-column chunk
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * sl + (j >> 2)][idx]),
                                                         __uint_as_float(v[2 * sl + (j >> 2)][idx + 1]));
                p[e] = *reinterpret_cast<uint32_t*>(&h);
              }
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)j ^ sw) << 4)),
                           "r"(p[0]), "r"(p[1]), "r"(p[2]), "r"(p[3]) : "memory");
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          const int x = col0 + sl * (OUT_F32 ? 32 : 64);
          if (lane == 0) {
            if (row0 < shape.M && x < shape.N) tma_store_2d(&tmC, x, row0, buf);
            tma_store_commit();
          }
        }
      } else if constexpr (OUT == 2) {
        static_assert(Cfg::BN == 256, "the quantising epilogue is written for 256-column tiles");
        // each thread holds 32 consecutive columns of its row per chunk: one microscaling block.
        // Round to bf16 first so the bytes equal "bf16 GEMM output, then quantise".
        const int64_t kchunks = (((int64_t)shape.N / 32) + 3) / 4;       // scale chunks per row block of C
        const int64_t rows_pad = (((int64_t)shape.M + 127) / 128) * 128;
        // this thread's 4 blocks are blocks 4q .. 4q+3 of its row (col0 is a multiple of 128): their
        // scale bytes are 4 consecutive, 4-byte-aligned bytes of the packed layout -> one 32-bit store
        uint32_t scale_word = 0;
        if constexpr (Cfg::EPI == 1) {
          if (lane == 0) tma_store_wait_read<0>();   // the previous tile's store has read the staging buffer
          __syncwarp();
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int col = col0 + c * 32;
          if (row < shape.M && col < shape.N) {
            uint32_t w[16], q[8];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[c][2 * e]), __uint_as_float(v[c][2 * e + 1]));
              w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            const uint32_t byte = mx::quantise_block(w, q);
            scale_word |= byte << (8 * c);
            if constexpr (Cfg::EPI == 1) {
              // stage this warp's 32 rows x 128 bytes (128-byte swizzle); chunks 2c and 2c + 1 of the row
              const uint32_t row_addr = sEpi0 + (uint32_t)(warp - 2) * Cfg::EPI_WARP_BUF + (uint32_t)lane * 128u;
              const uint32_t sw = (uint32_t)(lane & 7);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)(2 * c) ^ sw) << 4)),
                           "r"(q[0]), "r"(q[1]), "r"(q[2]), "r"(q[3]) : "memory");
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)(2 * c + 1) ^ sw) << 4)),
                           "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]) : "memory");
            } else {
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(Cptr) + (int64_t)row * ldc + col);
              dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
              dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
            }
          }
        }
        if constexpr (Cfg::EPI == 1) {
          // rows / columns outside C hold stale bytes in the staging buffer; the store clips them
          fence_proxy_async_smem();
          __syncwarp();
          const int row0 = (tm * CG + (int)cta_rank) * kBlockM + quad * 32;
          if (lane == 0) {
            if (row0 < shape.M && col0 < shape.N)
              tma_store_2d(&tmC, col0, row0, sEpi0 + (uint32_t)(warp - 2) * Cfg::EPI_WARP_BUF);
            tma_store_commit();
          }
        }
        const int64_t nb0 = col0 / 32;
        if (row < rows_pad && nb0 < kchunks * 4)                          // inside the padded scale buffer
          *reinterpret_cast<uint32_t*>(SFC + mx::scale_offset(kchunks, row, nb0)) = scale_word;   // padding -> 0
      } else if (row < shape.M) {
        // extent of everything this launch may store to (bounds-checking build)
        const long long c_elems = (long long)(shape.k_splits - 1) * shape.split_stride + (long long)(shape.M - 1) * ldc + shape.N;
        (void)c_elems;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int col = col0 + c * 32;
          if constexpr (OUT_F32) {
            float* dst = reinterpret_cast<float*>(Cptr) + (int64_t)split * shape.split_stride + (int64_t)row * ldc + col;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (col + 4 * j < shape.N && GEMM_B200_IN_BOUNDS(dst + 4 * j, Cptr, c_elems * 4, 16, 20))
                *reinterpret_cast<uint4*>(dst + 4 * j) =
                    make_uint4(v[c][4 * j], v[c][4 * j + 1], v[c][4 * j + 2], v[c][4 * j + 3]);
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cptr) + (int64_t)row * ldc + col;   // k_splits == 1
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (col + 8 * j < shape.N && GEMM_B200_IN_BOUNDS(dst + 8 * j, Cptr, c_elems * 2, 16, 21)) {
                uint32_t p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[c][8 * j + 2 * e]),
                                                           __uint_as_float(v[c][8 * j + 2 * e + 1]));
                  p[e] = *reinterpret_cast<uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(p[0], p[1], p[2], p[3]);
              }
            }
          }
        }
      }
      ++acc_it;
      if constexpr (DYN) {
        u = ring.wait_unit(acc_it, kRoleEpilogue);
        if (u == -2) failed = true;
      } else {
        u += num_clusters;
      }
    }
    if (warp == 2 && lane == 0) trace_stamp(7);
    if (Cfg::EPI == 1 && lane == 0) tma_store_wait_all<0>();
    if (warp == 2 && lane == 0) trace_stamp(8);
  }

  // ------------------------------------------------------------------ teardown
  if (failed || aborted()) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (CG == 2) {
    cluster_arrive();
    cluster_wait();
  }
  if (threadIdx.x == 0) trace_stamp(9);
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<CG>(tmem_base, kTmemCols);
    if (lane == 0) trace_stamp(10);
  }
}

// Sums the k_splits FP32 partial results of a split-K run (slice s at W + s * split_stride, row
// pitch ldw) in ascending s, and writes C as bf16 or f32.  One thread per 4 columns.
template <bool OUT_F32>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ W, int64_t split_stride, int64_t ldw, int k_splits,
                     void* __restrict__ Cptr, int64_t ldc, int M, int N) {
  const int64_t n4 = N / 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();   // launched early behind the GEMM that writes W: returns once that grid is complete
  pdl_launch_dependents();
  if (idx >= (int64_t)M * n4) return;
  const int64_t r = idx / n4, c = (idx % n4) * 4;
  const float* src = W + r * ldw + c;
  const long long w_bytes = ((long long)(k_splits - 1) * split_stride + (long long)(M - 1) * ldw + N) * 4;
  const long long c_elems = (long long)(M - 1) * ldc + N;
  (void)w_bytes; (void)c_elems;
  // four slices are fetched before the first of them is added (the loads are independent, the
  // additions keep their ascending order)
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s0 = 0; s0 < k_splits; s0 += 4) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s0 + j < k_splits && GEMM_B200_IN_BOUNDS(src + (int64_t)(s0 + j) * split_stride, W, w_bytes, 16, 30))
        v[j] = *reinterpret_cast<const float4*>(src + (int64_t)(s0 + j) * split_stride);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (s0 + j == 0) {
        acc = v[0];
      } else if (s0 + j < k_splits) {
        acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w;
      }
    }
  }
  if (!GEMM_B200_IN_BOUNDS(reinterpret_cast<char*>(Cptr) + (r * ldc + c) * (OUT_F32 ? 4 : 2), Cptr, c_elems * (OUT_F32 ? 4 : 2),
                           OUT_F32 ? 16 : 8, 31))
    return;
  if constexpr (OUT_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(Cptr) + r * ldc + c) = acc;
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    uint2 p = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(Cptr) + r * ldc + c) = p;
  }
}

}  // namespace tc
}  // namespace gemm_b200
