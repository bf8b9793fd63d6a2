// BF16 GEMM on the sm_100a tensor cores: C[M,N] = A[M,K] @ B, FP32 accumulation in TMEM.
//
// Extends the reference operator (naive/naive.cpp:6-22; kernels naive/naive_1.cu:5-15,
// shared/shared_2.cu:4-57, blocktile_1d/blocktile_1d.cu:5-68 compute the same C = A @ B in
// FP32 on CUDA cores) to BF16 operands.
//
// One persistent, warp-specialised kernel (192 threads):
//   warp 0     TMA producer: 128B-swizzled tiles of A and B into a STAGES-deep smem ring;
//   warp 1     owns TMEM; issues tcgen05.mma (UMMA K = 16) and commits to mbarriers.  Warps 0
//              and 1 run their loops as whole warps (warp-uniform addresses and descriptors);
//              one elect.sync-elected lane executes the issuing instructions;
//   warps 2-5  epilogue: tcgen05.ld the FP32 accumulator, convert, store (direct 16-byte global
//              stores, or per-warp swizzled staging + TMA store).
// The accumulator is double-buffered in TMEM (2 x 256 columns) so the epilogue of tile i
// overlaps the main loop of tile i+1.  With CG = 2 two CTAs on neighbouring SMs share one
// 256x256 tile: each loads its own 128 rows of A and its own 128 columns of B, and the leader
// CTA issues one cta_group::2 MMA that reads both halves.  No load uses cluster multicast.
// Tiles are assigned statically (tile = cluster id + i * clusters) along a grouped raster that
// keeps the tiles in flight on a compact patch of C so A/B tiles are re-read from L2.
//
// B row-major [K,N] is fed as an "MN-major" UMMA operand (the k rows of a tile are 128-byte
// rows of 64 consecutive n); B given as Bt[N,K] is the usual K-major operand.
#pragma once
#include <cuda_bf16.h>
#include "common.cuh"
#include "tc_common.cuh"

namespace gemm_b200 {
namespace tc {

constexpr int kBlockM = 128;   // rows of C per CTA
constexpr int kBlockN = 256;   // columns of C per MMA (per CTA for CG = 1, per CTA pair for CG = 2)
constexpr int kBlockK = 64;    // bf16 elements per 128-byte swizzled row
constexpr int kUmmaK = 16;
constexpr int kTmemCols = 512;

// ---------------------------------------------------------------------------------------
// Run-time hand-out of work units (used by the BF16 and the MXFP8 kernel).
//
// The producer warp of the leader CTA asks the hardware for the next unit one unit ahead
// (clc_try_cancel) and, once the answer is in, publishes it to every CTA of the cluster through a
// ring in shared memory: a 32-bit unit index (-1 = no work left) and an mbarrier per slot.  Every
// other warp role walks the same ring.  Slot (n - 1) % kSchedSlots carries the n-th unit of the
// cluster (n >= 1; unit 0 is the cluster's own blockIdx), in phase ((n - 1) / kSchedSlots) & 1 of
// the slot's barriers.  No "slot free" signal is needed: the producer
// runs at most STAGES K blocks ahead of the MMA issuer and the issuer at most two accumulators
// ahead of the epilogue, so the slot written for unit n + 1 was last read STAGES + 3 units ago at
// the latest, and the ring holds more slots than that.
//   [0, 256)    kSchedSlots x 16 B  hardware answers           (used in the leader CTA)
//   [256, 384)  kSchedSlots x 8 B   mbarriers of the answers   (used in the leader CTA)
//   [384, 512)  kSchedSlots x 8 B   "unit published" mbarriers (every CTA)
//   [512, 576)  kSchedSlots x 4 B   published unit index       (every CTA)
// ---------------------------------------------------------------------------------------
constexpr int kSchedSlots = 16;
constexpr int kSchedBytes = 576;
struct SchedRing {
  uint32_t base;   // 16-byte aligned shared-memory address
  __device__ __forceinline__ uint32_t resp(uint32_t s) const { return base + 16u * s; }
  __device__ __forceinline__ uint32_t hw_bar(uint32_t s) const { return base + 256u + 8u * s; }
  __device__ __forceinline__ uint32_t pub_bar(uint32_t s) const { return base + 384u + 8u * s; }
  __device__ __forceinline__ uint32_t unit(uint32_t s) const { return base + 512u + 4u * s; }
  __device__ __forceinline__ void init() const {   // one thread, before the CTA-wide barrier
    for (uint32_t i = 0; i < (uint32_t)kSchedSlots; ++i) {
      mbar_init(hw_bar(i), 1);
      mbar_init(pub_bar(i), 1);
    }
  }
  // leader CTA's producer warp, one lane: ask for the cluster's n-th unit
  __device__ __forceinline__ void request(uint32_t n) const {
    const uint32_t s = (n - 1) % kSchedSlots;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // earlier reads of this slot before the new answer
    mbar_arrive_expect_tx(hw_bar(s), 16);
    clc_try_cancel(resp(s), hw_bar(s));
  }
  // leader CTA's producer warp, whole warp: wait for the answer to request(n) and hand the unit to
  // every CTA of the cluster.  Returns the unit (-1: none left), -2 if the wait gave up.
  template <int CG>
  __device__ __forceinline__ int fetch_and_publish(uint32_t n, bool issuer) const {
    const uint32_t s = (n - 1) % kSchedSlots;
    if (!mbar_wait_warp(hw_bar(s), ((n - 1) / kSchedSlots) & 1u, kRoleProducer, 300)) return -2;
    const int first = clc_first_cta(resp(s));
    const int unit_idx = first < 0 ? -1 : first / CG;
    if (issuer) {
      st_shared_u32(unit(s), (uint32_t)unit_idx);
      mbar_arrive(pub_bar(s));
      if constexpr (CG == 2) {
        st_shared_cluster_u32(map_to_cta(unit(s), 1), (uint32_t)unit_idx);
        mbar_arrive_cluster(map_to_cta(pub_bar(s), 1));
      }
    }
    __syncwarp();
    return unit_idx;
  }
  // every other role: the cluster's n-th unit (n >= 1); -2 if the wait gave up
  __device__ __forceinline__ int wait_unit(uint32_t n, int role) const {
    const uint32_t s = (n - 1) % kSchedSlots;
    const bool ok = mbar_wait_cluster(pub_bar(s), ((n - 1) / kSchedSlots) & 1u, role, 310);
    if (!__all_sync(0xffffffffu, ok)) return -2;
    return (int)ld_shared_u32(unit(s));
  }
};

// EPI: 0 = direct global stores, 1 = swizzled smem staging + TMA store
// COMMIT_MASK: CTA-pair commits use the masked form (one instruction for both CTAs) instead of two
// NT: column tiles of kBlockN per work unit.
//   NT = 1: one 256-column accumulator per tile, double-buffered in TMEM (the epilogue of a tile
//           overlaps the main loop of the next), 4 epilogue warps.
//   NT = 2: two 256-column accumulators (all 512 TMEM columns) that share the A tile: every A
//           tile fetched from L2 feeds twice the math, i.e. 25 % fewer operand bytes per flop
//           (less L2 / fabric power on a power-capped board) at the price of an epilogue that
//           is not overlapped; 8 epilogue warps keep that short.
// BN: columns of C per MMA / accumulator (256, or 128 for problems whose 256-column tiles would
//     leave most of the SMs without work).
// DYN: work units are handed out at run time instead of the static unit = cluster + i * clusters:
//     the grid has one cluster per unit, the clusters that get to run first keep running and adopt
//     the units of clusters that have not started (cluster launch control), so the units in flight
//     are always a contiguous window of the raster however far the clusters drift apart in time.
template <int CG_, int STAGES_, int EPI_, bool COMMIT_MASK_, int NT_ = 1, int EPI_BUFS_ = (NT_ == 1 ? 2 : 1),
          int BN_ = kBlockN, bool DYN_ = false>
struct Bf16Cfg {
  static constexpr int CG = CG_, STAGES = STAGES_, EPI = EPI_, NT = NT_, BN = BN_;
  static constexpr bool COMMIT_MASK = COMMIT_MASK_, DYN = DYN_;
  static constexpr int ACC_STAGES = (NT == 1) ? 2 : 1;
  static constexpr int EPI_WARPS = 4 * NT;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int EPI_BUFS = EPI_BUFS_;                       // staging buffers per epilogue warp
  static constexpr int TILE_N = BN * NT;                       // columns of C per work unit
  static constexpr int BN_CTA = BN / CG;                       // columns of B each CTA loads per column tile
  static constexpr int A_BYTES = kBlockM * kBlockK * 2;             // 16 KB
  static constexpr int B_BYTES = BN_CTA * kBlockK * 2;              // 32 KB / 16 KB, per column tile
  static constexpr int STAGE_BYTES = A_BYTES + NT * B_BYTES;
  static constexpr int EPI_WARP_BUF = 32 * 128;                     // 32 rows x 128 bytes
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUFS * EPI_WARP_BUF;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16 + (DYN ? kSchedBytes : 0);
  static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + BAR_BYTES;
  static_assert(STAGES + 5 <= kSchedSlots, "the unit ring must outlast the producer's lead over the epilogue");
  static_assert(NT == 1 || NT == 2, "column tiles per unit");
  static_assert(BN == 256 || (BN == 128 && NT == 1), "tile width");
  static_assert(SMEM_BYTES <= 232448, "shared memory budget");
};

struct GemmShape {
  int M, N, K;
  int tiles_m, tiles_n;   // work units of (kBlockM * CG) rows x (kBlockN * NT) columns
  // split-K: every tile is cut into k_splits work units of
  // kb_per_split K blocks; unit (tile, split) writes FP32 partial sums to slice `split` of a
  // scratch buffer [k_splits][M][ldc].  k_splits == 1: the tile's result goes straight to C.
  int k_splits, kb_per_split;
  int64_t split_stride;   // elements between scratch slices
  // raster: tiles are walked in bands of `raster_group` row tiles (> 0: a band spans all column
  // tiles, row index fastest) or of `-raster_group` column tiles (< 0: a band spans all row tiles,
  // column index fastest); the operand panel of the band stays in L2 while the other streams.
  int raster_group;
  // batched BF16 GEMM: `batch` independent problems of the same shape; a work unit is
  // (matrix, tile).  a_z / b_z are 1 when the operand has one matrix per problem and 0 when all
  // problems share one (batch stride 0).  c_batch_stride: elements between the C matrices.
  int batch, a_z, b_z;
  int64_t c_batch_stride;
  // BF16 kernel, 1: load A tiles with L2 priority evict-first and B tiles evict-last.  Set for
  // problems whose raster band lasts many rounds of units: there the band's B panel is re-read
  // every round while an A tile is needed only by the clusters of one round.  2: B tiles
  // evict-first and A tiles evict-last, for problems of one row tile, which stream B once.
  // MXFP8 kernel, non-zero: B tiles evict-first (single-CTA variants, one row tile).
  int l2_stream_a_keep_b;
};

// Grouped (ragged) problems: group g multiplies rows [row_start[g], row_start[g + 1]) of one tall A
// by its own B_g into the same rows of one tall C.  tile_start[g] = index of the group's first
// work unit; units of a group are ordered row tile by row tile.  count == 0: not a grouped launch.
constexpr int kMaxGroups = 64;
struct GroupTable {
  int count;
  int tile_start[kMaxGroups + 1];
  int row_start[kMaxGroups + 1];
};

__device__ __forceinline__ void tile_coord(int t, const GemmShape& sh, int& tm, int& tn) {
  if (sh.raster_group > 0) {
    const int group = sh.raster_group;
    const int width = group * sh.tiles_n;
    const int first_m = (t / width) * group;
    const int gsz = min(sh.tiles_m - first_m, group);
    tm = first_m + (t % width) % gsz;
    tn = (t % width) / gsz;
  } else {
    const int group = -sh.raster_group;
    const int width = group * sh.tiles_m;
    const int first_n = (t / width) * group;
    const int gsz = min(sh.tiles_n - first_n, group);
    tn = first_n + (t % width) % gsz;
    tm = (t % width) / gsz;
  }
}

template <class Cfg, bool B_MN, bool OUT_F32, bool A_MN = false>
__global__ void __launch_bounds__(Cfg::THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, void* __restrict__ Cptr, int64_t ldc,
                 const GemmShape shape, const __grid_constant__ GroupTable groups) {
  constexpr int CG = Cfg::CG, STAGES = Cfg::STAGES, NT = Cfg::NT, ACC_STAGES = Cfg::ACC_STAGES, BN = Cfg::BN;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sA0 = smem_base;
  const uint32_t sB0 = smem_base + STAGES * Cfg::A_BYTES;     // [stage][column tile][B_BYTES]
  const uint32_t sEpi0 = smem_base + STAGES * Cfg::STAGE_BYTES;
  const uint32_t bar0 = sEpi0 + Cfg::EPI_BYTES;
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar0 + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar0 + 8u * (2 * STAGES + 4);
  const SchedRing ring{bar0 + 8u * (2 * STAGES + 4) + 16u};   // only with Cfg::DYN
  constexpr bool DYN = Cfg::DYN;

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / CG;
  const int num_clusters = gridDim.x / CG;
  const int tiles_per_matrix = shape.tiles_m * shape.tiles_n;
  const int num_kb = (shape.K + kBlockK - 1) / kBlockK;
  // work units: (matrix, tile, K split); consecutive units share the tile.  k_splits > 1 only with
  // the direct-store FP32 epilogue: unit (tile, split) writes its partial sums to slice `split`
  // of the scratch buffer Cptr ([k_splits][M][ldc] floats).
  const bool grouped = groups.count > 0;
  const int num_tiles = grouped ? groups.tile_start[groups.count] : tiles_per_matrix * shape.batch * shape.k_splits;
  // tile index -> (matrix or group, row tile, column tile) and the rows [row_base, row_end) of A / C it
  // may touch (row tiles count from row_base)
  auto decode = [&](int t, int& bi, int& tm, int& tn, int& row_base, int& row_end) {
    if (grouped) {
      int lo = 0, hi = groups.count - 1;          // the last group whose first unit is <= t
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (groups.tile_start[mid] <= t) lo = mid; else hi = mid - 1;
      }
      const int local = t - groups.tile_start[lo];
      tm = local / shape.tiles_n;
      tn = local - tm * shape.tiles_n;
      bi = lo;
      row_base = groups.row_start[lo];
      row_end = groups.row_start[lo + 1];
    } else {
      bi = t / tiles_per_matrix;
      tile_coord(t - bi * tiles_per_matrix, shape, tm, tn);
      row_base = 0;
      row_end = shape.M;
    }
  };
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
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), Cfg::EPI_WARPS * CG);   // one arrival per epilogue warp of every CTA of the pair
    }
    if constexpr (DYN) ring.init();
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
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
  // Programmatic dependent launch.  This grid may have been scheduled while the kernel before it in
  // the stream was still running: nothing above touches global memory, everything below may, so
  // wait here for that kernel to complete.  Then let the kernel behind this one (the split-K
  // reduction, or the next GEMM) be scheduled early in turn; it waits for this grid the same way.
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) trace_stamp(1);

  bool failed = false;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the schedule (coordinates and addresses stay warp-uniform); one
    // elected lane issues the copies.
    const bool issuer = elect_one();
    const bool hinted = shape.l2_stream_a_keep_b != 0;
    // 1: A tiles evict-first, B tiles evict-last (long raster bands); 2: the other way round (one row
    // tile: every byte of B is read once, by one CTA, while all CTAs share the few rows of A)
    const bool stream_b = shape.l2_stream_a_keep_b == 2;
    const uint64_t pol_a = !hinted ? 0ull : (stream_b ? l2_policy_evict_last() : l2_policy_evict_first());
    const uint64_t pol_b = !hinted ? 0ull : (stream_b ? l2_policy_evict_first() : l2_policy_evict_last());
    auto load_p = [&](uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar, uint64_t pol) {
      if (hinted) {
        if constexpr (CG == 1) tma_load_3d_hint(dst, map, x, y, z, bar, pol);
        else tma_load_3d_pair_hint(dst, map, x, y, z, bar, pol);
      } else {
        if constexpr (CG == 1) tma_load_3d(dst, map, x, y, z, bar);
        else tma_load_3d_pair(dst, map, x, y, z, bar);
      }
    };
    auto load = [&](uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
      load_p(dst, map, x, y, z, bar, pol_b);
    };
    uint32_t it = 0, n = 0;   // n: how many units this cluster has started
    int u = cluster_id;
    while (u >= 0 && u < num_tiles && !failed) {
      int t, split, kb0, kb1, tm, tn, bi, row_base, row_end;
      unit_range(u, t, split, kb0, kb1);
      decode(t, bi, tm, tn, row_base, row_end);
      const int az = grouped ? 0 : bi * shape.a_z, bz = grouped ? bi : bi * shape.b_z;   // a group has its own B, A is one matrix
      const int m0 = row_base + (tm * CG + (int)cta_rank) * kBlockM;
      if constexpr (DYN) {
        if (cta_rank == 0 && issuer) ring.request(n + 1);   // the answer arrives while this unit loads
      }
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1u;
        if (!mbar_wait_warp(empty_bar(s), ph ^ 1u, kRoleProducer, s)) { failed = true; break; }
        const uint32_t a_dst = sA0 + s * Cfg::A_BYTES;
        // Both CTAs of a pair report their bytes to the leader's barrier.
        const uint32_t bar = (CG == 1) ? full_bar(s) : map_to_cta(full_bar(s), 0);
        if (issuer) {
          if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(s), CG * Cfg::STAGE_BYTES);
          if (it == 0) trace_stamp(2);
          if constexpr (A_MN) {
            // A stored transposed ([K, M] row-major): 64-row chunks of 64 k x 128 bytes, like B in that layout
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j) load_p(a_dst + j * 8192, &tmA, m0 + j * 64, kb * kBlockK, az, bar, pol_a);
          } else {
            load_p(a_dst, &tmA, kb * kBlockK, m0, az, bar, pol_a);
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint32_t b_dst = sB0 + (s * NT + nt) * Cfg::B_BYTES;
            const int n0 = (tn * NT + nt) * BN + (int)cta_rank * Cfg::BN_CTA;
            if constexpr (B_MN) {
#pragma unroll
              for (int j = 0; j < Cfg::BN_CTA / 64; ++j) load(b_dst + j * 8192, &tmB, n0 + j * 64, kb * kBlockK, bz, bar);
            } else {
              load(b_dst, &tmB, kb * kBlockK, n0, bz, bar);
            }
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
    // The whole warp runs the loop, so shared-memory addresses and descriptors are warp-uniform;
    // one elected lane issues the tcgen05 instructions.
    if (cta_rank == 0) {
      const bool issuer = elect_one();
      constexpr uint32_t idesc = make_idesc_bf16(kBlockM * CG, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint64_t a_hi = A_MN ? make_smem_desc_hi(8192, 1024, kLayoutSw128)
                                     : make_smem_desc_hi(16, 1024, kLayoutSw128);
      constexpr uint32_t a_kstep = A_MN ? (kUmmaK * 128) : (kUmmaK * 2);
      constexpr uint64_t b_hi = B_MN ? make_smem_desc_hi(8192, 1024, kLayoutSw128)
                                     : make_smem_desc_hi(16, 1024, kLayoutSw128);
      constexpr uint32_t b_kstep = B_MN ? (kUmmaK * 128) : (kUmmaK * 2);
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
      uint32_t it = 0, acc_it = 0;
      int u = cluster_id;
      while (u >= 0 && u < num_tiles && !failed) {
        int t, split, kb0, kb1;
        unit_range(u, t, split, kb0, kb1);
        const uint32_t acc = acc_it % ACC_STAGES, aph = (acc_it / ACC_STAGES) & 1u;
        if (!mbar_wait_warp(tempty_bar(acc), aph ^ 1u, kRoleMma, 100 + (int)acc)) { failed = true; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * NT * BN;   // NT accumulators of 256 columns
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1u;
          if (!mbar_wait_warp(full_bar(s), ph, kRoleMma, s)) { failed = true; break; }
          tc_fence_after_sync();
          if (it == 0 && issuer) trace_stamp(4);
          const uint32_t a_addr = sA0 + s * Cfg::A_BYTES;
          const uint32_t first = kb != kb0 ? 1u : 0u;
          if (issuer) {
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const uint32_t b_addr = sB0 + (s * NT + nt) * Cfg::B_BYTES;
                mma_f16<CG>(d_tmem + nt * BN, smem_desc(a_hi, a_addr + k * a_kstep),
                            smem_desc(b_hi, b_addr + k * b_kstep), idesc, k != 0 ? 1u : first);
              }
            }
            commit(empty_bar(s));   // frees the smem slot in both CTAs once these MMAs have read it
          }
          __syncwarp();
        }
        if (failed) break;
        if (issuer) { trace_stamp(5); commit(tfull_bar(acc)); }   // accumulator complete -> epilogue warps of both CTAs
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
    // ------------------------------------------------------------------ epilogue warps 2..
    const int quad = warp & 3;   // TMEM lanes [32 quad, 32 quad + 32) are the ones this warp may read
    const int nt_w = (warp - 2) >> 2;   // which 256-column accumulator this warp drains (0 when NT = 1)
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    const uint32_t stage0 = sEpi0 + (uint32_t)(warp - 2) * (uint32_t)Cfg::EPI_BUFS * Cfg::EPI_WARP_BUF;
    uint32_t acc_it = 0, store_it = 0;
    int u = cluster_id;
    while (u >= 0 && u < num_tiles && !failed) {
      int t, split, kb0, kb1, tm, tn, bi, row_base, row_end;
      unit_range(u, t, split, kb0, kb1);
      decode(t, bi, tm, tn, row_base, row_end);
      const int m0 = row_base + (tm * CG + (int)cta_rank) * kBlockM + quad * 32;   // first row of this warp
      const int n0 = (tn * NT + nt_w) * BN;
      const uint32_t acc = acc_it % ACC_STAGES, aph = (acc_it / ACC_STAGES) & 1u;
      // every lane waits, and the warp moves on only if every lane saw the phase complete: the
      // TMEM loads below are warp-collective and must not run with part of the warp missing
      const bool ready = mbar_wait(tfull_bar(acc), aph, kRoleEpilogue, 200 + (int)acc);
      if (!__all_sync(0xffffffffu, ready)) { failed = true; break; }
      tc_fence_after_sync();
      if (warp == 2 && lane == 0) trace_stamp(6);
      const uint32_t t_addr = tmem_base + lane_base + (acc * NT + nt_w) * BN;
      bool released = false;   // TMEM already handed back inside the branch below
      const int row = m0 + lane;

      if constexpr (Cfg::EPI == 0) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, v);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          // extent of everything this launch may store to (bounds-checking build)
          const long long c_elems = (long long)(shape.batch - 1) * shape.c_batch_stride + (long long)(shape.k_splits - 1) * shape.split_stride +
                                    (long long)(shape.M - 1) * ldc + shape.N;
          (void)c_elems;
          if (row < row_end) {
            if constexpr (OUT_F32) {
              float* dst = reinterpret_cast<float*>(Cptr) + bi * shape.c_batch_stride + split * shape.split_stride + (int64_t)row * ldc + col;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (col + 4 * j < shape.N && GEMM_B200_IN_BOUNDS(dst + 4 * j, Cptr, c_elems * 4, 16, 10))
                  *reinterpret_cast<uint4*>(dst + 4 * j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            } else {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(Cptr) + bi * shape.c_batch_stride + (int64_t)row * ldc + col;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (col + 8 * j < shape.N && GEMM_B200_IN_BOUNDS(dst + 8 * j, Cptr, c_elems * 2, 16, 11)) {
                  uint32_t p[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]),
                                                             __uint_as_float(v[8 * j + 2 * e + 1]));
                    p[e] = *reinterpret_cast<uint32_t*>(&h);
                  }
                  *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(p[0], p[1], p[2], p[3]);
                }
              }
            }
          }
        }
      } else if constexpr (ACC_STAGES == 1 && !OUT_F32) {
        // Single-buffered accumulator: the MMA issuer is waiting for this TMEM.  Pull all 256
        // columns into registers as packed bf16 first (128 registers), hand TMEM back, and only
        // then stage and store, so the stores overlap the next tile's main loop.
        uint32_t packed[BN / 2];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[2 * e]), __uint_as_float(v[2 * e + 1]));
            packed[c * 16 + e] = *reinterpret_cast<uint32_t*>(&hh);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 1) mbar_arrive(tempty_bar(acc));
          else mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
        }
        released = true;
#pragma unroll
        for (int c = 0; c < BN / 64; ++c, ++store_it) {
          const uint32_t buf = stage0 + (store_it % Cfg::EPI_BUFS) * Cfg::EPI_WARP_BUF;
          if (lane == 0) tma_store_wait_read<Cfg::EPI_BUFS - 1>();
          __syncwarp();
          const uint32_t row_addr = buf + (uint32_t)lane * 128u;
          const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)j ^ sw) << 4)),
                         "r"(packed[c * 32 + 4 * j]), "r"(packed[c * 32 + 4 * j + 1]), "r"(packed[c * 32 + 4 * j + 2]),
                         "r"(packed[c * 32 + 4 * j + 3]) : "memory");
          fence_proxy_async_smem();
          __syncwarp();
          const int x = n0 + c * 64;
          if (lane == 0) {
            if (m0 < shape.M && x < shape.N) tma_store_3d(&tmC, x, m0, shape.k_splits > 1 ? split : bi, buf);   // split-K: slice `split` of the scratch
            tma_store_commit();
          }
        }
      } else {
        // 128-byte-wide column slabs: 64 bf16 or 32 f32 columns per TMA store of 32 rows.
        constexpr int SLAB_COLS = OUT_F32 ? 32 : 64;
#pragma unroll 1
        for (int c = 0; c < BN / SLAB_COLS; ++c, ++store_it) {
          const uint32_t buf = stage0 + (store_it % Cfg::EPI_BUFS) * Cfg::EPI_WARP_BUF;
          // the store that last read this buffer was committed EPI_BUFS slabs ago
          if (lane == 0) tma_store_wait_read<Cfg::EPI_BUFS - 1>();
          __syncwarp();
          const uint32_t row_addr = buf + (uint32_t)lane * 128u;
          const uint32_t sw = (uint32_t)(lane & 7);
          if constexpr (OUT_F32) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_addr + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)j ^ sw) << 4)),
                           "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3]) : "memory");
          } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t v[32];
              tmem_ld_32x32b_x32(t_addr + c * 64 + h * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]),
                                                            __uint_as_float(v[8 * j + 2 * e + 1]));
                  p[e] = *reinterpret_cast<uint32_t*>(&hh);
                }
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                             ::"r"(row_addr + (((uint32_t)(h * 4 + j) ^ sw) << 4)), "r"(p[0]), "r"(p[1]), "r"(p[2]), "r"(p[3])
                             : "memory");
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          const int x = n0 + c * SLAB_COLS;
          if (lane == 0) {
            if (m0 < shape.M && x < shape.N) tma_store_3d(&tmC, x, m0, shape.k_splits > 1 ? split : bi, buf);   // split-K: slice `split` of the scratch
            tma_store_commit();
          }
        }
      }
      // accumulator fully read: hand the TMEM buffer back to the MMA issuer (leader CTA)
      if (!released) {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CG == 1) mbar_arrive(tempty_bar(acc));
          else mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
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
    // give copies and MMAs still in flight time to land before shared memory and TMEM go away
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

}  // namespace tc
}  // namespace gemm_b200
