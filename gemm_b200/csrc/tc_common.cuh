// PTX building blocks for the sm_100a tensor-core kernels: mbarriers with BOUNDED waits,
// TMA tile loads/stores (never with cluster multicast), tcgen05 TMEM allocation, MMA issue,
// commit and TMEM loads, and the shared-memory / instruction descriptor encoders.
//
// Every wait in this file gives up after kWaitLimitNs, records where in a status word in
// global memory and lets the kernel run to its normal exit (barriers, TMEM free), so a
// logic error shows up as GEMM_B200_ERR_TIMEOUT on the host instead of a hung GPU.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

namespace gemm_b200 {
namespace tc {

// ---------------------------------------------------------------------------------------
// device status word: {code, block, role, stage}.  code != 0 means "some wait gave up";
// all later waits in every CTA return at once when they see it.
// ---------------------------------------------------------------------------------------
__device__ int32_t g_status[4];

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

enum Role : int { kRoleProducer = 1, kRoleMma = 2, kRoleEpilogue = 3, kRoleSetup = 4 };

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool aborted() {
  return *reinterpret_cast<volatile int32_t*>(&g_status[0]) != 0;
}

__device__ __noinline__ void record_timeout(int role, int stage) {
  if (atomicCAS(&g_status[0], 0, GEMM_B200_ERR_TIMEOUT) == 0) {
    g_status[1] = (int32_t)blockIdx.x;
    g_status[2] = role;
    g_status[3] = stage;
    __threadfence();
  }
}

// Opt-in stage timeline (-DGEMM_B200_TRACE builds only, `python -m gemm_b200.build --trace`): each
// of the first kTraceBlocks CTAs stamps the global nanosecond timer at fixed points of a
// tensor-core kernel; gemm_b200_trace_read() copies the table out.  Compiles to nothing otherwise.
// Slots: 0 kernel entry, 1 set-up done (barriers, TMEM, cluster sync), 2 first TMA issued, 3 last
// load of the CTA issued, 4 first operand stage arrived, 5 last MMA issued, 6 epilogue sees the
// accumulator, 7 stores issued (cluster split: partial sums sent), 8 stores complete (cluster
// split: all pieces landed), 9 before the teardown barrier, 10 TMEM freed.
#ifdef GEMM_B200_TRACE
constexpr int kTraceBlocks = 160, kTraceSlots = 16;
__device__ unsigned long long g_trace[kTraceBlocks][kTraceSlots];
__device__ __forceinline__ void trace_stamp(int slot) {
  if (blockIdx.x < kTraceBlocks) g_trace[blockIdx.x][slot] = globaltimer_ns();
}
#else
__device__ __forceinline__ void trace_stamp(int) {}
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------------------
// cluster helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive on a barrier that may live in another CTA of the cluster (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after recording the place) when the limit ran out or when
// another wait anywhere on the device has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int role, int stage,
                                          unsigned long long limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (aborted()) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        record_timeout(role, stage);
        return false;
      }
    }
  }
}

// Wait on a barrier that a thread of ANOTHER CTA of the cluster arrives on (acquire at cluster
// scope, so that CTA's shared::cluster stores before its arrive are visible afterwards).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, int role, int stage,
                                                  unsigned long long limit_ns = kWaitLimitNs) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (aborted()) return false;
      if (globaltimer_ns() - t0 > limit_ns) {
        record_timeout(role, stage);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_shared_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------
// Cluster launch control: a running cluster takes over the work of a cluster of the same grid
// that has not started yet.  try_cancel asks the hardware to cancel the launch of one pending
// cluster; the 16-byte answer lands in this CTA's shared memory and completes 16 bytes on `bar`.
// clc_first_cta returns blockIdx.x of the first CTA of the cancelled cluster, or -1 when no
// cluster was left to cancel (after which the CTA must not ask again).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void clc_try_cancel(uint32_t resp_smem, uint32_t bar) {
  asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
               ::"r"(resp_smem), "r"(bar) : "memory");
}
__device__ __forceinline__ int clc_first_cta(uint32_t resp_smem) {
  uint32_t ok, x;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b128 h;\n"
      "ld.shared.b128 h, [%2];\n"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, h;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "mov.u32 %1, 0;\n"
      "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, h;\n"
      "}\n"
      : "=r"(ok), "=r"(x)
      : "r"(resp_smem)
      : "memory");
  return ok ? (int)x : -1;
}

// Programmatic dependent launch: a kernel launched behind this one with the programmatic-
// serialization attribute may be scheduled once every CTA here has called pdl_launch_dependents()
// (or exited); it must call pdl_wait() before touching anything this grid wrote, which returns
// when this grid has completed and its writes are visible.  Both are no-ops otherwise.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Whole-warp form: every lane waits, and the warp goes on only if every lane saw the phase
// complete.  Keeps the producer and MMA-issuing warps convergent, so the values they compute
// (addresses, descriptors, coordinates) are warp-uniform and only the issuing instruction itself
// sits under the elected lane's predicate.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int role, int stage) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, role, stage));
}
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), 2-D tiles.  Loads complete on an mbarrier by byte count.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// destination and barrier in this CTA
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// the same load with an L2 eviction-priority policy (l2_policy_evict_first / _last)
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}
// destination in this CTA, barrier possibly in the peer CTA of a CTA pair (shared::cluster address)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
               : "memory");
}
// 3-D forms (x, y, z): z selects the matrix of a batch; the box is one matrix deep.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// The same loads with an L2 eviction-priority policy (l2_policy_evict_first / _last).
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair_hint(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                                      uint32_t cluster_bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int x, int y, int z, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05: TMEM allocation, fences, MMA, commit, TMEM load
// ---------------------------------------------------------------------------------------
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CG == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], BF16/F16 inputs, issued by ONE thread.
template <int CG>
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  if constexpr (CG == 1)
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= (A * SFA) * (B * SFB): e4m3/e5m2 data, one UE8M0 scale per 32 k, scales in TMEM.
template <int CG>
__device__ __forceinline__ void mma_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  if constexpr (CG == 1)
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %6, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%4], [%5], p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}

// smem -> TMEM copy of 32 rows x 16 bytes, replicated to the four 32-lane quarters (scale factors)
template <int CG>
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
  else
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// Make `bar` (this CTA) complete one arrival when all tcgen05 ops issued so far by this thread finish.
__device__ __forceinline__ void mma_commit_local(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// CTA-pair form: signals the barrier at shared::cluster address `cluster_bar` (either CTA of the pair).
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// CTA-pair form that signals the barrier at the same offset in every CTA of `cta_mask`.
__device__ __forceinline__ void mma_commit_pair_mask(uint32_t bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(cta_mask) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread i = TMEM lane base+i)
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1 (sm_100)
//   [61,64) layout: 0 none, 2 = 128-byte swizzle, 4 = 64-byte, 6 = 32-byte
// K-major operand, 128B swizzle (rows of 128 bytes, 8-row groups of 1024 bytes):
//   SBO = distance between 8-row groups; LBO unused.
// MN-major operand, 128B swizzle (k rows of 128 bytes = 64 bf16 along M/N):
//   LBO = distance between 64-element blocks along M/N; SBO = distance between 8-k-row groups.
__host__ __device__ constexpr uint64_t make_smem_desc_hi(uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return ((uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)layout << 61);
}
__device__ __forceinline__ uint64_t smem_desc(uint64_t hi_part, uint32_t smem_addr) {
  return hi_part | (uint64_t)((smem_addr >> 4) & 0x3fff);
}
constexpr uint32_t kLayoutNone = 0, kLayoutSw128 = 2;

// Instruction descriptor, kind::f16 (32 bit):
//   [4,6) D format (1 = F32)   [7,10) A format (1 = BF16)   [10,13) B format
//   [15] A major (0 = K, 1 = MN)   [16] B major   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Instruction descriptor, kind::mxf8f6f4 block-scaled (32 bit):
//   [4,6) B scale id   [7,10) A format (0 = E4M3)   [10,13) B format   [15] A major   [16] B major
//   [17,23) N >> 3   [23] scale format (1 = UE8M0)   [24,29) M >> 4   [29,31) A scale id
__host__ __device__ constexpr uint32_t make_idesc_mxf8(int m, int n, int a_sf_id, int b_sf_id) {
  return ((uint32_t)b_sf_id << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) |
         ((uint32_t)(m >> 4) << 24) | ((uint32_t)a_sf_id << 29);
}

}  // namespace tc
}  // namespace gemm_b200
