// Host side of the tensor-core entry points: argument checks, TMA descriptors, persistent
// grid sizing and launches.  Compiled for sm_100a only (tcgen05 needs the arch-specific target).
#include <map>
#include <mutex>
#include <stdlib.h>
#include <utility>

#include "gemm_bf16.cuh"
#include "gemm_bf16_ksplit.cuh"
#include "gemm_mxfp8.cuh"
#include "gemm_mxfp8_ksplit.cuh"

namespace gemm_b200 {
namespace tc {

// cuTensorMapEncodeTiled is fetched through the runtime so the library does not link libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Encoding a tensor map costs a microsecond or two on the host, and a GEMM call needs three to
// five of them: for small problems that is a visible share of the call.  A descriptor depends only
// on (address, shape, pitch, box, type, swizzle), so recently used ones are kept per thread.
struct MapKey {
  const void* ptr;
  int64_t rows, cols, ld, batch, batch_stride;   // batch == 0: a 2-D map
  int box_cols, box_rows, dtype, swizzle;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && batch == o.batch &&
           batch_stride == o.batch_stride && box_cols == o.box_cols && box_rows == o.box_rows && dtype == o.dtype &&
           swizzle == o.swizzle;
  }
};
struct MapCache {
  static constexpr int kEntries = 32;
  MapKey keys[kEntries];
  CUtensorMap maps[kEntries];
  int used = 0, next = 0;
  const CUtensorMap* find(const MapKey& k) const {
    for (int i = 0; i < used; ++i)
      if (keys[i] == k) return &maps[i];
    return nullptr;
  }
  void insert(const MapKey& k, const CUtensorMap& m) {
    const int slot = used < kEntries ? used++ : (next++ % kEntries);
    keys[slot] = k;
    maps[slot] = m;
  }
};
static MapCache& map_cache() {
  static thread_local MapCache c;
  return c;
}

// 2-D row-major tensor [rows, cols] with `ld` elements between rows; box = box_cols x box_rows.
static int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* ptr, int64_t rows,
                       int64_t cols, int64_t ld, int box_cols, int box_rows, CUtensorMapSwizzle swz) {
  const MapKey key{ptr, rows, cols, ld, 0, 0, box_cols, box_rows, (int)dt, (int)swz};
  if (const CUtensorMap* hit = map_cache().find(key)) {
    *map = *hit;
    return GEMM_B200_OK;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(GEMM_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (cuuint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GEMM_B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld ld=%lld box=%dx%d)",
                (int)r, (long long)rows, (long long)cols, (long long)ld, box_cols, box_rows);
  map_cache().insert(key, *map);
  return GEMM_B200_OK;
}

// `batch` row-major matrices [rows, cols] (pitch ld), `batch_stride` elements apart, as one 3-D
// tensor (cols, rows, matrix); a box is one matrix deep.
static int make_map_3d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* ptr, int64_t rows,
                       int64_t cols, int64_t ld, int64_t batch, int64_t batch_stride, int box_cols, int box_rows,
                       CUtensorMapSwizzle swz) {
  const MapKey key{ptr, rows, cols, ld, batch, batch_stride, box_cols, box_rows, (int)dt, (int)swz};
  if (const CUtensorMap* hit = map_cache().find(key)) {
    *map = *hit;
    return GEMM_B200_OK;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(GEMM_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * (cuuint64_t)elem_bytes, (cuuint64_t)batch_stride * (cuuint64_t)elem_bytes};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(GEMM_B200_ERR_CUDA,
                "cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld ld=%lld batch=%lld stride=%lld box=%dx%d)",
                (int)r, (long long)rows, (long long)cols, (long long)ld, (long long)batch, (long long)batch_stride,
                box_cols, box_rows);
  map_cache().insert(key, *map);
  return GEMM_B200_OK;
}

// Band width of the tile raster: bands of column tiles, walked column-fastest (on B200 1-5 %
// faster and 10-20 % less DRAM traffic than bands of row tiles).  The band's B panel
// (`col_tile_bytes` per column tile) is sized near 32 MB so that it survives in the L2 from one
// round of units to the next, but a band is never narrower than `min_cols` columns of C.
// Measured with units handed out at run time, BF16, TFLOP/s in a loop:
//   131072 x 8192 x 8192, 512-wide tiles: bands of 4 / 6 / 8 / 16 tiles 1420 / 1414 / 1386 / 1277
//   (DRAM 13.6 / - / 14.7 / - GB per launch); 32768 x 4096 x 4096: 4 / 8 / 16 tiles 1576 / 1591 /
//   1611; 256-wide tiles, K = 8192: 2 / 4 / 8 tiles 1431 / 1511 / 1544.
// MXFP8 16384 x 8192 x 28672 (256-wide tiles): bands of 14-16 tiles 2940-2957, of 8: 2917, of 28: 2807.
// GEMM_B200_RASTER_GROUP overrides it (tuning knob): n > 0 = bands of n row tiles, n < 0 = bands
// of -n column tiles.
static int raster_group_for(int64_t col_tile_bytes, int tile_cols, int min_cols) {
  static const int forced = [] {
    const char* e = getenv("GEMM_B200_RASTER_GROUP");
    return e ? atoi(e) : 0;
  }();
  if (forced != 0) return forced;
  int64_t g = (32ll << 20) / (col_tile_bytes > 0 ? col_tile_bytes : 1);
  const int64_t g_min = (min_cols + tile_cols - 1) / tile_cols;
  if (g < g_min) g = g_min;
  if (g < 4) g = 4;
  if (g > 32) g = 32;
  return -(int)g;
}

struct DeviceInfo {
  int dev = -1, sms = 0, cc_major = 0;
};
static int device_info(DeviceInfo* out) {
  static thread_local DeviceInfo cached;
  int dev = 0;
  GEMM_B200_CUDA_TRY(cudaGetDevice(&dev));
  if (cached.dev != dev) {
    GEMM_B200_CUDA_TRY(cudaDeviceGetAttribute(&cached.sms, cudaDevAttrMultiProcessorCount, dev));
    GEMM_B200_CUDA_TRY(cudaDeviceGetAttribute(&cached.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    cached.dev = dev;
  }
  *out = cached;
  return GEMM_B200_OK;
}


// Number of CTA clusters of `kern` that can be resident at once on the current device (the size
// of the persistent grid), looked up once per device and kernel.  Also opts the kernel in to its
// dynamic shared memory size.
template <class Kern>
static int persistent_clusters(Kern kern, int cg, int threads, int smem_bytes, const DeviceInfo& di, int* out) {
  // keyed by (device, kernel): kernels of one signature share this function's instantiation
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> cache;
  std::lock_guard<std::mutex> lk(mu);
  const std::pair<int, const void*> key(di.dev, reinterpret_cast<const void*>(kern));
  auto hit = cache.find(key);
  if (hit == cache.end()) {
    GEMM_B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    int n = di.sms / cg;
    if (cg > 1) {
      cudaLaunchConfig_t qc = {};
      qc.gridDim = dim3((unsigned)(di.sms / cg * cg));
      qc.blockDim = dim3((unsigned)threads);
      qc.dynamicSmemBytes = (size_t)smem_bytes;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = (unsigned)cg;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      qc.attrs = qa;
      qc.numAttrs = 1;
      int active = 0;
      GEMM_B200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&active, kern, &qc));
      if (active < 1) return fail(GEMM_B200_ERR_CUDA, "no CTA pair of this kernel fits on the device");
      if (active < n) n = active;
    }
    hit = cache.emplace(key, n).first;
  }
  *out = hit->second;
  return GEMM_B200_OK;
}

// Launches `kern` on `clusters` clusters of `cg` CTAs.
template <class Kern, class... Args>
static int launch_clusters(Kern kern, int clusters, int cg, int threads, int smem_bytes, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(clusters * cg));
  cfg.blockDim = dim3((unsigned)threads);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = (unsigned)cg;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  // Programmatic dependent launch: behind another kernel of this library (which signals
  // griddepcontrol.launch_dependents once it is set up) the launch is processed and the CTAs set
  // themselves up while that kernel still runs; every kernel here waits (griddepcontrol.wait)
  // before it touches global memory.  Behind any other kernel the launch waits for it to finish
  // as usual.  A train of ten BF16 GEMMs replayed from a CUDA graph, us per call without / with:
  // 1024^3 8.2 / 7.2, 1024 x 2048 x 1024 11.1 / 10.0, 128 x 4096 x 4096 12.3 / 11.7, 2048^3 17.0 / 16.0;
  // the same train issued call by call: 128 x 4096 x 4096 14.8 / 12.5, 2048^3 18.7 / 16.5.
  // GEMM_B200_PDL=0 launches without it.
  static const bool pdl = env_int("GEMM_B200_PDL", 1) != 0;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = pdl ? 2 : 1;
  GEMM_B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, args...));
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  return GEMM_B200_OK;
}

// Number of K splits for a problem whose tiles alone do not fill the GPU: the split count that
// wastes the fewest CTA slots in the last round, mildly preferring fewer splits (each split
// writes and re-reads an M x N FP32 slice).  1 = do not split.
static int auto_splits_units(int64_t tiles, int64_t num_kb, int sms) {
  // Splitting pays for a second (reduce) launch and an M x N FP32 round trip per split: measured on
  // B200, 112 tiles on 148 SMs run as fast unsplit (16 x 8192 x 28672: 62 us either way; 64 rows:
  // 62 us unsplit, 70 us split), 32 tiles do not (128 x 8192 x 8192: 42 -> 34 us; 16 x 16384 x 4096
  // with 16 tiles: 64 -> 28 us).  Split only when the tiles leave more than a third of the SMs idle.
  if (3 * tiles >= 2 * (int64_t)sms || num_kb < 8) return 1;
  int best = 1;
  double best_score = (double)tiles / (double)(ceil_div64(tiles, sms) * sms);
  for (int s = 2; s <= 16 && num_kb / s >= 4; ++s) {
    const int64_t kb_per = ceil_div64(num_kb, s);
    if (ceil_div64(num_kb, kb_per) != s) continue;
    const int64_t units = tiles * s;
    const double score = (double)units / (double)(ceil_div64(units, sms) * sms) - 0.01 * s;
    if (score > best_score + 1e-9) { best_score = score; best = s; }
  }
  return best;
}

// K ranges for an MXFP8 problem of more than one row tile, by the estimate bf16_auto_splits uses (the
// operand bytes per K block are the same: 128 one-byte elements instead of 64 two-byte ones); the
// partial sums come from single-CTA 128 x 256 tiles.  1 = do not split.
static int mxfp8_model_splits(int64_t M, int64_t N, int64_t K, int sms) {
  const int64_t tiles = ceil_div64(M, kBlockM) * ceil_div64(N, kBlockN), slots = sms;
  const int64_t num_kb = ceil_div64(K, kMxBlockK);
  if (3 * tiles >= 2 * slots || num_kb < 32) return 1;
  const int64_t pair_slots = sms / 2 > 0 ? sms / 2 : 1;
  const int64_t units256 = ceil_div64(M, 2 * kBlockM) * ceil_div64(N, kBlockN), units128 = ceil_div64(M, 2 * kBlockM) * ceil_div64(N, 128);
  double best_cost = (double)ceil_div64(units256, pair_slots) * (double)num_kb * 0.30;
  const double c128 = (double)ceil_div64(units128, pair_slots) * (double)num_kb * 0.195;
  if (c128 < best_cost) best_cost = c128;
  const double slice_us = (double)M * (double)N * 8.0 / 7.8e6;
  int best = 1;
  for (int s = 2; s <= 32; ++s) {
    const int64_t kb_per = ceil_div64(num_kb, s);
    if (kb_per < 8) break;
    if ((double)s * (double)M * (double)N * 4.0 > 268435456.0) break;   // scratch of at most 256 MiB
    if (ceil_div64(num_kb, kb_per) != s) continue;
    const double cost = (double)ceil_div64(tiles * s, slots) * (double)kb_per * 0.39 + s * slice_us + 6.0;
    if (cost < best_cost) { best_cost = cost; best = s; }
  }
  return best;
}

static int auto_splits(int64_t M, int64_t N, int64_t K, int sms) {
  // counted in K units of 256: no split below K = 2048, at least 1024 of K per split (1024^3 with
  // 32 tiles: 13.2 us unsplit, 19.4 us cut in two)
  return auto_splits_units(ceil_div64(M, kBlockM) * ceil_div64(N, kBlockN), ceil_div64(K, 2 * kMxBlockK), sms);
}

// Library-owned scratch of the automatic split-K path: one buffer per (device, stream), grown on
// demand.  Work on one stream is ordered, so calls that share a buffer never overlap; calls on
// different streams get different buffers and may run side by side.  At most kScratchSlots
// streams per process keep a buffer; beyond that the least recently used one is released
// (cudaFree waits for the device, so nothing still reads it).
struct ScratchSlot {
  int dev = -1;
  cudaStream_t stream = nullptr;
  void* ptr = nullptr;
  size_t bytes = 0;
  uint64_t last_use = 0;
};
constexpr int kScratchSlots = 32;
static std::mutex g_scratch_mu;
static ScratchSlot g_scratch[kScratchSlots];
static uint64_t g_scratch_clock = 0;
// *out stays null (and the call succeeds) when a buffer would have to be allocated or grown while
// `stream` is being captured into a graph: allocation is not allowed there, and the caller runs
// unsplit.
static int cached_scratch(int dev, size_t bytes, float** out, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  *out = nullptr;
  ScratchSlot* slot = nullptr;      // this stream's buffer, if it has one
  ScratchSlot* victim = nullptr;    // else: a free slot, or the least recently used one
  for (ScratchSlot& c : g_scratch) {
    if (c.ptr && c.dev == dev && c.stream == stream) { slot = &c; break; }
    if (!victim || (victim->ptr && (!c.ptr || c.last_use < victim->last_use))) victim = &c;
  }
  if (!slot || slot->bytes < bytes) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    GEMM_B200_CUDA_TRY(cudaStreamIsCapturing(stream, &cs));
    if (cs != cudaStreamCaptureStatusNone) return GEMM_B200_OK;
    if (!slot) slot = victim;
    if (slot->ptr) {
      int cur = dev;
      if (slot->dev != dev) GEMM_B200_CUDA_TRY(cudaSetDevice(slot->dev));
      cudaError_t e = cudaFree(slot->ptr);
      if (slot->dev != dev) GEMM_B200_CUDA_TRY(cudaSetDevice(cur));
      GEMM_B200_CUDA_TRY(e);
    }
    *slot = ScratchSlot();
    GEMM_B200_CUDA_TRY(cudaMalloc(&slot->ptr, bytes));
    slot->dev = dev;
    slot->stream = stream;
    slot->bytes = bytes;
  }
  slot->last_use = ++g_scratch_clock;
  *out = static_cast<float*>(slot->ptr);
  return GEMM_B200_OK;
}

// The split-K reduce pass, launched with programmatic stream serialization so that its launch
// overlaps the tail of the GEMM that feeds it (the kernel itself waits for that grid).
static int launch_splitk_reduce(const float* scratch, int64_t M, int64_t N, int splits, void* C, int64_t ldc, int out_dtype,
                                cudaStream_t stream) {
  const int64_t threads = M * (N / 4);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ceil_div64(threads, 256));
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  const int64_t split_stride = M * N;
  if (out_dtype == GEMM_B200_OUT_F32)
    GEMM_B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<true>, scratch, split_stride, N, splits, C, ldc, (int)M, (int)N));
  else
    GEMM_B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, splitk_reduce_kernel<false>, scratch, split_stride, N, splits, C, ldc, (int)M, (int)N));
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  return GEMM_B200_OK;
}

struct Bf16Args {
  const void *A, *B;
  void* C;
  int64_t M, N, K, lda, ldb, ldc;
  cudaStream_t stream;
  // batched call: `batch` problems; a stride of 0 on A or B shares that operand between them
  int64_t batch = 1, stride_a = 0, stride_b = 0, stride_c = 0;
  // split-K (FP32 output only): C is then the scratch [k_splits][M][N], ldc = N
  int k_splits = 1;
};

// One instantiation per (config, B layout, output type); A_MN: A is stored transposed, [K, M] row-major.
template <class Cfg, bool B_MN, bool OUT_F32, bool A_MN = false>
static int launch_bf16(const Bf16Args& a) {
  constexpr int CG = Cfg::CG;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  CUtensorMap tmA, tmB, tmC;
  // a shared operand (stride 0) is mapped as one matrix; the kernel then always asks for matrix 0
  const int64_t za = a.stride_a ? a.batch : 1, zb = a.stride_b ? a.batch : 1;
  const int64_t sa = a.stride_a ? a.stride_a : (A_MN ? a.K : a.M) * a.lda;
  const int64_t sb = a.stride_b ? a.stride_b : (B_MN ? a.K : a.N) * a.ldb;
  const int64_t sc = a.batch > 1 ? a.stride_c : a.M * a.ldc;
  if (A_MN) {
    if (int rc = make_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.A, a.K, a.M, a.lda, za, sa, 64, kBlockK,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    if (int rc = make_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.A, a.M, a.K, a.lda, za, sa, kBlockK, kBlockM,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  if (B_MN) {
    if (int rc = make_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.B, a.K, a.N, a.ldb, zb, sb, 64, kBlockK,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    if (int rc = make_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.B, a.N, a.K, a.ldb, zb, sb, kBlockK, Cfg::BN_CTA,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  if (Cfg::EPI == 1) {
    // third dimension: the problems of a batch, or the K ranges of a split run (slices of the scratch)
    if (int rc = make_map_3d(&tmC, OUT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                             OUT_F32 ? 4 : 2, a.C, a.M, a.N, a.ldc, a.k_splits > 1 ? a.k_splits : a.batch, sc, OUT_F32 ? 32 : 64, 32,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    tmC = tmA;   // unused by the kernel
  }

  auto kern = gemm_bf16_kernel<Cfg, B_MN, OUT_F32, A_MN>;
  int max_clusters = 0;
  if (int rc = persistent_clusters(kern, CG, Cfg::THREADS, Cfg::SMEM_BYTES, di, &max_clusters)) return rc;

  GemmShape shape;
  shape.M = (int)a.M;
  shape.N = (int)a.N;
  shape.K = (int)a.K;
  shape.tiles_m = (int)ceil_div64(a.M, kBlockM * CG);
  shape.tiles_n = (int)ceil_div64(a.N, Cfg::TILE_N);
  const int num_kb = (int)ceil_div64(a.K, kBlockK);
  if (a.k_splits > 1 && !(OUT_F32 && a.batch == 1))
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: K splits need FP32 output and one problem");
  shape.kb_per_split = (int)ceil_div64(num_kb, a.k_splits);
  shape.k_splits = (int)ceil_div64(num_kb, shape.kb_per_split);   // no empty split
  shape.split_stride = a.M * a.ldc;
  shape.raster_group = raster_group_for((int64_t)Cfg::TILE_N * a.K * 2, Cfg::TILE_N, 2048);
  shape.batch = (int)a.batch;
  shape.a_z = a.stride_a ? 1 : 0;
  shape.b_z = a.stride_b ? 1 : 0;
  shape.c_batch_stride = a.batch > 1 ? a.stride_c : 0;
  // L2 priorities (A evict-first, B evict-last) when a raster band lasts at least three rounds of
  // units.  Run-time hand-out only: on the static schedule clusters drift apart and an
  // evict-first A tile is gone before the last of them asks for it.  Measured (TFLOP/s in a
  // loop, without / with): 131072 x 8192 x 8192 (28 rounds per band) 1420 / 1428 with DRAM
  // 14.8 -> 13.6 GB per launch; 32768 x 4096 x 4096 (14) 1591 / 1610; 16384 x 8192 x 8192 (3.5)
  // 1609 / 1617; 8192^3 (1.7) 1600 / 1603; 8192 x 16384 x 4096 (1.7) 1521 / 1498.
  {
    const int64_t band = shape.raster_group < 0 ? (-shape.raster_group < shape.tiles_n ? -shape.raster_group : shape.tiles_n) : 0;
    shape.l2_stream_a_keep_b = (Cfg::DYN && a.batch == 1 && band > 0 && (int64_t)shape.tiles_m * band >= 3 * (int64_t)max_clusters) ? 1 : 0;
    // one row tile of a single-CTA variant: B is read exactly once; keep the stream from pushing other
    // data (or dirty lines that would have to be written back meanwhile) out of the L2.  Per call after a
    // 252 MB write flush, without / with: 16 x 8192 x 28672 90.2 / 78.8 us (cuBLAS 86.8), 128 x 8192 x 28672
    // 90.9 / 80.7 (95.3), 16 x 8192 x 8192 39.9 / 35.8 (33.7); after a read flush the same either way.
    static const bool stream_ok = env_int("GEMM_B200_BF16_STREAM_B", 1) != 0;
    if (stream_ok && CG == 1 && shape.tiles_m == 1 && a.batch == 1) shape.l2_stream_a_keep_b = 2;
  }
  const int64_t num_tiles = (int64_t)shape.tiles_m * shape.tiles_n * a.batch * shape.k_splits;
  if (num_tiles > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_bf16: too many tiles");
  // static schedule: one cluster per resident slot, each walks unit = cluster + i * clusters;
  // run-time hand-out: one cluster per unit, the ones that run adopt the units of the others
  const int clusters = Cfg::DYN ? (int)num_tiles : (int)(num_tiles < max_clusters ? num_tiles : max_clusters);
  if (Cfg::DYN && shape.k_splits > 1)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: K splits run on the static schedule");

  static const GroupTable no_groups = {};   // count == 0
  return launch_clusters(kern, clusters, CG, Cfg::THREADS, Cfg::SMEM_BYTES, a.stream, tmA, tmB, tmC, a.C, a.ldc, shape, no_groups);
}

// Grouped (ragged) BF16 GEMM, at most kMaxGroups groups per launch: single-CTA 128 x 256 tiles with
// the direct-store epilogue, whose row guard stops at the end of the group (a TMA store would
// write the first rows of the next group).  Units are handed out statically.
template <bool B_MN, bool OUT_F32>
static int launch_bf16_grouped(const void* A, const void* B, void* C, int groups, const int64_t* m_sizes, int64_t N, int64_t K,
                               int64_t lda, int64_t ldb, int64_t stride_b, int64_t ldc, cudaStream_t stream) {
  using Cfg = Bf16Cfg<1, 4, 0, false>;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  GroupTable table;
  table.count = groups;
  int64_t rows = 0, tiles = 0;
  const int tiles_n = (int)ceil_div64(N, Cfg::TILE_N);
  for (int g = 0; g < groups; ++g) {
    table.tile_start[g] = (int)tiles;
    table.row_start[g] = (int)rows;
    rows += m_sizes[g];
    tiles += ceil_div64(m_sizes[g], kBlockM) * tiles_n;
    if (rows > 0x7fffffff || tiles > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_bf16_grouped: too many rows or tiles");
  }
  for (int g = groups; g <= kMaxGroups; ++g) {
    table.tile_start[g] = (int)tiles;
    table.row_start[g] = (int)rows;
  }
  if (tiles == 0) return GEMM_B200_OK;
  CUtensorMap tmA, tmB;
  if (int rc = make_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, rows, K, lda, 1, rows * lda, kBlockK, kBlockM,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (B_MN) {
    if (int rc = make_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, K, N, ldb, groups, stride_b, 64, kBlockK,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    if (int rc = make_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, N, K, ldb, groups, stride_b, kBlockK, Cfg::BN_CTA,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  auto kern = gemm_bf16_kernel<Cfg, B_MN, OUT_F32>;
  int max_clusters = 0;
  if (int rc = persistent_clusters(kern, 1, Cfg::THREADS, Cfg::SMEM_BYTES, di, &max_clusters)) return rc;
  GemmShape shape;
  shape.M = (int)rows;
  shape.N = (int)N;
  shape.K = (int)K;
  shape.tiles_m = 0;                  // unused: the table says where every group's tiles start
  shape.tiles_n = tiles_n;
  shape.k_splits = 1;
  shape.kb_per_split = (int)ceil_div64(K, kBlockK);
  shape.split_stride = 0;
  shape.raster_group = 1;
  shape.batch = 1;
  shape.a_z = shape.b_z = 0;
  shape.c_batch_stride = 0;
  shape.l2_stream_a_keep_b = 0;
  const int clusters = (int)(tiles < max_clusters ? tiles : max_clusters);
  return launch_clusters(kern, clusters, 1, Cfg::THREADS, Cfg::SMEM_BYTES, stream, tmA, tmB, tmA, C, ldc, shape, table);
}

struct Bf16ConfigEntry {
  const char* name;
  int (*launch[2][2])(const Bf16Args&);   // [b_layout][out_dtype]
};

#define GEMM_B200_BF16_ENTRY(NAME, CFG)                                                          \
  {                                                                                              \
    NAME, {                                                                                      \
      {launch_bf16<CFG, true, false>, launch_bf16<CFG, true, true>},                             \
      {launch_bf16<CFG, false, false>, launch_bf16<CFG, false, true>}                            \
    }                                                                                            \
  }

//                          CG ST EPI MASK
using Bf16_1cta_direct = Bf16Cfg<1, 4, 0, false>;
using Bf16_1cta_tma    = Bf16Cfg<1, 4, 1, false>;
using Bf16_2cta_tma_m  = Bf16Cfg<2, 6, 1, true>;
using Bf16_2cta_n512_s3 = Bf16Cfg<2, 3, 1, true, 2, 2>;
using Bf16_2cta_n128    = Bf16Cfg<2, 7, 1, true, 1, 2, 128>;
using Bf16_1cta_n128    = Bf16Cfg<1, 6, 1, false, 1, 2, 128>;
// the two multi-round shapes with units handed out at run time
using Bf16_2cta_tma_m_dyn   = Bf16Cfg<2, 6, 1, true, 1, 2, kBlockN, true>;
using Bf16_2cta_n512_s3_dyn = Bf16Cfg<2, 3, 1, true, 2, 2, kBlockN, true>;
#ifdef GEMM_B200_TUNING
// variants the heuristics never pick; built only for tuning sweeps
using Bf16_2cta_direct = Bf16Cfg<2, 6, 0, false>;
using Bf16_2cta_tma    = Bf16Cfg<2, 6, 1, false>;
using Bf16_2cta_n512    = Bf16Cfg<2, 4, 1, true, 2>;
using Bf16_2cta_n512_d  = Bf16Cfg<2, 4, 0, true, 2>;
#endif

// index of every variant in kBf16Configs (the order of the table below)
enum Bf16ConfigId : int {
  kBf16Cfg1ctaDirect = 0,   // single CTA, 128x256 tiles, direct stores: the split-K partial sums
  kBf16Cfg1cta,             // single CTA, 128x256 tiles, TMA store
  kBf16Cfg256,              // CTA pair, 256x256 tiles, double-buffered accumulator
  kBf16Cfg512,              // CTA pair, 256x512 tiles (A shared by two accumulators)
  kBf16Cfg2ctaN128,         // CTA pair, 256x128 tiles: at most half a round of 256-wide tiles
  kBf16Cfg1ctaN128,         // single CTA, 128x128 tiles: one row tile and few column tiles
  kBf16Cfg256Dyn,           // 256x256 tiles, units handed out at run time (problems of several rounds)
  kBf16Cfg512Dyn,           // 256x512 tiles, units handed out at run time
#ifdef GEMM_B200_TUNING
  kBf16Tune2ctaDirect, kBf16Tune2ctaTma, kBf16Tune512s4, kBf16Tune512Direct,
#endif
  kNumBf16Configs
};

static const Bf16ConfigEntry kBf16Configs[] = {
    GEMM_B200_BF16_ENTRY("1cta_128x256x64_s4_direct", Bf16_1cta_direct),
    GEMM_B200_BF16_ENTRY("1cta_128x256x64_s4_tmastore", Bf16_1cta_tma),
    GEMM_B200_BF16_ENTRY("2cta_256x256x64_s6_tmastore_maskcommit", Bf16_2cta_tma_m),
    GEMM_B200_BF16_ENTRY("2cta_256x512x64_s3_tmastore2_maskcommit", Bf16_2cta_n512_s3),
    GEMM_B200_BF16_ENTRY("2cta_256x128x64_s7_tmastore_maskcommit", Bf16_2cta_n128),
    GEMM_B200_BF16_ENTRY("1cta_128x128x64_s6_tmastore", Bf16_1cta_n128),
    GEMM_B200_BF16_ENTRY("2cta_256x256x64_s6_tmastore_maskcommit_dynamic", Bf16_2cta_tma_m_dyn),
    GEMM_B200_BF16_ENTRY("2cta_256x512x64_s3_tmastore2_maskcommit_dynamic", Bf16_2cta_n512_s3_dyn),
#ifdef GEMM_B200_TUNING
    GEMM_B200_BF16_ENTRY("2cta_256x256x64_s6_direct", Bf16_2cta_direct),
    GEMM_B200_BF16_ENTRY("2cta_256x256x64_s6_tmastore", Bf16_2cta_tma),
    GEMM_B200_BF16_ENTRY("2cta_256x512x64_s4_tmastore_maskcommit", Bf16_2cta_n512),
    GEMM_B200_BF16_ENTRY("2cta_256x512x64_s4_direct_maskcommit", Bf16_2cta_n512_d),
#endif
};
static_assert(sizeof(kBf16Configs) / sizeof(kBf16Configs[0]) == kNumBf16Configs, "table and enum out of step");

// A stored transposed ([K, M] row-major, the layout of an activation matrix in the weight-gradient
// product X^T dY): the multi-round tile shapes and the single-CTA tile.
struct Bf16AtEntry {
  int config;
  int (*launch[2][2])(const Bf16Args&);   // [b_layout][out_dtype]
};
#define GEMM_B200_BF16_AT_ENTRY(ID, CFG)                                                         \
  {                                                                                              \
    ID, {                                                                                        \
      {launch_bf16<CFG, true, false, true>, launch_bf16<CFG, true, true, true>},                 \
      {launch_bf16<CFG, false, false, true>, launch_bf16<CFG, false, true, true>}                \
    }                                                                                            \
  }
static const Bf16AtEntry kBf16AtConfigs[] = {
    GEMM_B200_BF16_AT_ENTRY(kBf16Cfg1cta, Bf16_1cta_tma),
    GEMM_B200_BF16_AT_ENTRY(kBf16Cfg256, Bf16_2cta_tma_m),
    GEMM_B200_BF16_AT_ENTRY(kBf16Cfg512, Bf16_2cta_n512_s3),
    GEMM_B200_BF16_AT_ENTRY(kBf16Cfg256Dyn, Bf16_2cta_tma_m_dyn),
    GEMM_B200_BF16_AT_ENTRY(kBf16Cfg512Dyn, Bf16_2cta_n512_s3_dyn),
};

// 256x512 tiles move 25 % fewer operand bytes per flop and measure ~4 % faster when both tile
// shapes fill their rounds equally well; with few tiles the coarser grid wastes more of the last
// round of the persistent schedule.  Pick by estimated round efficiency.
static int pick_bf16_config(int64_t M, int64_t N, int64_t K, int sms, int64_t batch = 1) {
  // one row tile: the problem streams B from HBM; single-CTA tiles give twice as many independent
  // streams (16 x 8192 x 28672: 91 us = 5.2 TB/s against 110-118 us with CTA pairs)
  if (M <= kBlockM) return kBf16Cfg1cta;
  const int64_t clusters = sms / 2 > 0 ? sms / 2 : 1;
  auto eff = [&](int64_t tile_n) {
    const int64_t units = batch * ceil_div64(M, 2 * kBlockM) * ceil_div64(N, tile_n);
    const double fill = (double)units / (double)(ceil_div64(units, clusters) * clusters);
    const double used = (double)N / (double)(ceil_div64(N, tile_n) * tile_n);   // columns of the last tile in use
    return fill * used;
  };
  // the 512-wide tile's epilogue is not hidden under a main loop: it pays off from K ~ 4096 up
  // (8192^2 x K, TFLOP/s 256-wide / 512-wide: K=2048 1607 / 1570, 4096 1627 / 1662, 8192 1591 / 1660)
  // (interleaved with the 256-wide tile on other shapes: 4096^3 1414 / 1444 for 512- / 256-wide,
  // 16384 x 4096 x 4096 1704 / 1737, 6144^3 1672 / 1671, 8192 x 8192 x 10240 1592 / 1527)
  const double gain = K >= 6144 ? 1.04 : 0.97;
  const bool wide = gain * eff(2 * kBlockN) >= eff(kBlockN);
  // More than one round of units: hand them out at run time, so that clusters which fall behind
  // do not end up alone on tiles whose operands the others streamed through the L2 long ago.
  // GEMM_B200_BF16_DYNAMIC=0 keeps the static schedule (A/B comparisons).
  static const bool dyn_ok = env_int("GEMM_B200_BF16_DYNAMIC", 1) != 0;
  const int64_t units = batch * ceil_div64(M, 2 * kBlockM) * ceil_div64(N, wide ? 2 * kBlockN : kBlockN);
  // The hand-out costs a fixed time per unit and pays through L2 locality over many long units: with
  // short tiles the static schedule is faster (TFLOP/s static / run-time, timed alternately:
  // 8192 x 1024 x 8192 1508 / 1357, 16384 x 1024 x 16384 1593 / 1405, 8192 x 2048 x 8192 1667 / 1607,
  // 16384 x 4096 x 4096 1737 / 1704; 6144^3 1671 / 1683, 8192 x 8192 x 10240 1527 / 1538).
  if (dyn_ok && units > clusters && K >= 6144) return wide ? kBf16Cfg512Dyn : kBf16Cfg256Dyn;
  return wide ? kBf16Cfg512 : kBf16Cfg256;
}

// Split-K BF16 GEMM: FP32 partial sums of every (tile, K range) unit go to `scratch`
// ([k_splits][M][N] floats) through TMA stores, then one pass sums the slices in
// ascending split order and writes C.
static bool bf16_splitk_pairs(int64_t M) {
  // From two row tiles up the partial sums come from CTA pairs (256 x 256 per pair): each CTA then
  // fetches 128 + 128 rows of operands per K block instead of 128 + 256, and these launches are
  // bound by what one SM can take in from the L2.  GEMM_B200_BF16_SPLITK_PAIR=0 keeps single CTAs.
  static const bool pair = env_int("GEMM_B200_BF16_SPLITK_PAIR", 1) != 0;
  return pair && M > kBlockM;
}

static int launch_bf16_splitk(const Bf16Args& a, int b_layout, int out_dtype, int k_splits, float* scratch, bool a_mn = false) {
  Bf16Args part = a;
  part.C = scratch;
  part.ldc = a.N;
  part.k_splits = k_splits;
  // The partial sums leave through TMA stores (32 x 32 boxes, whole 128-byte rows).  All CTAs finish
  // together, so the stores arrive as one burst of k_splits x M x N x 4 bytes; per-thread 16-byte
  // stores to 32 different rows per instruction took 6 us for 16.8 MB (1024 x 8192 x 1024, four K
  // ranges), the TMA stores 3.2.
  const bool kn = b_layout == GEMM_B200_B_ROW_MAJOR_KN;
  int rc;
  if (bf16_splitk_pairs(a.M)) {
    rc = a_mn ? (kn ? launch_bf16<Bf16_2cta_tma_m, true, true, true>(part) : launch_bf16<Bf16_2cta_tma_m, false, true, true>(part))
              : (kn ? launch_bf16<Bf16_2cta_tma_m, true, true>(part) : launch_bf16<Bf16_2cta_tma_m, false, true>(part));
  } else {
    rc = a_mn ? (kn ? launch_bf16<Bf16_1cta_tma, true, true, true>(part) : launch_bf16<Bf16_1cta_tma, false, true, true>(part))
              : (kn ? launch_bf16<Bf16_1cta_tma, true, true>(part) : launch_bf16<Bf16_1cta_tma, false, true>(part));
  }
  if (rc) return rc;
  const int num_kb = (int)ceil_div64(a.K, kBlockK);
  const int kb_per = (int)ceil_div64(num_kb, k_splits);
  const int splits = (int)ceil_div64(num_kb, kb_per);
  return launch_splitk_reduce(scratch, a.M, a.N, splits, a.C, a.ldc, out_dtype, a.stream);
}

// K split across the CTAs of a cluster, partial sums combined through distributed shared memory
// (gemm_bf16_ksplit.cuh): one launch, no scratch.  `splits` = CTAs per cluster, 2, 4 or 8.
template <bool B_MN, bool OUT_F32>
static int launch_bf16_cluster_splitk(const Bf16Args& a, int splits) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  CUtensorMap tmA, tmB;
  if (int rc = make_map_3d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.A, a.M, a.K, a.lda, 1, a.M * a.lda, kBlockK, kBlockM,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (B_MN) {
    if (int rc = make_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.B, a.K, a.N, a.ldb, 1, a.K * a.ldb, 64, kBlockK,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    if (int rc = make_map_3d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.B, a.N, a.K, a.ldb, 1, a.N * a.ldb, kBlockK, kKsBN,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  auto kern = gemm_bf16_cluster_splitk_kernel<B_MN, OUT_F32>;
  {
    // opt in to the dynamic shared memory size once per device
    static std::mutex mu;
    static bool done[64] = {false};
    std::lock_guard<std::mutex> lk(mu);
    if (!done[di.dev & 63]) {
      GEMM_B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kKsSmemBytes));
      done[di.dev & 63] = true;
    }
  }
  KsShape shape;
  shape.M = (int)a.M;
  shape.N = (int)a.N;
  shape.K = (int)a.K;
  shape.tiles_n = (int)ceil_div64(a.N, kKsBN);
  const int64_t tiles = ceil_div64(a.M, kBlockM) * shape.tiles_n;
  const int num_kb = (int)ceil_div64(a.K, kBlockK);
  shape.kb_per_split = (int)ceil_div64(num_kb, splits);
  if ((int64_t)(splits - 1) * shape.kb_per_split >= num_kb)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_cluster_splitk: %d splits would leave a CTA without K blocks (K = %lld)",
                splits, (long long)a.K);
  if (tiles * splits > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_bf16_cluster_splitk: too many tiles");
  return launch_clusters(kern, (int)tiles, splits, kKsThreads, kKsSmemBytes, a.stream, tmA, tmB, a.C, a.ldc, shape);
}

static int launch_bf16_cluster_splitk_dispatch(const Bf16Args& a, int b_layout, int out_dtype, int splits) {
  const bool mn = b_layout == GEMM_B200_B_ROW_MAJOR_KN, f32 = out_dtype == GEMM_B200_OUT_F32;
  return mn ? (f32 ? launch_bf16_cluster_splitk<true, true>(a, splits) : launch_bf16_cluster_splitk<true, false>(a, splits))
            : (f32 ? launch_bf16_cluster_splitk<false, true>(a, splits) : launch_bf16_cluster_splitk<false, false>(a, splits));
}

// Cluster size for the in-cluster K split, 1 = do not use it.  Measured on a B200 (call time in us,
// default path / clusters of 4): 128 x 4096 x 4096 23.6 / 21.5, 64 x 2048 x 2048 19.3 / 15.3,
// 384 x 4096 x 1024 23.4 / 17.4, 256 x 4096 x 2048 23.6 / 19.5, 256 x 2048 x 2048 21.4 / 15.4,
// 16 x 4096 x 4096 19.4 / 19.5; clusters of 8 for at most 8 tiles: 32 x 4096 x 1024 17.3 / 15.3.
// It loses where the tiles alone fill half the SMs (1024^3: 13.3 / 23.5) and for very long K,
// where the two-launch split with many more ranges wins (512 x 32768 x 512: 39.9 / 54.3).
static int bf16_cluster_splits(int64_t M, int64_t N, int64_t K) {
  const int64_t tiles = ceil_div64(M, kBlockM) * ceil_div64(N, kKsBN), num_kb = ceil_div64(K, kBlockK);
  int s = 1;
  if (tiles <= 8 && K <= 16384) s = 8;
  else if (tiles <= 32 && K <= 8192) s = 4;
  if (s == 1 || num_kb < 8 * s) return 1;                                   // at least 512 of K per CTA
  if ((int64_t)(s - 1) * ceil_div64(num_kb, s) >= num_kb) return 1;         // no CTA without K blocks
  return s;
}

// K ranges for a BF16 problem whose tiles alone leave most of the GPU idle; 1 = do not split.
// Estimated call time in us, fitted to measurements on a B200:
//   unsplit   rounds x K blocks x t_kb                      (256-wide tiles; t_kb = 0.195 for 256 x 128 pair tiles)
//   s ranges  rounds(s) x K blocks per range x t_kb  +  s x (M N 8 bytes / 7.8 TB/s)  +  6
// with t_kb = 0.30 us per 64-wide K block for a CTA pair on a 256 x 256 tile and 0.39 for a single CTA
// on 128 x 256 (both bound by the ~64 bytes per clock one SM takes in from the L2), the second term
// the FP32 slice every range writes and the reduction reads, the third the reduction launch.
// 1024 x 8192 x 1024: unsplit 33.8 us measured, 4 ranges 27.6 (the choice), 8 ranges 31.7;
// 1024 x 16384 x 1024: 85 / 39.8 / 43.9; 512 x 32768 x 512: 16 ranges 33.8 (the choice), 8 ranges 37.9.
static int bf16_auto_splits(int64_t M, int64_t N, int64_t K, int sms) {
  if (N % 4 != 0) return 1;
  const bool pair = bf16_splitk_pairs(M);
  const int64_t tiles = ceil_div64(M, pair ? 2 * kBlockM : kBlockM) * ceil_div64(N, kBlockN);
  const int64_t slots = pair ? (sms / 2 > 0 ? sms / 2 : 1) : sms;
  const int64_t num_kb = ceil_div64(K, kBlockK);
  if (3 * tiles >= 2 * slots || num_kb < 32) return 1;          // the tiles fill two thirds of the GPU, or K < 2048
  const double t_kb = pair ? 0.30 : 0.39;
  const double slice_us = (double)M * (double)N * 8.0 / 7.8e6;
  double best_cost = (double)ceil_div64(tiles, slots) * (double)num_kb * t_kb;
  if (pair) {
    const int64_t units128 = ceil_div64(M, 2 * kBlockM) * ceil_div64(N, 128);
    const double c128 = (double)ceil_div64(units128, slots) * (double)num_kb * 0.195;
    if (c128 < best_cost) best_cost = c128;
  }
  int best = 1;
  for (int s = 2; s <= 32; ++s) {
    const int64_t kb_per = ceil_div64(num_kb, s);
    if (kb_per < 8) break;                                       // at least 512 of K per range
    if ((double)s * (double)M * (double)N * 4.0 > 268435456.0) break;   // scratch of at most 256 MiB
    if (ceil_div64(num_kb, kb_per) != s) continue;               // no empty range
    const double cost = (double)ceil_div64(tiles * s, slots) * (double)kb_per * t_kb + s * slice_us + 6.0;
    if (cost < best_cost) { best_cost = cost; best = s; }
  }
  return best;
}

}  // namespace tc
}  // namespace gemm_b200

namespace gemm_b200 {
namespace tc {

// Shared body of the plain and the batched BF16 entry points (batch == 1, strides 0: plain).
// k_splits: 0 = let the library decide (its own scratch), 1 = never split, > 1 = split into that
// many K ranges on `scratch` (k_splits * M * N floats).
static int bf16_entry(const void* A, const void* B, void* C, int64_t batch, int64_t M, int64_t N, int64_t K, int64_t lda,
                      int64_t ldb, int64_t ldc, int64_t stride_a, int64_t stride_b, int64_t stride_c, int b_layout,
                      int out_dtype, int config, void* stream, int k_splits = 0, float* scratch = nullptr) {
  if (M < 0 || N < 0 || K < 0 || batch < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: negative size");
  if (b_layout != GEMM_B200_B_ROW_MAJOR_KN && b_layout != GEMM_B200_B_ROW_MAJOR_NK)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: b_layout %d", b_layout);
  if (out_dtype != GEMM_B200_OUT_BF16 && out_dtype != GEMM_B200_OUT_F32)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: out_dtype %d", out_dtype);
  if (config >= kNumBf16Configs) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: config %d out of range", config);
  if (M == 0 || N == 0 || batch == 0) return GEMM_B200_OK;
  if (!C || (K > 0 && (!A || !B))) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: null pointer");
  const int64_t b_row = (b_layout == GEMM_B200_B_ROW_MAJOR_KN) ? N : K;
  const int64_t b_rows = (b_layout == GEMM_B200_B_ROW_MAJOR_KN) ? K : N;
  if (lda < K || ldb < b_row || ldc < N)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16: leading dimension smaller than the row (lda=%lld ldb=%lld ldc=%lld)",
                (long long)lda, (long long)ldb, (long long)ldc);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff || batch > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_bf16: a dimension exceeds 2^31-1");
  const int c_elem = out_dtype == GEMM_B200_OUT_F32 ? 4 : 2;
  if (batch > 1) {
    // matrices of one operand must not interleave; 0 shares A or B between the problems
    if (stride_a < 0 || stride_b < 0 || (stride_a != 0 && stride_a < (M - 1) * lda + K) ||
        (stride_b != 0 && stride_b < (b_rows - 1) * ldb + b_row) || stride_c < (M - 1) * ldc + N)
      return fail(GEMM_B200_ERR_INVALID_ARG,
                  "gemm_bf16_batched: a batch stride is smaller than its matrix (stride_a=%lld stride_b=%lld stride_c=%lld)",
                  (long long)stride_a, (long long)stride_b, (long long)stride_c);
    if (stride_a % 8 != 0 || stride_b % 8 != 0 || (stride_c * c_elem) % 16 != 0)
      return fail(GEMM_B200_ERR_ALIGNMENT,
                  "gemm_bf16_batched: stride_a and stride_b must be multiples of 8, stride_c*sizeof(C) of 16 bytes");
  } else {
    stride_a = stride_b = stride_c = 0;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    for (int64_t b = 0; b < batch; ++b)
      GEMM_B200_CUDA_TRY(cudaMemset2DAsync(static_cast<char*>(C) + b * stride_c * c_elem, (size_t)ldc * c_elem, 0,
                                           (size_t)N * c_elem, (size_t)M, st));
    return GEMM_B200_OK;
  }
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_bf16: A, B and C must be 16-byte aligned");
  if (lda % 8 != 0 || ldb % 8 != 0 || (ldc * c_elem) % 16 != 0 || N % (16 / c_elem) != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT,
                "gemm_bf16: lda and ldb must be multiples of 8, ldc*sizeof(C) and N*sizeof(C) multiples of 16 bytes "
                "(lda=%lld ldb=%lld ldc=%lld N=%lld)", (long long)lda, (long long)ldb, (long long)ldc, (long long)N);
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  if (di.cc_major != 10)
    return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_bf16: device has compute capability %d.x, need 10.x (sm_100a)", di.cc_major);
  Bf16Args args{A, B, C, M, N, K, lda, ldb, ldc, st, batch, stride_a, stride_b, stride_c};
  if (k_splits > 1) return launch_bf16_splitk(args, b_layout, out_dtype, k_splits, scratch);
  if (k_splits < 0) return launch_bf16_cluster_splitk_dispatch(args, b_layout, out_dtype, -k_splits);
  if (config < 0 && k_splits == 0 && batch == 1 && static_cast<int>(env_int("GEMM_B200_BF16_CONFIG", -1)) < 0) {
    // few output tiles: split K inside a cluster (one launch, partial sums through shared memory)
    static const bool cluster_ok = env_int("GEMM_B200_BF16_CLUSTER_SPLITK", 1) != 0;
    const int cs = cluster_ok ? bf16_cluster_splits(M, N, K) : 1;
    if (cs > 1) {
      if (log_enabled())
        fprintf(stderr, "[gemm_b200] gemm_bf16 %lldx%lldx%lld -> 128x128 tiles, K split over clusters of %d\n", (long long)M,
                (long long)K, (long long)N, cs);
      return launch_bf16_cluster_splitk_dispatch(args, b_layout, out_dtype, cs);
    }
  }
  if (config < 0 && k_splits == 0 && batch == 1 && static_cast<int>(env_int("GEMM_B200_BF16_CONFIG", -1)) < 0) {
    // few output tiles and a long K: cut K so the whole GPU works on the problem
    const int splits = bf16_auto_splits(M, N, K, di.sms);
    if (splits > 1) {
      float* ws = nullptr;
      if (int rc = cached_scratch(di.dev, (size_t)splits * M * N * sizeof(float), &ws, st)) return rc;
      if (ws) {
        if (log_enabled())
          fprintf(stderr, "[gemm_b200] gemm_bf16 %lldx%lldx%lld -> %s, %d K splits\n", (long long)M, (long long)K,
                  (long long)N, kBf16Configs[bf16_splitk_pairs(M) ? kBf16Cfg256 : kBf16Cfg1cta].name, splits);
        return launch_bf16_splitk(args, b_layout, out_dtype, splits, ws);
      }
    }
  }
  if (config < 0 && batch == 1 && static_cast<int>(env_int("GEMM_B200_BF16_CONFIG", -1)) < 0) {
    // Problems whose 256-column tiles leave most SMs idle and whose K is not long enough for K
    // splits to pay: 128-column tiles give twice the units in one launch (256 x 8192 x 8192:
    // 54 -> 48 us, 512 x 4096 x 4096: 31.5 -> 25.4 us, 1024^3: 15.2 -> 13.2 us, 128 x 4096 x 4096:
    // 25.6 us with K splits -> 22.6 us; from 64 tiles of 256 columns up the wider tile wins again).
    const int64_t row_pairs = ceil_div64(M, 2 * kBlockM);
    const int64_t units256 = row_pairs * ceil_div64(N, kBlockN), units128 = row_pairs * ceil_div64(N, 128);
    const int64_t tiles128 = ceil_div64(N, 128);
    if (M > kBlockM && 4 * units256 <= di.sms && 8 * units128 >= di.sms && K <= 8192)
      config = kBf16Cfg2ctaN128;
    else if (M > 32 && M <= kBlockM && tiles128 >= 24 && tiles128 <= di.sms && K <= 4096)
      config = kBf16Cfg1ctaN128;
  }
  if (config < 0) {
    static const int forced = env_int("GEMM_B200_BF16_CONFIG", -1);
    // a batch of single-row-tile problems is a well-filled grid, not a skinny one
    config = (forced >= 0 && forced < kNumBf16Configs) ? forced
             : (batch > 1 && M <= kBlockM)             ? kBf16Cfg1cta
                                                       : pick_bf16_config(M, N, K, di.sms, batch);
  }
  if (log_enabled())
    fprintf(stderr, "[gemm_b200] gemm_bf16 %lld x %lldx%lldx%lld -> %s\n", (long long)batch, (long long)M, (long long)K,
            (long long)N, kBf16Configs[config].name);
  return kBf16Configs[config].launch[b_layout][out_dtype](args);
}

// C = A^T-stored @ B: A is [K, M] row-major (lda >= M).  One launch, tile shape by the same rule as
// the plain entry; no K splits.
static int bf16_at_entry(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int64_t ldc, int b_layout, int out_dtype, void* stream) {
  if (M < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_at: negative size");
  if (b_layout != GEMM_B200_B_ROW_MAJOR_KN && b_layout != GEMM_B200_B_ROW_MAJOR_NK)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_at: b_layout %d", b_layout);
  if (out_dtype != GEMM_B200_OUT_BF16 && out_dtype != GEMM_B200_OUT_F32)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_at: out_dtype %d", out_dtype);
  if (M == 0 || N == 0) return GEMM_B200_OK;
  if (!C || (K > 0 && (!A || !B))) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_at: null pointer");
  const int64_t b_row = (b_layout == GEMM_B200_B_ROW_MAJOR_KN) ? N : K;
  if (lda < M || ldb < b_row || ldc < N)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_at: leading dimension smaller than the row (lda=%lld ldb=%lld ldc=%lld)",
                (long long)lda, (long long)ldb, (long long)ldc);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_bf16_at: a dimension exceeds 2^31-1");
  const int c_elem = out_dtype == GEMM_B200_OUT_F32 ? 4 : 2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    GEMM_B200_CUDA_TRY(cudaMemset2DAsync(C, (size_t)ldc * c_elem, 0, (size_t)N * c_elem, (size_t)M, st));
    return GEMM_B200_OK;
  }
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_bf16_at: A, B and C must be 16-byte aligned");
  if (lda % 8 != 0 || ldb % 8 != 0 || (ldc * c_elem) % 16 != 0 || N % (16 / c_elem) != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT,
                "gemm_bf16_at: lda and ldb must be multiples of 8, ldc*sizeof(C) and N*sizeof(C) multiples of 16 bytes "
                "(lda=%lld ldb=%lld ldc=%lld N=%lld)", (long long)lda, (long long)ldb, (long long)ldc, (long long)N);
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  if (di.cc_major != 10)
    return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_bf16_at: device has compute capability %d.x, need 10.x (sm_100a)", di.cc_major);
  Bf16Args args{A, B, C, M, N, K, lda, ldb, ldc, st};
  {
    // few output tiles and a long K (a weight gradient over many tokens): FP32 partial sums per
    // K range on the library's scratch, then the reduction pass, as in the plain entry
    const int splits = bf16_auto_splits(M, N, K, di.sms);
    float* ws = nullptr;
    if (splits > 1) {
      if (int rc = cached_scratch(di.dev, (size_t)splits * M * N * sizeof(float), &ws, st)) return rc;
    }
    if (ws) {
      if (log_enabled())
        fprintf(stderr, "[gemm_b200] gemm_bf16_at %lldx%lldx%lld -> %d K splits\n", (long long)M, (long long)K, (long long)N, splits);
      return launch_bf16_splitk(args, b_layout, out_dtype, splits, ws, /*a_mn=*/true);
    }
  }
  const int config = pick_bf16_config(M, N, K, di.sms);
  if (log_enabled())
    fprintf(stderr, "[gemm_b200] gemm_bf16_at %lldx%lldx%lld -> %s\n", (long long)M, (long long)K, (long long)N,
            kBf16Configs[config].name);
  for (const Bf16AtEntry& e : kBf16AtConfigs)
    if (e.config == config) return e.launch[b_layout][out_dtype](args);
  return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_bf16_at: no transposed-A build of %s", kBf16Configs[config].name);
}

}  // namespace tc
}  // namespace gemm_b200

extern "C" int gemm_b200_gemm_bf16_at(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                      int64_t ldb, int64_t ldc, int b_layout, int out_dtype, void* stream) {
  return gemm_b200::tc::bf16_at_entry(A, B, C, M, N, K, lda, ldb, ldc, b_layout, out_dtype, stream);
}

extern "C" int gemm_b200_gemm_bf16_cfg(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                       int64_t lda, int64_t ldb, int64_t ldc, int b_layout, int out_dtype,
                                       int config, void* stream) {
  return gemm_b200::tc::bf16_entry(A, B, C, 1, M, N, K, lda, ldb, ldc, 0, 0, 0, b_layout, out_dtype, config, stream);
}

extern "C" size_t gemm_b200_gemm_bf16_splitk_scratch_bytes(int64_t M, int64_t N, int k_splits) {
  if (M <= 0 || N <= 0 || k_splits <= 0) return 0;
  return (size_t)k_splits * (size_t)M * (size_t)N * sizeof(float);
}

extern "C" int gemm_b200_gemm_bf16_auto_splits(int64_t M, int64_t N, int64_t K) {
  gemm_b200::tc::DeviceInfo di;
  if (gemm_b200::tc::device_info(&di)) return 1;
  return gemm_b200::tc::bf16_auto_splits(M, N, K, di.sms);
}

extern "C" int gemm_b200_gemm_bf16_splitk(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                          int64_t lda, int64_t ldb, int64_t ldc, int b_layout, int out_dtype,
                                          int k_splits, void* scratch, size_t scratch_bytes, void* stream) {
  using namespace gemm_b200;
  if (k_splits < 1 || k_splits > 64) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_splitk: k_splits %d not in [1, 64]", k_splits);
  if (k_splits > 1) {
    if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 16 != 0)
      return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_splitk: scratch must be a 16-byte aligned device buffer");
    if (M > 0 && N > 0 && scratch_bytes < gemm_b200_gemm_bf16_splitk_scratch_bytes(M, N, k_splits))
      return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_splitk: scratch holds %zu bytes, %zu needed", scratch_bytes,
                  gemm_b200_gemm_bf16_splitk_scratch_bytes(M, N, k_splits));
    if (N % 4 != 0) return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_bf16_splitk: N must be a multiple of 4");
  }
  return tc::bf16_entry(A, B, C, 1, M, N, K, lda, ldb, ldc, 0, 0, 0, b_layout, out_dtype, -1, stream, k_splits,
                        static_cast<float*>(scratch));
}

extern "C" int gemm_b200_gemm_bf16_cluster_splitk(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                                  int64_t lda, int64_t ldb, int64_t ldc, int b_layout, int out_dtype,
                                                  int k_splits, void* stream) {
  using namespace gemm_b200;
  if (k_splits != 2 && k_splits != 4 && k_splits != 8)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_cluster_splitk: k_splits %d is not 2, 4 or 8", k_splits);
  if (K <= 0 || M <= 0 || N <= 0)   // nothing to split: the plain entry point handles empty problems and K == 0
    return gemm_b200_gemm_bf16(A, B, C, M, N, K, lda, ldb, ldc, b_layout, out_dtype, stream);
  return tc::bf16_entry(A, B, C, 1, M, N, K, lda, ldb, ldc, 0, 0, 0, b_layout, out_dtype, -1, stream, -k_splits);
}

extern "C" int gemm_b200_gemm_bf16_grouped(const void* A, const void* B, void* C, int64_t groups, const int64_t* m_sizes,
                                           int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t stride_b, int64_t ldc,
                                           int b_layout, int out_dtype, void* stream) {
  using namespace gemm_b200;
  if (groups < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_grouped: negative size");
  if (b_layout != GEMM_B200_B_ROW_MAJOR_KN && b_layout != GEMM_B200_B_ROW_MAJOR_NK)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_grouped: b_layout %d", b_layout);
  if (out_dtype != GEMM_B200_OUT_BF16 && out_dtype != GEMM_B200_OUT_F32)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_grouped: out_dtype %d", out_dtype);
  if (groups == 0 || N == 0) return GEMM_B200_OK;
  if (!m_sizes) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_grouped: null m_sizes");
  int64_t rows = 0;
  for (int64_t g = 0; g < groups; ++g) {
    if (m_sizes[g] < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_grouped: negative group size");
    rows += m_sizes[g];
    if (rows > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_bf16_grouped: more than 2^31-1 rows");
  }
  if (rows == 0) return GEMM_B200_OK;
  if (N > 0x7fffffff || K > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_bf16_grouped: a dimension exceeds 2^31-1");
  if (!C || (K > 0 && (!A || !B))) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_grouped: null pointer");
  const int64_t b_row = (b_layout == GEMM_B200_B_ROW_MAJOR_KN) ? N : K, b_rows = (b_layout == GEMM_B200_B_ROW_MAJOR_KN) ? K : N;
  if (lda < K || ldb < b_row || ldc < N || (groups > 1 && stride_b < (b_rows - 1) * ldb + b_row))
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_bf16_grouped: a leading dimension or stride_b is smaller than its matrix");
  const int c_elem = out_dtype == GEMM_B200_OUT_F32 ? 4 : 2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    GEMM_B200_CUDA_TRY(cudaMemset2DAsync(C, (size_t)ldc * c_elem, 0, (size_t)N * c_elem, (size_t)rows, st));
    return GEMM_B200_OK;
  }
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_bf16_grouped: A, B and C must be 16-byte aligned");
  if (lda % 8 != 0 || ldb % 8 != 0 || stride_b % 8 != 0 || (ldc * c_elem) % 16 != 0 || N % (16 / c_elem) != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT,
                "gemm_bf16_grouped: lda, ldb and stride_b must be multiples of 8, ldc*sizeof(C) and N*sizeof(C) of 16 bytes");
  tc::DeviceInfo di;
  if (int rc = tc::device_info(&di)) return rc;
  if (di.cc_major != 10)
    return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_bf16_grouped: device has compute capability %d.x, need 10.x (sm_100a)", di.cc_major);
  const bool mn = b_layout == GEMM_B200_B_ROW_MAJOR_KN, f32 = out_dtype == GEMM_B200_OUT_F32;
  // kMaxGroups groups per launch; their rows of A and C and their B matrices follow one another
  int64_t row0 = 0;
  for (int64_t g0 = 0; g0 < groups; g0 += tc::kMaxGroups) {
    const int n = (int)(groups - g0 < tc::kMaxGroups ? groups - g0 : tc::kMaxGroups);
    const char* a = static_cast<const char*>(A) + row0 * lda * 2;
    const char* b = static_cast<const char*>(B) + g0 * stride_b * 2;
    char* c = static_cast<char*>(C) + row0 * ldc * c_elem;
    const int rc = mn ? (f32 ? tc::launch_bf16_grouped<true, true>(a, b, c, n, m_sizes + g0, N, K, lda, ldb, stride_b, ldc, st)
                             : tc::launch_bf16_grouped<true, false>(a, b, c, n, m_sizes + g0, N, K, lda, ldb, stride_b, ldc, st))
                      : (f32 ? tc::launch_bf16_grouped<false, true>(a, b, c, n, m_sizes + g0, N, K, lda, ldb, stride_b, ldc, st)
                             : tc::launch_bf16_grouped<false, false>(a, b, c, n, m_sizes + g0, N, K, lda, ldb, stride_b, ldc, st));
    if (rc) return rc;
    for (int g = 0; g < n; ++g) row0 += m_sizes[g0 + g];
  }
  return GEMM_B200_OK;
}

extern "C" int gemm_b200_gemm_bf16_batched(const void* A, const void* B, void* C, int64_t batch, int64_t M, int64_t N,
                                           int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t stride_a,
                                           int64_t stride_b, int64_t stride_c, int b_layout, int out_dtype, void* stream) {
  return gemm_b200::tc::bf16_entry(A, B, C, batch, M, N, K, lda, ldb, ldc, stride_a, stride_b, stride_c, b_layout,
                                   out_dtype, -1, stream);
}

extern "C" int gemm_b200_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                                   int64_t lda, int64_t ldb, int64_t ldc, int b_layout, int out_dtype, void* stream) {
  return gemm_b200_gemm_bf16_cfg(A, B, C, M, N, K, lda, ldb, ldc, b_layout, out_dtype, -1, stream);
}
extern "C" int gemm_b200_gemm_bf16_num_configs(void) { return gemm_b200::tc::kNumBf16Configs; }
extern "C" const char* gemm_b200_gemm_bf16_config_name(int config) {
  if (config < 0 || config >= gemm_b200::tc::kNumBf16Configs) return "";
  return gemm_b200::tc::kBf16Configs[config].name;
}

extern "C" int gemm_b200_check_status(void* stream, int32_t detail[4]) {
  using namespace gemm_b200;
  GEMM_B200_CUDA_TRY(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  int32_t h[4] = {0, 0, 0, 0};
  GEMM_B200_CUDA_TRY(cudaMemcpyFromSymbol(h, tc::g_status, sizeof(h)));
  if (detail)
    for (int i = 0; i < 4; ++i) detail[i] = h[i];
  if (h[0] != 0) {
    const int32_t z[4] = {0, 0, 0, 0};
    GEMM_B200_CUDA_TRY(cudaMemcpyToSymbol(tc::g_status, z, sizeof(z)));
    return fail(GEMM_B200_ERR_TIMEOUT, "a device-side wait gave up: block %d role %d stage %d", h[1], h[2], h[3]);
  }
  return GEMM_B200_OK;
}


// =========================================================================================
// MXFP8
// =========================================================================================
namespace gemm_b200 {
namespace tc {

struct MxArgs {
  const void *Aq, *SFA, *Bq, *SFB;
  void* C;
  int64_t M, N, K, ldc;
  cudaStream_t stream;
  int k_splits = 1;        // > 1: FP32 partials go to `scratch` ([k_splits][M][N]), then a reduce pass
  float* scratch = nullptr;
  uint8_t* SFC = nullptr;  // packed scales of C for the quantising epilogue
  MxGroups groups = {};    // count > 0: grouped launch, Bq / SFB hold count matrices one after another
};

// packed scale buffer of `rows` rows viewed as int32 [row blocks][kchunks * 128]
static int make_scale_map(CUtensorMap* map, const void* sf, int64_t rows, int64_t K, int box_blocks) {
  const int64_t kchunks = ceil_div64(K / 32, 4), blocks = ceil_div64(rows, 128);
  return make_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, sf, blocks, kchunks * 128, kchunks * 128, 128, box_blocks,
                     CU_TENSOR_MAP_SWIZZLE_NONE);
}

template <class Cfg, int OUT>
static int launch_mxfp8(const MxArgs& a) {
  constexpr bool OUT_F32 = (OUT == 1);
  constexpr int CG = Cfg::CG;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  CUtensorMap tmA, tmB, tmSFA, tmSFB;
  if (Cfg::A_ROWS != kBlockM && a.M > Cfg::A_ROWS)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: this variant handles at most %d rows of A", Cfg::A_ROWS);
  if (int rc = make_map_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.Aq, a.M, a.K, a.K, kMxBlockK, Cfg::A_ROWS,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  // grouped launch: the B matrices (and their scale buffers, ceil(N / 128) blocks each) as one tall matrix
  const int64_t nb = a.groups.count > 0 ? a.groups.count : 1;
  if (int rc = make_map_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.Bq, nb * a.N, a.K, a.K, kMxBlockK, Cfg::BN_CTA,
                           CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_scale_map(&tmSFA, a.SFA, a.M, a.K, 1)) return rc;
  if (int rc = make_scale_map(&tmSFB, a.SFB, nb > 1 ? nb * ceil_div64(a.N, 128) * 128 : a.N, a.K, Cfg::BN / 128)) return rc;
  CUtensorMap tmC = tmA;   // only read by the TMA-store epilogue
  if (Cfg::EPI == 1) {
    if (OUT == 2) {   // e4m3 bytes: 128 columns x 32 rows per store
      if (int rc = make_map_2d(&tmC, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.C, a.M, a.N, a.ldc, 128, 32, CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;
    } else if (int rc = make_map_2d(&tmC, OUT_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                    OUT_F32 ? 4 : 2, a.C, a.M, a.N, a.ldc, OUT_F32 ? 32 : 64, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
      return rc;
    }
  }

  auto kern = gemm_mxfp8_kernel<Cfg, OUT>;
  int max_clusters = 0;
  if (int rc = persistent_clusters(kern, CG, kMxThreads, Cfg::SMEM_BYTES, di, &max_clusters)) return rc;

  GemmShape shape;
  shape.M = (int)a.M;
  shape.N = (int)a.N;
  shape.K = (int)a.K;
  shape.tiles_m = (int)ceil_div64(a.M, kBlockM * CG);
  shape.tiles_n = (int)ceil_div64(a.N, Cfg::BN);
  const int num_kb = (int)ceil_div64(a.K, kMxBlockK);
  shape.kb_per_split = (int)ceil_div64(num_kb, a.k_splits);
  shape.batch = 1;
  shape.a_z = shape.b_z = 0;
  shape.c_batch_stride = 0;
  // MXFP8 kernel: B tiles evict-first when there is one row tile (B is then read exactly once).
  // Per call after a 252 MB write flush (an L2 full of dirty lines), without / with: 16 x 8192 x 28672
  // 57.4 / 53.2 us, 128 x 8192 x 28672 61.7 / 52.0, 16 x 8192 x 8192 27.6 / 23.7; after a read flush the same.
  static const bool stream_ok = env_int("GEMM_B200_MXFP8_STREAM_B", 1) != 0;
  shape.l2_stream_a_keep_b = (stream_ok && CG == 1 && shape.tiles_m == 1) ? 1 : 0;
  shape.k_splits = (int)ceil_div64(num_kb, shape.kb_per_split);   // no empty split
  shape.split_stride = a.M * a.N;
  shape.raster_group = raster_group_for((int64_t)Cfg::BN * a.K, Cfg::BN, 0);
  const int64_t num_tiles = (int64_t)shape.tiles_m * shape.tiles_n * shape.k_splits;
  if (num_tiles > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8: too many tiles");
  const int clusters = Cfg::DYN ? (int)num_tiles : (int)(num_tiles < max_clusters ? num_tiles : max_clusters);
  if (Cfg::DYN && shape.k_splits > 1)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: K splits run on the static schedule");
  return launch_clusters(kern, clusters, CG, kMxThreads, Cfg::SMEM_BYTES, a.stream, tmA, tmB, tmSFA, tmSFB, tmC, a.C, a.ldc, a.SFC, shape,
                         a.groups);
}

// Split-K: FP32 partial sums of every (tile, K split) into scratch, then one reduce pass into C.
template <class Cfg>
static int launch_mxfp8_splitk(const MxArgs& a, int out_dtype) {
  MxArgs part = a;
  part.C = a.scratch;
  part.ldc = a.N;
  if (int rc = launch_mxfp8<Cfg, 1>(part)) return rc;
  const int num_kb = (int)ceil_div64(a.K, kMxBlockK);
  const int kb_per = (int)ceil_div64(num_kb, a.k_splits);
  const int splits = (int)ceil_div64(num_kb, kb_per);
  return launch_splitk_reduce(a.scratch, a.M, a.N, splits, a.C, a.ldc, out_dtype, a.stream);
}

// K split across the CTAs of a cluster (gemm_mxfp8_ksplit.cuh): one launch, no scratch.
template <bool OUT_F32>
static int launch_mxfp8_cluster_splitk(const MxArgs& a, int splits) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  CUtensorMap tmA, tmB, tmSFA, tmSFB;
  if (int rc = make_map_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.Aq, a.M, a.K, a.K, kMxBlockK, kBlockM, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_map_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.Bq, a.N, a.K, a.K, kMxBlockK, kKsBN, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_scale_map(&tmSFA, a.SFA, a.M, a.K, 1)) return rc;
  if (int rc = make_scale_map(&tmSFB, a.SFB, a.N, a.K, 1)) return rc;
  auto kern = gemm_mxfp8_cluster_splitk_kernel<OUT_F32>;
  {
    static std::mutex mu;
    static bool done[64] = {false};
    std::lock_guard<std::mutex> lk(mu);
    if (!done[di.dev & 63]) {
      GEMM_B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMxKsSmemBytes));
      done[di.dev & 63] = true;
    }
  }
  KsShape shape;
  shape.M = (int)a.M;
  shape.N = (int)a.N;
  shape.K = (int)a.K;
  shape.tiles_n = (int)ceil_div64(a.N, kKsBN);
  const int64_t tiles = ceil_div64(a.M, kBlockM) * shape.tiles_n;
  const int num_kb = (int)ceil_div64(a.K, kMxBlockK);
  shape.kb_per_split = (int)ceil_div64(num_kb, splits);
  if ((int64_t)(splits - 1) * shape.kb_per_split >= num_kb)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_cluster_splitk: %d splits would leave a CTA without K blocks (K = %lld)",
                splits, (long long)a.K);
  if (tiles * splits > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8_cluster_splitk: too many tiles");
  return launch_clusters(kern, (int)tiles, splits, kKsThreads, kMxKsSmemBytes, a.stream, tmA, tmB, tmSFA, tmSFB, a.C, a.ldc, shape);
}

// Cluster size for the in-cluster K split of the MXFP8 GEMM, 1 = do not use it.  Measured on a B200
// (call time in us, default path / clusters of 4; torch._scaled_mm beside it): 128 x 4096 x 4096
// 18.4 / 16.4 (17.2), 64 x 2048 x 2048 15.1 / 13.2 (13.1), 384 x 4096 x 1024 17.2 / 15.2 (15.4),
// 128 x 8192 x 2048 21.5 / 18.4 (21.5), 256 x 8192 x 2048 22.5 / 18.5 (21.5).  Up to 32 rows the
// narrow-A kernel with the scratch-based split stays ahead (16 x 8192 x 4096: 19.2 / 20.5,
// 16 x 16384 x 1024: 17.4 / 18.4 with clusters of 8), so those keep it.
static int mxfp8_cluster_splits(int64_t M, int64_t N, int64_t K) {
  if (M <= 32) return 1;
  const int64_t tiles = ceil_div64(M, kBlockM) * ceil_div64(N, kKsBN), num_kb = ceil_div64(K, kMxBlockK);
  int s = 1;
  if (tiles <= 8 && K <= 16384) s = 8;
  else if (tiles <= 32 && K <= 8192) s = 4;
  if (s == 1 || num_kb < 4 * s) return 1;                                   // at least 512 of K per CTA
  if ((int64_t)(s - 1) * ceil_div64(num_kb, s) >= num_kb) return 1;         // no CTA without K blocks
  return s;
}

struct MxConfigEntry {
  const char* name;
  int (*launch[2])(const MxArgs&);   // [out_dtype]
};
using Mx_1cta = MxCfg<1, 4, false>;
using Mx_2cta_m_tma = MxCfg<2, 5, true, 1>;
using Mx_1cta_a32 = MxCfg<1, 5, false, 0, 32>;   // M <= 32: 4 KB of A per stage, 5 stages of B in flight
using Mx_2cta_n128 = MxCfg<2, 7, true, 1, kBlockM, 128>;   // 256 x 128 tiles for one-round problems
using Mx_1cta_n128 = MxCfg<1, 6, false, 0, kBlockM, 128>;   // 128 x 128 tiles: 32 < M <= 128 with few column tiles
using Mx_2cta_m_tma_dyn = MxCfg<2, 5, true, 1, kBlockM, kBlockN, true>;   // units handed out at run time
#ifdef GEMM_B200_TUNING
using Mx_2cta = MxCfg<2, 6, false>;
using Mx_2cta_m = MxCfg<2, 6, true>;
#endif
// index of every variant in kMxConfigs (the order of the table below)
enum MxConfigId : int {
  kSkinnyMxConfig = 0,   // single CTA, 128 x 256 tiles: 33..128 rows, and the split-K partial sums
  kDefaultMxConfig,      // CTA pair, masked commit, TMA-store epilogue
  kNarrowMxConfig,       // M <= 32: single CTA with 32-row A stages and a deeper B pipeline
  kN128MxConfig,         // CTA pair, 256 x 128 tiles: at most half a round of 256-wide tiles
  k1ctaN128MxConfig,     // single CTA, 128 x 128 tiles
  kDynMxConfig,          // the default tile with units handed out at run time (problems of several rounds)
#ifdef GEMM_B200_TUNING
  kMxTune2cta, kMxTune2ctaMask,
#endif
  kNumMxConfigs
};
static const MxConfigEntry kMxConfigs[] = {
    {"1cta_128x256x128_s4", {launch_mxfp8<Mx_1cta, 0>, launch_mxfp8<Mx_1cta, 1>}},
    {"2cta_256x256x128_s5_maskcommit_tmastore", {launch_mxfp8<Mx_2cta_m_tma, 0>, launch_mxfp8<Mx_2cta_m_tma, 1>}},
    {"1cta_32x256x128_s5_narrowA", {launch_mxfp8<Mx_1cta_a32, 0>, launch_mxfp8<Mx_1cta_a32, 1>}},
    {"2cta_256x128x128_s7_maskcommit_tmastore", {launch_mxfp8<Mx_2cta_n128, 0>, launch_mxfp8<Mx_2cta_n128, 1>}},
    {"1cta_128x128x128_s6", {launch_mxfp8<Mx_1cta_n128, 0>, launch_mxfp8<Mx_1cta_n128, 1>}},
    {"2cta_256x256x128_s5_maskcommit_tmastore_dynamic", {launch_mxfp8<Mx_2cta_m_tma_dyn, 0>, launch_mxfp8<Mx_2cta_m_tma_dyn, 1>}},
#ifdef GEMM_B200_TUNING
    {"2cta_256x256x128_s6", {launch_mxfp8<Mx_2cta, 0>, launch_mxfp8<Mx_2cta, 1>}},
    {"2cta_256x256x128_s6_maskcommit", {launch_mxfp8<Mx_2cta_m, 0>, launch_mxfp8<Mx_2cta_m, 1>}},
#endif
};
static_assert(sizeof(kMxConfigs) / sizeof(kMxConfigs[0]) == kNumMxConfigs, "table and enum out of step");

}  // namespace tc
}  // namespace gemm_b200

extern "C" size_t gemm_b200_mxfp8_scale_bytes(int64_t rows, int64_t K) {
  if (rows <= 0 || K <= 0) return 0;
  return (size_t)(gemm_b200::ceil_div64(rows, 128) * gemm_b200::ceil_div64(gemm_b200::ceil_div64(K, 32), 4) * 512);
}
extern "C" size_t gemm_b200_mxfp8_scale_offset(int64_t rows, int64_t K, int64_t row, int64_t kb) {
  (void)rows;
  return gemm_b200::mx::scale_offset(gemm_b200::ceil_div64(gemm_b200::ceil_div64(K, 32), 4), row, kb);
}

extern "C" int gemm_b200_quantize_mxfp8(const void* X, int64_t rows, int64_t K, int64_t ldx, int transposed_in,
                                        void* Xq, void* SF, void* stream) {
  using namespace gemm_b200;
  if (rows < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "quantize_mxfp8: negative size");
  if (rows == 0 || K == 0) return GEMM_B200_OK;
  if (!X || !Xq || !SF) return fail(GEMM_B200_ERR_INVALID_ARG, "quantize_mxfp8: null pointer");
  if (K % 32 != 0) return fail(GEMM_B200_ERR_INVALID_ARG, "quantize_mxfp8: K=%lld is not a multiple of 32", (long long)K);
  if (ldx < (transposed_in ? rows : K)) return fail(GEMM_B200_ERR_INVALID_ARG, "quantize_mxfp8: ldx too small");
  if (reinterpret_cast<uintptr_t>(Xq) % 16 != 0) return fail(GEMM_B200_ERR_ALIGNMENT, "quantize_mxfp8: Xq must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t kb_pad = ceil_div64(K / 32, 4) * 4, rows_pad = ceil_div64(rows, 128) * 128;
  if (!transposed_in) {
    if (reinterpret_cast<uintptr_t>(X) % 16 != 0 || ldx % 8 != 0)
      return fail(GEMM_B200_ERR_ALIGNMENT, "quantize_mxfp8: X must be 16-byte aligned with ldx a multiple of 8");
    const int64_t threads = rows_pad * kb_pad;
    const int64_t blocks = ceil_div64(threads, 256);
    if (blocks > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "quantize_mxfp8: too large");
    mx::quantize_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(X), rows, K, ldx,
                                                               static_cast<uint8_t*>(Xq), static_cast<uint8_t*>(SF),
                                                               kb_pad, rows_pad);
  } else {
    if (kb_pad / 4 > 65535) return fail(GEMM_B200_ERR_TOO_LARGE, "quantize_mxfp8: K too large for the transposed path");
    // K chunks per CTA (fetched one ahead of the one being quantised): as many as leave about three
    // rounds of CTAs, at most kQcMaxTiles.  28672 x 8192: 138 us with one chunk per CTA, 129 us with eight.
    tc::DeviceInfo di;
    if (int rc = tc::device_info(&di)) return rc;
    const int64_t units = (rows_pad / mx::kQcCols) * (kb_pad / 4);
    int64_t tiles_per_cta = units / ((int64_t)di.sms * 6 * 3);
    tiles_per_cta = tiles_per_cta < 1 ? 1 : (tiles_per_cta > mx::kQcMaxTiles ? mx::kQcMaxTiles : tiles_per_cta);
    dim3 grid((unsigned)(rows_pad / mx::kQcCols), (unsigned)ceil_div64(kb_pad / 4, tiles_per_cta));
    const int vec_ok = (reinterpret_cast<uintptr_t>(X) % 16 == 0 && ldx % 8 == 0 && rows % 8 == 0) ? 1 : 0;
    mx::quantize_cols_kernel<mx::kQcCols><<<grid, mx::kQcCols * 4, 0, st>>>(
        static_cast<const __nv_bfloat16*>(X), rows, K, ldx, static_cast<uint8_t*>(Xq), static_cast<uint8_t*>(SF), kb_pad, vec_ok, (int)tiles_per_cta);
  }
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  GEMM_B200_CUDA_TRY(cudaGetLastError());
  return GEMM_B200_OK;
}

extern "C" int gemm_b200_gemm_mxfp8_grouped(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C,
                                            int64_t groups, const int64_t* m_sizes, int64_t N, int64_t K, int64_t ldc,
                                            int out_dtype, void* stream) {
  using namespace gemm_b200;
  if (groups < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_grouped: negative size");
  if (out_dtype != GEMM_B200_OUT_BF16 && out_dtype != GEMM_B200_OUT_F32)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_grouped: out_dtype %d", out_dtype);
  if (K % 32 != 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_grouped: K must be a multiple of 32");
  if (groups == 0 || N == 0) return GEMM_B200_OK;
  if (!m_sizes) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_grouped: null m_sizes");
  int64_t rows = 0;
  for (int64_t g = 0; g < groups; ++g) {
    if (m_sizes[g] < 0 || m_sizes[g] % 256 != 0)
      return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_grouped: group %lld has %lld rows, not a multiple of 256 (pad the group)",
                  (long long)g, (long long)m_sizes[g]);
    rows += m_sizes[g];
    if (rows > 0x7fffffff) return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8_grouped: more than 2^31-1 rows");
  }
  if (rows == 0) return GEMM_B200_OK;
  if (N > 0x7fffffff || K > 0x7fffffff || groups * N > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8_grouped: a dimension exceeds 2^31-1");
  if (!C || (K > 0 && (!Aq || !Bq || !SFA || !SFB))) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_grouped: null pointer");
  if (ldc < N) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_grouped: ldc smaller than N");
  const int c_elem = out_dtype == GEMM_B200_OUT_F32 ? 4 : 2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    GEMM_B200_CUDA_TRY(cudaMemset2DAsync(C, (size_t)ldc * c_elem, 0, (size_t)N * c_elem, (size_t)rows, st));
    return GEMM_B200_OK;
  }
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Bq) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(SFA) | reinterpret_cast<uintptr_t>(SFB)) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_mxfp8_grouped: all pointers must be 16-byte aligned");
  if ((ldc * c_elem) % 16 != 0 || N % (16 / c_elem) != 0 || (N * K) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_mxfp8_grouped: ldc*sizeof(C), N*sizeof(C) and N*K must be multiples of 16 bytes");
  tc::DeviceInfo di;
  if (int rc = tc::device_info(&di)) return rc;
  if (di.cc_major != 10)
    return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_mxfp8_grouped: device has compute capability %d.x, need 10.x (sm_100a)", di.cc_major);
  const size_t sf_b = gemm_b200_mxfp8_scale_bytes(N, K);           // scale bytes of one B matrix
  const size_t sf_row_block = (size_t)ceil_div64(K / 32, 4) * 512; // scale bytes of one 128-row block of A
  int64_t row0 = 0;
  for (int64_t g0 = 0; g0 < groups; g0 += tc::kMaxGroups) {
    const int n = (int)(groups - g0 < tc::kMaxGroups ? groups - g0 : tc::kMaxGroups);
    tc::MxArgs args{static_cast<const char*>(Aq) + row0 * K, static_cast<const char*>(SFA) + (size_t)(row0 / 128) * sf_row_block,
                    static_cast<const char*>(Bq) + g0 * N * K, static_cast<const char*>(SFB) + (size_t)g0 * sf_b,
                    static_cast<char*>(C) + row0 * ldc * c_elem, 0, N, K, ldc, st};
    args.groups.count = n;
    int64_t r = 0;
    for (int g = 0; g < n; ++g) {
      args.groups.first_block[g] = (int)(r / 128);
      r += m_sizes[g0 + g];
    }
    args.groups.first_block[n] = (int)(r / 128);
    args.M = r;
    row0 += r;
    if (r == 0) continue;
    // CTA-pair tiles; units handed out at run time for long K and several rounds, as in the plain entry
    const int64_t units256 = ceil_div64(r, 2 * tc::kBlockM) * ceil_div64(N, tc::kBlockN);
    static const bool dyn_ok = env_int("GEMM_B200_MXFP8_DYNAMIC", 1) != 0;
    const int config = (dyn_ok && 2 * units256 > (int64_t)di.sms && K >= 8192) ? tc::kDynMxConfig : tc::kDefaultMxConfig;
    if (log_enabled())
      fprintf(stderr, "[gemm_b200] gemm_mxfp8_grouped %d groups, %lld rows x %lldx%lld -> %s\n", n, (long long)r, (long long)K,
              (long long)N, tc::kMxConfigs[config].name);
    if (int rc = tc::kMxConfigs[config].launch[out_dtype](args)) return rc;
  }
  return GEMM_B200_OK;
}

extern "C" int gemm_b200_gemm_mxfp8_cfg(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C,
                                        int64_t M, int64_t N, int64_t K, int64_t ldc, int out_dtype, int config,
                                        void* stream) {
  using namespace gemm_b200;
  if (M < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: negative size");
  if (out_dtype != GEMM_B200_OUT_BF16 && out_dtype != GEMM_B200_OUT_F32)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: out_dtype %d", out_dtype);
  if (config >= tc::kNumMxConfigs) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: config %d out of range", config);
  if (M == 0 || N == 0) return GEMM_B200_OK;
  if (!C || (K > 0 && (!Aq || !Bq || !SFA || !SFB))) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: null pointer");
  if (ldc < N) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: ldc smaller than N");
  if (K % 32 != 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8: K=%lld is not a multiple of 32", (long long)K);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8: a dimension exceeds 2^31-1");
  const int c_elem = out_dtype == GEMM_B200_OUT_F32 ? 4 : 2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (K == 0) {
    GEMM_B200_CUDA_TRY(cudaMemset2DAsync(C, (size_t)ldc * c_elem, 0, (size_t)N * c_elem, (size_t)M, st));
    return GEMM_B200_OK;
  }
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Bq) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(SFA) | reinterpret_cast<uintptr_t>(SFB)) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_mxfp8: all pointers must be 16-byte aligned");
  if ((ldc * c_elem) % 16 != 0 || N % (16 / c_elem) != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_mxfp8: ldc*sizeof(C) and N*sizeof(C) must be multiples of 16 bytes");
  tc::DeviceInfo di;
  if (int rc = tc::device_info(&di)) return rc;
  if (di.cc_major != 10)
    return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_mxfp8: device has compute capability %d.x, need 10.x (sm_100a)", di.cc_major);
  tc::MxArgs args{Aq, SFA, Bq, SFB, C, M, N, K, ldc, st};
  if (config <= -4) {   // explicit in-cluster K split (gemm_b200_gemm_mxfp8_cluster_splitk): -2 - splits
    return out_dtype == GEMM_B200_OUT_F32 ? tc::launch_mxfp8_cluster_splitk<true>(args, -2 - config)
                                          : tc::launch_mxfp8_cluster_splitk<false>(args, -2 - config);
  }
  if (config < 0) {
    static const int forced = env_int("GEMM_B200_MXFP8_CONFIG", -1);
    if (forced >= 0 && forced < tc::kNumMxConfigs) config = forced;
  }
  if (config < 0) {
    // few output tiles: split K inside a cluster (one launch, partial sums through shared memory)
    static const bool cluster_ok = env_int("GEMM_B200_MXFP8_CLUSTER_SPLITK", 1) != 0;
    const int cs = cluster_ok ? tc::mxfp8_cluster_splits(M, N, K) : 1;
    if (cs > 1) {
      if (log_enabled())
        fprintf(stderr, "[gemm_b200] gemm_mxfp8 %lldx%lldx%lld -> 128x128 tiles, K split over clusters of %d\n", (long long)M,
                (long long)K, (long long)N, cs);
      return out_dtype == GEMM_B200_OUT_F32 ? tc::launch_mxfp8_cluster_splitk<true>(args, cs)
                                            : tc::launch_mxfp8_cluster_splitk<false>(args, cs);
    }
  }
  if (config < 0) {
    if (M <= 128) {
      // skinny: single-CTA tiles, and K splits when the column tiles alone leave SMs idle.  (Taller
      // problems with few tiles were tried on this path too: 256-384 x 8192 x 8192 ran 40-50 us
      // split against 38 us on CTA-pair tiles.)
      // 33..128 rows and so few 256-column tiles that half the SMs would idle: 128-column tiles in
      // one launch beat K splits with their reduce pass (128 x 8192 x 8192: 31.6 vs 33.5 us,
      // 128 x 4096 x 4096: 19.2 vs 23.3 us); below 24 such tiles K splits fill the GPU better
      const int64_t tiles128 = ceil_div64(N, 128);
      if (M > 32 && tiles128 >= 24 && tiles128 <= (int64_t)di.sms) {
        if (log_enabled())
          fprintf(stderr, "[gemm_b200] gemm_mxfp8 %lldx%lldx%lld -> %s\n", (long long)M, (long long)K, (long long)N,
                  tc::kMxConfigs[tc::k1ctaN128MxConfig].name);
        return tc::kMxConfigs[tc::k1ctaN128MxConfig].launch[out_dtype](args);
      }
      const int splits = (N % 4 == 0) ? tc::auto_splits(M, N, K, di.sms) : 1;
      if (splits > 1) {
        if (int rc = tc::cached_scratch(di.dev, (size_t)splits * M * N * sizeof(float), &args.scratch, st)) return rc;
        if (args.scratch) {
          args.k_splits = splits;
          if (log_enabled())
            fprintf(stderr, "[gemm_b200] gemm_mxfp8 %lldx%lldx%lld -> %s, %d K splits\n", (long long)M, (long long)K,
                    (long long)N, tc::kMxConfigs[tc::kSkinnyMxConfig].name, splits);
          return tc::launch_mxfp8_splitk<tc::Mx_1cta>(args, out_dtype);
        }
      }
      config = (M <= tc::Mx_1cta_a32::A_ROWS) ? tc::kNarrowMxConfig : tc::kSkinnyMxConfig;
    } else {
      // 256-column tiles that fill at most half of one round of CTA pairs: 128-column tiles give
      // twice the units (256 x 8192 x 8192: 37.7 -> 29.7 us, 512 x 4096 x 4096: 22.6 -> 19.5 us; from
      // 64 tiles of 256 columns up the wider tile wins again)
      const int64_t units256 = ceil_div64(M, 2 * tc::kBlockM) * ceil_div64(N, tc::kBlockN);
      config = (4 * units256 <= (int64_t)di.sms) ? tc::kN128MxConfig : tc::kDefaultMxConfig;
      // several rounds of units: hand them out at run time (GEMM_B200_MXFP8_DYNAMIC=0: static schedule)
      static const bool dyn_ok = env_int("GEMM_B200_MXFP8_DYNAMIC", 1) != 0;
      // (and from K = 8192 up: with shorter tiles the static schedule is ~3 % faster, as in the BF16 kernel)
      if (dyn_ok && config == tc::kDefaultMxConfig && 2 * units256 > (int64_t)di.sms && K >= 8192) config = tc::kDynMxConfig;
      // a handful of tiles and a very long K (e.g. 256 x 65536 x 256): only K splits put the GPU to work
      const int64_t tiles_1cta = ceil_div64(M, tc::kBlockM) * ceil_div64(N, tc::kBlockN);
      // ... and so does a long K over a larger output when the estimate of tc::mxfp8_model_splits says so
      // (1024 x 32768 x 1024: 63.5 us on 256 x 128 pair tiles, 49.9 with four K ranges)
      const int model_splits = (K >= 16384 && N % 4 == 0) ? tc::mxfp8_model_splits(M, N, K, di.sms) : 1;
      if ((8 * tiles_1cta <= (int64_t)di.sms && K >= 16384 && N % 4 == 0) || model_splits > 1) {
        const int splits = model_splits > 1 ? model_splits : tc::auto_splits(M, N, K, di.sms);
        if (splits > 1) {
          if (int rc = tc::cached_scratch(di.dev, (size_t)splits * M * N * sizeof(float), &args.scratch, st)) return rc;
          if (args.scratch) {
            args.k_splits = splits;
            if (log_enabled())
              fprintf(stderr, "[gemm_b200] gemm_mxfp8 %lldx%lldx%lld -> %s, %d K splits\n", (long long)M, (long long)K,
                      (long long)N, tc::kMxConfigs[tc::kSkinnyMxConfig].name, splits);
            return tc::launch_mxfp8_splitk<tc::Mx_1cta>(args, out_dtype);
          }
        }
      }
    }
  }
  if (log_enabled())
    fprintf(stderr, "[gemm_b200] gemm_mxfp8 %lldx%lldx%lld -> %s\n", (long long)M, (long long)K, (long long)N,
            tc::kMxConfigs[config].name);
  return tc::kMxConfigs[config].launch[out_dtype](args);
}

extern "C" int gemm_b200_gemm_mxfp8_quant_out(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                                              void* Cq, void* SFC, int64_t M, int64_t N, int64_t K, void* stream) {
  using namespace gemm_b200;
  if (M < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_quant_out: negative size");
  if (M == 0 || N == 0) return GEMM_B200_OK;
  if (!Cq || !SFC || !Aq || !Bq || !SFA || !SFB) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_quant_out: null pointer");
  if (K <= 0 || K % 32 != 0 || N % 32 != 0)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_quant_out: K=%lld and N=%lld must be positive multiples of 32",
                (long long)K, (long long)N);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8_quant_out: a dimension exceeds 2^31-1");
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Bq) | reinterpret_cast<uintptr_t>(Cq) |
       reinterpret_cast<uintptr_t>(SFA) | reinterpret_cast<uintptr_t>(SFB) | reinterpret_cast<uintptr_t>(SFC)) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_mxfp8_quant_out: all pointers must be 16-byte aligned");
  tc::DeviceInfo di;
  if (int rc = tc::device_info(&di)) return rc;
  if (di.cc_major != 10)
    return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_mxfp8_quant_out: device has compute capability %d.x, need 10.x (sm_100a)", di.cc_major);
  tc::MxArgs args{Aq, SFA, Bq, SFB, Cq, M, N, K, /*ldc (bytes per row of Cq)*/ N, static_cast<cudaStream_t>(stream)};
  args.SFC = static_cast<uint8_t*>(SFC);
  return (M <= 128) ? tc::launch_mxfp8<tc::Mx_1cta, 2>(args) : tc::launch_mxfp8<tc::Mx_2cta_m_tma, 2>(args);
}

extern "C" int gemm_b200_gemm_mxfp8_auto_splits(int64_t M, int64_t N, int64_t K) {
  gemm_b200::tc::DeviceInfo di;
  if (gemm_b200::tc::device_info(&di)) return 1;
  return gemm_b200::tc::auto_splits(M, N, K, di.sms);
}

extern "C" size_t gemm_b200_gemm_mxfp8_splitk_scratch_bytes(int64_t M, int64_t N, int k_splits) {
  if (M <= 0 || N <= 0 || k_splits <= 1) return 0;
  return (size_t)k_splits * (size_t)M * (size_t)N * sizeof(float);
}

extern "C" int gemm_b200_gemm_mxfp8_splitk(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C,
                                           int64_t M, int64_t N, int64_t K, int64_t ldc, int out_dtype, int k_splits,
                                           void* scratch, size_t scratch_bytes, void* stream) {
  using namespace gemm_b200;
  if (k_splits < 1 || k_splits > 64) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk: k_splits %d not in [1, 64]", k_splits);
  if (k_splits == 1 || M == 0 || N == 0 || K == 0)
    return gemm_b200_gemm_mxfp8_cfg(Aq, SFA, Bq, SFB, C, M, N, K, ldc, out_dtype, tc::kSkinnyMxConfig, stream);
  // same argument checks as the unsplit entry point
  if (M < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk: negative size");
  if (out_dtype != GEMM_B200_OUT_BF16 && out_dtype != GEMM_B200_OUT_F32)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk: out_dtype %d", out_dtype);
  if (!C || !Aq || !Bq || !SFA || !SFB || !scratch) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk: null pointer");
  if (ldc < N) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk: ldc smaller than N");
  if (K % 32 != 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk: K=%lld is not a multiple of 32", (long long)K);
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8_splitk: a dimension exceeds 2^31-1");
  const int c_elem = out_dtype == GEMM_B200_OUT_F32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(Aq) | reinterpret_cast<uintptr_t>(Bq) | reinterpret_cast<uintptr_t>(C) |
       reinterpret_cast<uintptr_t>(SFA) | reinterpret_cast<uintptr_t>(SFB) | reinterpret_cast<uintptr_t>(scratch)) % 16 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_mxfp8_splitk: all pointers must be 16-byte aligned");
  if ((ldc * c_elem) % 16 != 0 || N % 8 != 0)
    return fail(GEMM_B200_ERR_ALIGNMENT, "gemm_mxfp8_splitk: ldc*sizeof(C) must be a multiple of 16 bytes and N of 8");
  const size_t need = gemm_b200_gemm_mxfp8_splitk_scratch_bytes(M, N, k_splits);
  if (scratch_bytes < need)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk: scratch holds %zu bytes, %zu needed", scratch_bytes, need);
  tc::DeviceInfo di;
  if (int rc = tc::device_info(&di)) return rc;
  if (di.cc_major != 10)
    return fail(GEMM_B200_ERR_UNSUPPORTED, "gemm_mxfp8_splitk: device has compute capability %d.x, need 10.x (sm_100a)", di.cc_major);
  tc::MxArgs args{Aq, SFA, Bq, SFB, C, M, N, K, ldc, static_cast<cudaStream_t>(stream)};
  args.k_splits = k_splits;
  args.scratch = static_cast<float*>(scratch);
  return tc::launch_mxfp8_splitk<tc::Mx_1cta>(args, out_dtype);
}
extern "C" int gemm_b200_gemm_mxfp8_cluster_splitk(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C,
                                                   int64_t M, int64_t N, int64_t K, int64_t ldc, int out_dtype, int k_splits,
                                                   void* stream) {
  using namespace gemm_b200;
  if (k_splits != 2 && k_splits != 4 && k_splits != 8)
    return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_cluster_splitk: k_splits %d is not 2, 4 or 8", k_splits);
  if (M <= 0 || N <= 0 || K <= 0)   // nothing to split: the plain entry point handles empty problems and K == 0
    return gemm_b200_gemm_mxfp8(Aq, SFA, Bq, SFB, C, M, N, K, ldc, out_dtype, stream);
  // the argument checks of the plain entry point, then the split (config -2 - k_splits selects it)
  return gemm_b200_gemm_mxfp8_cfg(Aq, SFA, Bq, SFB, C, M, N, K, ldc, out_dtype, -2 - k_splits, stream);
}

extern "C" int gemm_b200_gemm_mxfp8(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C, int64_t M,
                                    int64_t N, int64_t K, int64_t ldc, int out_dtype, void* stream) {
  return gemm_b200_gemm_mxfp8_cfg(Aq, SFA, Bq, SFB, C, M, N, K, ldc, out_dtype, -1, stream);
}
extern "C" int gemm_b200_gemm_mxfp8_num_configs(void) { return gemm_b200::tc::kNumMxConfigs; }
extern "C" const char* gemm_b200_gemm_mxfp8_config_name(int config) {
  if (config < 0 || config >= gemm_b200::tc::kNumMxConfigs) return "";
  return gemm_b200::tc::kMxConfigs[config].name;
}

// =========================================================================================
// Split-K MXFP8 GEMM on a scratch buffer that is part of the library image
// =========================================================================================
// The FP32 partial sums of the split-K path normally live in memory somebody allocates: the
// caller (gemm_b200_gemm_mxfp8_splitk) or the library on first use (gemm_b200_gemm_mxfp8).
// This entry point is for callers that can do neither on their call path: a serving loop that
// handed all of HBM to its own pool at start-up (a later cudaMalloc fails, and even when it
// succeeds it synchronises the whole device), or a plugin host whose execute callback forbids
// allocation.  The scratch is a fixed array in the library's device image, so every GPU that
// loads the library carries GEMM_B200_STATIC_SCRATCH_BYTES of it until the process exits.
namespace gemm_b200 {
namespace tc {

static __device__ __align__(256) float g_static_scratch[GEMM_B200_STATIC_SCRATCH_BYTES / sizeof(float)];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the
// address kernels can use comes from cudaGetSymbolAddress, looked up once per device with that
// device current.
static std::mutex g_static_mu;
static float* g_static_ptr[64] = {nullptr};

// First call on a device: besides the address look-up, load every kernel this entry point can
// launch (the split-K GEMM, the unsplit single-CTA GEMM for k_splits == 1, both reduce kernels) and
// opt them in to their shared-memory size, so that no later call on that device loads code,
// whichever output type it asks for.
static int static_scratch_for_current_device(float** out) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  std::lock_guard<std::mutex> lk(g_static_mu);
  const int slot = di.dev & 63;
  if (!g_static_ptr[slot]) {
    void* p = nullptr;
    GEMM_B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    int clusters = 0;
    if (int rc = persistent_clusters(gemm_mxfp8_kernel<Mx_1cta, 0>, 1, kMxThreads, Mx_1cta::SMEM_BYTES, di, &clusters)) return rc;
    if (int rc = persistent_clusters(gemm_mxfp8_kernel<Mx_1cta, 1>, 1, kMxThreads, Mx_1cta::SMEM_BYTES, di, &clusters)) return rc;
    cudaFuncAttributes fa;
    GEMM_B200_CUDA_TRY(cudaFuncGetAttributes(&fa, splitk_reduce_kernel<true>));
    GEMM_B200_CUDA_TRY(cudaFuncGetAttributes(&fa, splitk_reduce_kernel<false>));
    g_static_ptr[slot] = static_cast<float*>(p);
  }
  *out = g_static_ptr[slot];
  return GEMM_B200_OK;
}

}  // namespace tc
}  // namespace gemm_b200

extern "C" int gemm_b200_gemm_mxfp8_splitk_static(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                                                  void* C, int64_t M, int64_t N, int64_t K, int64_t ldc, int out_dtype,
                                                  int k_splits, void* stream) {
  using namespace gemm_b200;
  if (M < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk_static: negative size");
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
    return fail(GEMM_B200_ERR_TOO_LARGE, "gemm_mxfp8_splitk_static: a dimension exceeds 2^31-1");
  if (k_splits > 64) return fail(GEMM_B200_ERR_INVALID_ARG, "gemm_mxfp8_splitk_static: k_splits %d above 64", k_splits);
  if (k_splits <= 0) {
    // the library's own choice; the split path stores 8 columns at a time, other widths run unsplit
    k_splits = (N % 8 == 0) ? gemm_b200_gemm_mxfp8_auto_splits(M, N, K) : 1;
    // a choice that does not fit the built-in array is reduced until it does
    while (k_splits > 1 && gemm_b200_gemm_mxfp8_splitk_scratch_bytes(M, N, k_splits) > (size_t)GEMM_B200_STATIC_SCRATCH_BYTES)
      --k_splits;
  }
  const size_t need = gemm_b200_gemm_mxfp8_splitk_scratch_bytes(M, N, k_splits);   // M, N < 2^31, k_splits <= 64: no overflow
  if (need > (size_t)GEMM_B200_STATIC_SCRATCH_BYTES)
    return fail(GEMM_B200_ERR_TOO_LARGE,
                "gemm_mxfp8_splitk_static: %d splits of a %lld x %lld result need %zu bytes of scratch, the built-in "
                "buffer holds %zu; use gemm_b200_gemm_mxfp8_splitk with your own scratch",
                k_splits, (long long)M, (long long)N, need, (size_t)GEMM_B200_STATIC_SCRATCH_BYTES);
  float* scratch = nullptr;
  if (int rc = tc::static_scratch_for_current_device(&scratch)) return rc;
  return gemm_b200_gemm_mxfp8_splitk(Aq, SFA, Bq, SFB, C, M, N, K, ldc, out_dtype, k_splits, scratch,
                                     (size_t)GEMM_B200_STATIC_SCRATCH_BYTES, stream);
}

// =========================================================================================
// Self-test of the bounded-wait / status path
// =========================================================================================
namespace gemm_b200 {
namespace tc {

// One warp waits on an mbarrier that nothing ever arrives on.  The wait gives up after
// `limit_ns`, records {code, block, role = setup, stage = 777} in the status word and the kernel
// returns normally — the same path a real kernel takes when a pipeline wait runs out.
__global__ void __launch_bounds__(32) wait_timeout_selftest_kernel(unsigned long long limit_ns, int* returned_normally) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    fence_mbar_init();
  }
  __syncwarp();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(b, 0, kRoleSetup, 777, limit_ns);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  __syncwarp();
  if (threadIdx.x == 0) *returned_normally = ok ? 2 : 1;   // 1: the wait ran out and the kernel still got here
}

}  // namespace tc
}  // namespace gemm_b200

extern "C" int gemm_b200_selftest_wait_timeout(int64_t limit_us, int* device_flag, void* stream) {
  using namespace gemm_b200;
  if (limit_us < 1 || limit_us > 100000) return fail(GEMM_B200_ERR_INVALID_ARG, "selftest_wait_timeout: limit_us must be in [1, 100000]");
  if (!device_flag) return fail(GEMM_B200_ERR_INVALID_ARG, "selftest_wait_timeout: null flag pointer");
  tc::wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((unsigned long long)limit_us * 1000ull, device_flag);
  launch_counter().fetch_add(1, std::memory_order_relaxed);
  GEMM_B200_CUDA_TRY(cudaGetLastError());
  return GEMM_B200_OK;
}

#ifdef GEMM_B200_TRACE
// Tuning builds only: copies the stage timeline of the last tensor-core launch out (see trace_stamp).
extern "C" int gemm_b200_trace_read(unsigned long long* out, int blocks) {
  using namespace gemm_b200;
  if (!out || blocks < 1 || blocks > tc::kTraceBlocks) return fail(GEMM_B200_ERR_INVALID_ARG, "trace_read: bad arguments");
  GEMM_B200_CUDA_TRY(cudaDeviceSynchronize());
  GEMM_B200_CUDA_TRY(cudaMemcpyFromSymbol(out, tc::g_trace, sizeof(unsigned long long) * tc::kTraceSlots * blocks));
  return GEMM_B200_OK;
}
#endif

#ifdef GEMM_B200_DEBUG
// Bounds-checking build only: reads and clears the status word of the tensor-core side's checks
// (direct-store epilogues, split-K partial sums and their reduction, the row-wise quantiser) and
// sets the test knob `shrink`.  {code, block, site, byte offset}; code 0 = clean.
extern "C" int gemm_b200_debug_bounds_tc(int32_t out[4], long long shrink) { return gemm_b200::dbg::read_bounds(out, shrink); }
#endif
