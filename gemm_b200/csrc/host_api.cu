// Host-buffer entry points: the operators of this library for callers that hold HOST arrays.
// Operands go to a cached per-device workspace, C comes back, and the call returns after
// everything has finished.  Large problems are cut into row slabs of A / C so the upload of
// slab i+1, the GEMM of slab i and the download of slab i-1 overlap on three streams
// (B is uploaded once, first).  Pinned host memory makes the copies asynchronous; pageable
// memory still works, just without the overlap.
#include <mutex>

#include "common.cuh"

namespace gemm_b200 {
namespace host {

struct Workspace {
  void* ptr = nullptr;
  size_t bytes = 0;
  cudaStream_t s_in = nullptr, s_mm = nullptr, s_out = nullptr;
  static constexpr int kMaxSlabs = 64;
  cudaEvent_t up[kMaxSlabs] = {}, done[kMaxSlabs] = {};
  cudaEvent_t b_up = nullptr;
  bool ready = false;
};

static std::mutex g_mu;
static Workspace g_ws[64];

static int workspace(size_t bytes, Workspace** out) {
  int dev = 0;
  GEMM_B200_CUDA_TRY(cudaGetDevice(&dev));
  Workspace& w = g_ws[dev & 63];
  if (!w.ready) {
    GEMM_B200_CUDA_TRY(cudaStreamCreateWithFlags(&w.s_in, cudaStreamNonBlocking));
    GEMM_B200_CUDA_TRY(cudaStreamCreateWithFlags(&w.s_mm, cudaStreamNonBlocking));
    GEMM_B200_CUDA_TRY(cudaStreamCreateWithFlags(&w.s_out, cudaStreamNonBlocking));
    for (int i = 0; i < Workspace::kMaxSlabs; ++i) {
      GEMM_B200_CUDA_TRY(cudaEventCreateWithFlags(&w.up[i], cudaEventDisableTiming));
      GEMM_B200_CUDA_TRY(cudaEventCreateWithFlags(&w.done[i], cudaEventDisableTiming));
    }
    GEMM_B200_CUDA_TRY(cudaEventCreateWithFlags(&w.b_up, cudaEventDisableTiming));
    w.ready = true;
  }
  if (w.bytes < bytes) {
    if (w.ptr) GEMM_B200_CUDA_TRY(cudaFree(w.ptr));
    w.ptr = nullptr;
    w.bytes = 0;
    GEMM_B200_CUDA_TRY(cudaMalloc(&w.ptr, bytes));
    w.bytes = bytes;
  }
  *out = &w;
  return GEMM_B200_OK;
}

static size_t align_up(size_t x) { return (x + 255) & ~(size_t)255; }

// Queues everything: B up, then per slab A up -> GEMM -> C down, on the three streams.
template <class Launch>
static int enqueue(Workspace* w, const void* hA, const void* hB, void* hC, int64_t M, int64_t N, int64_t K, size_t ea,
                   size_t eb, size_t ec, char* dA, char* dB, char* dC, int64_t slab, int nslabs, Launch launch) {
  if (K > 0) GEMM_B200_CUDA_TRY(cudaMemcpyAsync(dB, hB, (size_t)K * N * eb, cudaMemcpyHostToDevice, w->s_in));
  GEMM_B200_CUDA_TRY(cudaEventRecord(w->b_up, w->s_in));
  GEMM_B200_CUDA_TRY(cudaStreamWaitEvent(w->s_mm, w->b_up, 0));
  for (int i = 0; i < nslabs; ++i) {
    const int64_t r0 = (int64_t)i * slab, rows = (M - r0 < slab) ? (M - r0) : slab;
    if (K > 0)
      GEMM_B200_CUDA_TRY(cudaMemcpyAsync(dA + (size_t)r0 * K * ea, static_cast<const char*>(hA) + (size_t)r0 * K * ea,
                                         (size_t)rows * K * ea, cudaMemcpyHostToDevice, w->s_in));
    GEMM_B200_CUDA_TRY(cudaEventRecord(w->up[i], w->s_in));
    GEMM_B200_CUDA_TRY(cudaStreamWaitEvent(w->s_mm, w->up[i], 0));
    if (int rc = launch(dA + (size_t)r0 * K * ea, dB, dC + (size_t)r0 * N * ec, rows, w->s_mm)) return rc;
    GEMM_B200_CUDA_TRY(cudaEventRecord(w->done[i], w->s_mm));
    GEMM_B200_CUDA_TRY(cudaStreamWaitEvent(w->s_out, w->done[i], 0));
    GEMM_B200_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(hC) + (size_t)r0 * N * ec, dC + (size_t)r0 * N * ec,
                                       (size_t)rows * N * ec, cudaMemcpyDeviceToHost, w->s_out));
  }
  return GEMM_B200_OK;
}

// launch(dA, dB, dC, rows, stream) runs the GEMM of `rows` rows of A on device pointers.
// check_tc: the launch runs tensor-core kernels, whose bounded waits report through the device
// status word; it is read (and cleared) before returning, so a wait that gave up comes back as
// GEMM_B200_ERR_TIMEOUT instead of a silently wrong hC.
template <class Launch>
static int run(const void* hA, const void* hB, void* hC, int64_t M, int64_t N, int64_t K, size_t ea, size_t eb,
               size_t ec, bool check_tc, Launch launch) {
  if (M < 0 || N < 0 || K < 0) return fail(GEMM_B200_ERR_INVALID_ARG, "host gemm: negative size");
  if (M == 0 || N == 0) return GEMM_B200_OK;
  if (!hC || (K > 0 && (!hA || !hB))) return fail(GEMM_B200_ERR_INVALID_ARG, "host gemm: null pointer");
  std::lock_guard<std::mutex> lk(g_mu);
  const size_t a_bytes = align_up((size_t)M * K * ea), b_bytes = align_up((size_t)K * N * eb);
  const size_t c_bytes = align_up((size_t)M * N * ec);
  Workspace* w = nullptr;
  if (int rc = workspace(a_bytes + b_bytes + c_bytes + 256, &w)) return rc;
  char* dA = static_cast<char*>(w->ptr);
  char* dB = dA + a_bytes;
  char* dC = dB + b_bytes;

  // slabs of at least ~32 MiB of A+C traffic, multiples of 256 rows, at most kMaxSlabs
  int64_t slab = M;
  const size_t row_bytes = (size_t)K * ea + (size_t)N * ec;
  if ((size_t)M * row_bytes > ((size_t)64 << 20)) {
    slab = (int64_t)((((size_t)32 << 20) + row_bytes - 1) / row_bytes);
    slab = ((slab + 255) / 256) * 256;
    if (ceil_div64(M, slab) > Workspace::kMaxSlabs) slab = ((ceil_div64(M, Workspace::kMaxSlabs) + 255) / 256) * 256;
  }
  const int nslabs = (int)ceil_div64(M, slab);

  const int rc = enqueue(w, hA, hB, hC, M, N, K, ea, eb, ec, dA, dB, dC, slab, nslabs, launch);
  // Success or not, nothing queued above may outlive this call: copies still in flight read and
  // write the caller's host buffers, and the next call reuses the workspace.
  const cudaError_t e_out = cudaStreamSynchronize(w->s_out);
  const cudaError_t e_mm = cudaStreamSynchronize(w->s_mm);
  const cudaError_t e_in = cudaStreamSynchronize(w->s_in);
  if (rc != GEMM_B200_OK) return rc;   // the message of the first failure stays in last_error
  GEMM_B200_CUDA_TRY(e_out);
  GEMM_B200_CUDA_TRY(e_mm);
  GEMM_B200_CUDA_TRY(e_in);
  if (check_tc) return gemm_b200_check_status(w->s_mm, nullptr);
  return GEMM_B200_OK;
}

}  // namespace host
}  // namespace gemm_b200

extern "C" int gemm_b200_sgemm_f32_host(const float* hA, const float* hB, float* hC, int64_t M, int64_t N, int64_t K) {
  return gemm_b200::host::run(hA, hB, hC, M, N, K, 4, 4, 4, /*check_tc=*/false,
                              [&](const void* dA, const void* dB, void* dC, int64_t rows, cudaStream_t st) {
                                return gemm_b200_sgemm_f32(static_cast<const float*>(dA), static_cast<const float*>(dB),
                                                           static_cast<float*>(dC), rows, N, K, K, N, N, st);
                              });
}

extern "C" int gemm_b200_gemm_bf16_host(const void* hA, const void* hB, void* hC, int64_t M, int64_t N, int64_t K,
                                        int b_layout, int out_dtype) {
  const size_t ec = out_dtype == GEMM_B200_OUT_F32 ? 4 : 2;
  const int64_t ldb = b_layout == GEMM_B200_B_ROW_MAJOR_KN ? N : K;
  return gemm_b200::host::run(hA, hB, hC, M, N, K, 2, 2, ec, /*check_tc=*/true,
                              [&](const void* dA, const void* dB, void* dC, int64_t rows, cudaStream_t st) {
                                return gemm_b200_gemm_bf16(dA, dB, dC, rows, N, K, K, ldb, N, b_layout, out_dtype, st);
                              });
}

extern "C" int gemm_b200_release_workspace(void) {
  using namespace gemm_b200;
  std::lock_guard<std::mutex> lk(host::g_mu);
  int dev = 0;
  GEMM_B200_CUDA_TRY(cudaGetDevice(&dev));
  host::Workspace& w = host::g_ws[dev & 63];
  if (w.ptr) GEMM_B200_CUDA_TRY(cudaFree(w.ptr));
  w.ptr = nullptr;
  w.bytes = 0;
  return GEMM_B200_OK;
}
