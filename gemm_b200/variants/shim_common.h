// Shared body of the three reference-named PyTorch extension wrappers.
//
// The reference wrappers (naive/naive.cpp:6-22, shared/shared.cpp:6-22,
// blocktile_1d/blocktile_1d.cpp:6-22) take (A, B, C), read M = A.size(0), K = A.size(1),
// N = B.size(1), pass raw float pointers to their launcher and return C itself.  This wrapper
// keeps that contract — C is written in place and returned, the launch is asynchronous — and
// adds the checks the reference leaves out (device, dtype, rank, shapes, contiguity) plus the
// current-stream / current-device handling a multi-stream or multi-GPU caller needs.
#pragma once
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "../../include/gemm_b200.h"

namespace gemm_b200_shim {

inline torch::Tensor gemm_into(torch::Tensor A, torch::Tensor B, torch::Tensor C) {
  TORCH_CHECK(A.is_cuda() && B.is_cuda() && C.is_cuda(), "gemm_b200: A, B and C must be CUDA tensors");
  TORCH_CHECK(A.get_device() == B.get_device() && A.get_device() == C.get_device(),
              "gemm_b200: A, B and C must be on the same device");
  TORCH_CHECK(A.scalar_type() == torch::kFloat32 && B.scalar_type() == torch::kFloat32 &&
                  C.scalar_type() == torch::kFloat32,
              "gemm_b200: expected float32 tensors");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && C.dim() == 2, "gemm_b200: expected 2-D tensors");
  const int64_t M = A.size(0), K = A.size(1), N = B.size(1);
  TORCH_CHECK(B.size(0) == K, "gemm_b200: A is [", M, ",", K, "] but B is [", B.size(0), ",", N, "]");
  TORCH_CHECK(C.size(0) == M && C.size(1) == N, "gemm_b200: C must be [", M, ",", N, "]");
  // Row-major with unit column stride, as the reference kernels index (naive/naive_1.cu:11,13).
  // A silent .contiguous() copy of C would break the out-parameter aliasing, so refuse instead.
  auto row_major = [](const torch::Tensor& t) { return t.size(1) <= 1 || t.stride(1) == 1; };
  TORCH_CHECK(row_major(A) && row_major(B) && row_major(C), "gemm_b200: tensors must be row-major (unit column stride)");
  const int64_t lda = A.size(0) > 1 ? A.stride(0) : K, ldb = B.size(0) > 1 ? B.stride(0) : N,
                ldc = C.size(0) > 1 ? C.stride(0) : N;
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream();
  const int rc = gemm_b200_sgemm_f32(A.data_ptr<float>(), B.data_ptr<float>(), C.data_ptr<float>(), M, N, K, lda, ldb,
                                     ldc, stream);
  TORCH_CHECK(rc == 0, "gemm_b200_sgemm_f32 failed (", rc, "): ", gemm_b200_last_error());
  return C;
}

// Allocating form: C = A @ B.
inline torch::Tensor matmul(torch::Tensor A, torch::Tensor B) {
  TORCH_CHECK(A.dim() == 2 && B.dim() == 2, "gemm_b200: expected 2-D tensors");
  auto C = torch::empty({A.size(0), B.size(1)}, A.options());
  return gemm_into(A, B, C);
}

}  // namespace gemm_b200_shim
