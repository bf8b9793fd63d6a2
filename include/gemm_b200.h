/*
 * gemm_b200 — C-ABI of the B200 (sm_100a) GEMM library.
 *
 * Every entry point takes plain pointers and sizes; none takes a torch type.
 * Unless a comment says otherwise all data pointers are DEVICE pointers on the
 * current CUDA device, matrices are row-major, leading dimensions are counted
 * in elements, and `stream` is a `cudaStream_t` passed as `void*` (NULL = the
 * legacy default stream, which is what the reference launches on).
 *
 * Every function returns 0 on success or a negative GEMM_B200_ERR_* code;
 * `gemm_b200_last_error()` then holds a human-readable reason for the calling
 * thread.  Launches are asynchronous, like the reference's.
 *
 * The reference interface each entry point stands in for is cited by its path
 * inside the danielvegamyhre/gemm project.
 */
#ifndef GEMM_B200_H_
#define GEMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GEMM_B200_VERSION 100

/* status codes */
#define GEMM_B200_OK                 0
#define GEMM_B200_ERR_INVALID_ARG   -1  /* null pointer, negative size, ld too small       */
#define GEMM_B200_ERR_ALIGNMENT     -2  /* pointer / leading dimension not aligned enough  */
#define GEMM_B200_ERR_UNSUPPORTED   -3  /* device is not sm_100, or shape class not built  */
#define GEMM_B200_ERR_CUDA          -4  /* a CUDA runtime / driver call failed             */
#define GEMM_B200_ERR_TIMEOUT       -5  /* a bounded device-side wait ran out              */
#define GEMM_B200_ERR_TOO_LARGE     -6  /* size exceeds a documented maximum               */
#define GEMM_B200_ERR_BOUNDS        -7  /* bounds-checking build: an access fell outside its matrix (skipped, not made) */

/* element types of C for the tensor-core paths */
#define GEMM_B200_OUT_BF16 0
#define GEMM_B200_OUT_F32  1

/* layout of the B operand for the tensor-core paths */
#define GEMM_B200_B_ROW_MAJOR_KN 0   /* B[K,N], N contiguous: the reference's layout            */
#define GEMM_B200_B_ROW_MAJOR_NK 1   /* B given as its transpose Bt[N,K], K contiguous          */

/* -------------------------------------------------------------------------
 * FP32 CUDA-core GEMM:  C[M,N] = A[M,K] @ B[K,N], beta = 0, C overwritten.
 *
 * Replaces, with one kernel family, all three reference launchers:
 *   launch_naive_gemm(float*,float*,float*,int M,int N,int K)   naive/naive_1.cu:17-24
 *   launch_gemm(float*,float*,float*,int M,int N,int K)         shared/shared_2.cu:59-66
 *   launch_gemm(float*,float*,float*,int M,int N,int K)         blocktile_1d/blocktile_1d.cu:70-82
 * Same semantics as those kernels: one FP32 accumulator per element of C,
 * k strictly ascending, fused multiply-add, denormals flushed (the reference
 * is built with --use_fast_math), so the result is bit-identical to theirs.
 * Any M, N, K >= 0 is accepted (K == 0 writes zeros).  Addressing is 64-bit.
 * ------------------------------------------------------------------------- */
int gemm_b200_sgemm_f32(const float* A, const float* B, float* C,
                        int64_t M, int64_t N, int64_t K,
                        int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* Same, with the tile configuration forced (tests and tuning sweeps).
 * `config` indexes the table printed by gemm_b200_sgemm_f32_config_name();
 * -1 = the library's heuristic. */
int gemm_b200_sgemm_f32_cfg(const float* A, const float* B, float* C,
                            int64_t M, int64_t N, int64_t K,
                            int64_t lda, int64_t ldb, int64_t ldc,
                            int config, void* stream);
/* Strided-batched form: `batch` independent problems of one shape,
 *   C_i[M,N] = A_i[M,K] @ B_i[K,N],   X_i = X + i * stride_x (strides in elements),
 * each with the arithmetic of gemm_b200_sgemm_f32 (bit-identical to one call per problem).
 * The reference multiplies one pair of matrices per call (naive/naive.cpp:6-22); this is the
 * loop a caller would write around it, as one launch.  stride_a == 0 or stride_b == 0 shares
 * that operand between the problems; the C matrices must not overlap. */
int gemm_b200_sgemm_f32_batched(const float* A, const float* B, float* C, int64_t batch,
                                int64_t M, int64_t N, int64_t K,
                                int64_t lda, int64_t ldb, int64_t ldc,
                                int64_t stride_a, int64_t stride_b, int64_t stride_c, void* stream);
int gemm_b200_sgemm_f32_num_configs(void);
const char* gemm_b200_sgemm_f32_config_name(int config);

/* -------------------------------------------------------------------------
 * BF16 tensor-core GEMM (tcgen05, FP32 accumulation in TMEM):
 *   C[M,N] = A[M,K] @ B,  A bf16 row-major, C bf16 or f32 row-major.
 * The reference has no BF16 path; this extends the same operator
 * (naive/naive.cpp:6-22: M = A.size(0), K = A.size(1), N = B.size(1), C
 * overwritten and returned) to BF16 operands.
 * Requirements: pointers 16-byte aligned; lda, ldb (and ldc for bf16 output)
 * multiples of 8 elements (ldc multiple of 4 for f32 output).
 * ------------------------------------------------------------------------- */
int gemm_b200_gemm_bf16(const void* A, const void* B, void* C,
                        int64_t M, int64_t N, int64_t K,
                        int64_t lda, int64_t ldb, int64_t ldc,
                        int b_layout, int out_dtype, void* stream);

/* Same with the kernel variant forced (-1 = heuristic). */
int gemm_b200_gemm_bf16_cfg(const void* A, const void* B, void* C,
                            int64_t M, int64_t N, int64_t K,
                            int64_t lda, int64_t ldb, int64_t ldc,
                            int b_layout, int out_dtype, int config, void* stream);
int gemm_b200_gemm_bf16_num_configs(void);
const char* gemm_b200_gemm_bf16_config_name(int config);

/* Split-K form for problems with few output tiles and a long K (e.g. 256 x 256 x 65536): every
 * tile is cut into `k_splits` ranges of K whose FP32 partial sums go to `scratch`
 * ([k_splits][M][N] floats, device memory, 16-byte aligned, at least
 * gemm_b200_gemm_bf16_splitk_scratch_bytes() bytes) and are then summed in ascending split order
 * into C by a second kernel.  k_splits == 1 runs the plain kernel and never splits.
 * gemm_b200_gemm_bf16() takes the split path by itself with the count of
 * gemm_b200_gemm_bf16_auto_splits() (1 = it does not split), on scratch the library owns: one
 * buffer per (device, stream), so calls on different streams may overlap and calls on one stream
 * are ordered anyway (at most 256 MiB per buffer).  The first split call on a stream, and a later one that needs a larger
 * buffer, allocate (cudaMalloc; growing also frees, which waits for the device); during stream
 * capture such a call runs unsplit instead.  The library keeps buffers for the 32 most recently
 * used streams.  N % 4 == 0.  The reference always walks K inside one thread
 * (naive/naive_1.cu:9-12); it has no counterpart. */
int gemm_b200_gemm_bf16_splitk(const void* A, const void* B, void* C,
                               int64_t M, int64_t N, int64_t K,
                               int64_t lda, int64_t ldb, int64_t ldc,
                               int b_layout, int out_dtype, int k_splits,
                               void* scratch, size_t scratch_bytes, void* stream);
size_t gemm_b200_gemm_bf16_splitk_scratch_bytes(int64_t M, int64_t N, int k_splits);
int gemm_b200_gemm_bf16_auto_splits(int64_t M, int64_t N, int64_t K);

/* Split-K inside a thread-block cluster, for problems with few 128 x 128 output tiles: the
 * k_splits (2, 4 or 8) CTAs of a cluster each multiply one range of K for the same tile and
 * combine their FP32 partial sums through distributed shared memory, in ascending order of the
 * ranges: one launch, no scratch memory, no allocation, results independent of timing.
 * Every range must hold at least one block of 64 k.  gemm_b200_gemm_bf16() takes this path by
 * itself for problems of at most 32 tiles (clusters of 4; of 8 for at most 8 tiles) whose K
 * leaves every CTA at least 512 and is not so long that the scratch-based split with many more
 * ranges wins.  The reference walks K inside one thread (naive/naive_1.cu:9-12); no counterpart. */
int gemm_b200_gemm_bf16_cluster_splitk(const void* A, const void* B, void* C,
                                       int64_t M, int64_t N, int64_t K,
                                       int64_t lda, int64_t ldb, int64_t ldc,
                                       int b_layout, int out_dtype, int k_splits, void* stream);

/* Strided-batched form: `batch` independent problems of one shape in one launch,
 *   C_i[M,N] = A_i[M,K] @ B_i,   X_i = X + i * stride_x (strides in elements).
 * The reference multiplies one pair of matrices per call (naive/naive.cpp:6-22);
 * this is the loop a caller would write around it, scheduled as one persistent
 * grid over all (matrix, tile) pairs.  stride_a == 0 or stride_b == 0 shares that
 * operand between the problems (e.g. one weight matrix B for every A_i).
 * Requirements as above; stride_a and stride_b multiples of 8 elements,
 * stride_c * sizeof(C) a multiple of 16 bytes, the C matrices must not overlap. */
int gemm_b200_gemm_bf16_batched(const void* A, const void* B, void* C, int64_t batch,
                                int64_t M, int64_t N, int64_t K,
                                int64_t lda, int64_t ldb, int64_t ldc,
                                int64_t stride_a, int64_t stride_b, int64_t stride_c,
                                int b_layout, int out_dtype, void* stream);

/* Transposed-A form: A is given as its transpose At[K, M] row-major (lda >= M, M contiguous),
 *   C[M,N] = At^T @ B,
 * the layout in which an activation matrix X[tokens, features] enters the weight-gradient product
 * X^T dY without a transposing copy.  The reference assumes row-major A[M,K] silently
 * (naive/naive.cpp:15-17); no counterpart.  Requirements as gemm_b200_gemm_bf16 (lda a multiple
 * of 8).  Few output tiles with a long K are cut into K ranges on library-owned scratch as in
 * gemm_b200_gemm_bf16 (same per-(device, stream) ownership).  Results are bit-identical to
 * gemm_b200_gemm_bf16 on a transposed copy of At whenever both take the same tile shape. */
int gemm_b200_gemm_bf16_at(const void* At, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                           int64_t lda, int64_t ldb, int64_t ldc,
                           int b_layout, int out_dtype, void* stream);

/* Grouped (ragged) form: `groups` problems that share N and K but have their own row count,
 *   C[rows of group g, :] = A[rows of group g, :] @ B_g,   B_g = B + g * stride_b,
 * where the groups' rows follow one another in one tall A [sum m_sizes, K] (lda) and one tall
 * C [sum m_sizes, N] (ldc): the layout of tokens sorted by expert in a mixture-of-experts layer.
 * m_sizes is a HOST array of `groups` row counts (zero allowed).  One launch per 64 groups, each
 * walking all (group, tile) pairs; bit-identical to one gemm_b200_gemm_bf16_cfg call per group with
 * variant "1cta_128x256x64_s4_direct".  The reference multiplies one pair of matrices per call
 * (naive/naive.cpp:6-22); no counterpart. */
int gemm_b200_gemm_bf16_grouped(const void* A, const void* B, void* C, int64_t groups, const int64_t* m_sizes,
                                int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t stride_b, int64_t ldc,
                                int b_layout, int out_dtype, void* stream);

/* -------------------------------------------------------------------------
 * MXFP8 (OCP microscaling): e4m3 data with one UE8M0 scale per 32 consecutive
 * K elements.  No counterpart in the reference; same operator semantics as
 * above (naive/naive.cpp:6-22) on quantised operands.
 *
 * gemm_b200_quantize_mxfp8 quantises X (bf16) along K.
 *   transposed_in = 0: X is [rows, K] row-major (ldx >= K)          -> used for A[M,K]
 *   transposed_in = 1: X is [K, rows] row-major (ldx >= rows)       -> used for B[K,N]
 * Outputs: Xq  e4m3 [rows, K] row-major, K contiguous (ld = K);
 *          SF  UE8M0 bytes in the packed layout described by
 *              gemm_b200_mxfp8_scale_offset() — gemm_b200_mxfp8_scale_bytes(rows, K) bytes.
 * Recipe: per block amax -> e = floor(log2(amax)) - 8 (amax == 0 or a block
 * of denormals -> e clamped to -127), scale byte = e + 127,
 * q = saturate_e4m3(x * 2^-e) with round-to-nearest-even.  K % 32 == 0.
 * ------------------------------------------------------------------------- */
int gemm_b200_quantize_mxfp8(const void* X_bf16, int64_t rows, int64_t K, int64_t ldx,
                             int transposed_in, void* Xq_e4m3, void* SF_ue8m0, void* stream);
size_t gemm_b200_mxfp8_scale_bytes(int64_t rows, int64_t K);
/* Byte offset of the scale of (row, K-block kb) inside the packed scale buffer. */
size_t gemm_b200_mxfp8_scale_offset(int64_t rows, int64_t K, int64_t row, int64_t kb);

/* C[M,N] = dequant(Aq,SFA)[M,K] @ dequant(Bq,SFB)[N,K]^T, FP32 accumulation. */
int gemm_b200_gemm_mxfp8(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                         void* C, int64_t M, int64_t N, int64_t K, int64_t ldc,
                         int out_dtype, void* stream);
int gemm_b200_gemm_mxfp8_cfg(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                             void* C, int64_t M, int64_t N, int64_t K, int64_t ldc,
                             int out_dtype, int config, void* stream);
/* Same GEMM with a quantising epilogue: C is rounded to bf16 and quantised to MXFP8 along its
 * columns inside the kernel (e4m3 to Cq[M,N], ld = N; scales to SFC in the packed layout of
 * gemm_b200_mxfp8_scale_offset(M, N, row, n / 32), gemm_b200_mxfp8_scale_bytes(M, N) bytes), so
 * the result can feed the next GEMM as its A operand without a bf16 round trip through memory.
 * Bit-identical to gemm_b200_gemm_mxfp8 (bf16 output) followed by gemm_b200_quantize_mxfp8.
 * N % 32 == 0.  No counterpart in the reference. */
int gemm_b200_gemm_mxfp8_quant_out(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                                   void* Cq, void* SFC, int64_t M, int64_t N, int64_t K, void* stream);

/* Split-K form for problems with few output tiles (skinny M): every tile is cut into `k_splits`
 * ranges of K whose FP32 partial sums go to `scratch` ([k_splits][M][N] floats, device memory,
 * 16-byte aligned, at least gemm_b200_gemm_mxfp8_splitk_scratch_bytes() bytes) and are then
 * summed in ascending split order into C by a second kernel.  gemm_b200_gemm_mxfp8() takes this
 * path by itself for M <= 128 and for a handful of tiles with K >= 16384, with the split count
 * of gemm_b200_gemm_mxfp8_auto_splits(), and for taller problems with K >= 16384 where its estimate
 * of the call time favours K ranges, on library-owned scratch kept per (device, stream) under
 * the rules given for gemm_b200_gemm_bf16_splitk above (at most 256 MiB of it).  No counterpart in
 * the reference. */
int gemm_b200_gemm_mxfp8_splitk(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                                void* C, int64_t M, int64_t N, int64_t K, int64_t ldc, int out_dtype,
                                int k_splits, void* scratch, size_t scratch_bytes, void* stream);
size_t gemm_b200_gemm_mxfp8_splitk_scratch_bytes(int64_t M, int64_t N, int k_splits);

/* Grouped form (tokens sorted by expert in a mixture-of-experts layer, in MXFP8): `groups` problems
 * that share N and K,
 *   C[rows of group g, :] = A[rows of group g, :] @ B_g,
 * with the groups' rows following one another in one tall Aq [sum m_sizes, K] (its packed scales SFA
 * cover the tall matrix) and one tall C (ldc).  Bq holds the `groups` quantised matrices [N, K] one
 * after another and SFB their packed scale buffers one after another
 * (gemm_b200_mxfp8_scale_bytes(N, K) bytes each).  m_sizes is a HOST array; every entry must be a
 * multiple of 256 (zero allowed): scales are packed per 128 rows and a CTA pair owns 256 rows, so
 * the caller pads each group.  One launch per 64 groups; each group's rows equal, bit for bit,
 * gemm_b200_gemm_mxfp8_cfg on that group alone with variant "2cta_256x256x128_s5_maskcommit_tmastore".
 * The reference multiplies one pair of FP32 matrices per call (naive/naive.cpp:6-22); no counterpart. */
int gemm_b200_gemm_mxfp8_grouped(const void* Aq, const void* SFA, const void* Bq, const void* SFB, void* C,
                                 int64_t groups, const int64_t* m_sizes, int64_t N, int64_t K, int64_t ldc,
                                 int out_dtype, void* stream);

/* Split-K inside a thread-block cluster (see gemm_b200_gemm_bf16_cluster_splitk): k_splits = 2, 4
 * or 8 CTAs per 128 x 128 tile, partial sums combined through distributed shared memory, one
 * launch, no scratch.  Every range must hold at least one block of 128 k.  gemm_b200_gemm_mxfp8()
 * takes this path by itself for problems of at most 32 tiles.  No counterpart in the reference. */
int gemm_b200_gemm_mxfp8_cluster_splitk(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                                        void* C, int64_t M, int64_t N, int64_t K, int64_t ldc, int out_dtype,
                                        int k_splits, void* stream);

/* The same split-K GEMM for callers that cannot allocate device memory where they call it: a
 * serving loop that gave all of HBM to its own pool at start-up (cudaMalloc would fail there, and
 * it synchronises the device even when it succeeds), or a plugin host that forbids allocation
 * inside its execute callback.  It has no counterpart in the reference.
 *   - The FP32 partial sums go to a GEMM_B200_STATIC_SCRATCH_BYTES array built into the library's
 *     device image; every GPU that loads the library holds that much until the process exits.
 *   - Limit: k_splits * M * N * 4 bytes must fit; larger problems get GEMM_B200_ERR_TOO_LARGE and
 *     should use gemm_b200_gemm_mxfp8_splitk.  k_splits <= 0 picks the library's split count,
 *     lowered as far as needed to fit (down to 1 = unsplit, which needs no scratch).
 *   - The call performs no cudaMalloc / cudaFree and calls no allocating library routine.
 *   - The first call on each device does the one-time set-up: it looks the array's device address
 *     up and loads every kernel the entry point can launch (both output types), so later calls on
 *     that device load nothing.  Make that first call before starting any stream capture on that
 *     device and outside the region where allocation is forbidden (loading code takes memory).
 *   - All calls on a device share the one array, which keeps whatever the last call left there
 *     (nothing in it has to start at zero: every value read is written by the same call first).
 *     Two calls whose kernels can overlap on the GPU (different streams) race on it; keep them on
 *     one stream or order them with events. */
#define GEMM_B200_STATIC_SCRATCH_BYTES (16u << 20)
int gemm_b200_gemm_mxfp8_splitk_static(const void* Aq, const void* SFA, const void* Bq, const void* SFB,
                                       void* C, int64_t M, int64_t N, int64_t K, int64_t ldc,
                                       int out_dtype, int k_splits, void* stream);
int gemm_b200_gemm_mxfp8_auto_splits(int64_t M, int64_t N, int64_t K);
int gemm_b200_gemm_mxfp8_num_configs(void);
const char* gemm_b200_gemm_mxfp8_config_name(int config);

/* -------------------------------------------------------------------------
 * Host-buffer entry points: the same operators on HOST pointers.  Each call
 * copies the operands to a cached device workspace, launches, copies C back
 * and synchronises before returning — what a caller holding host arrays sees
 * end to end.  (The reference's wrapper, naive/naive.cpp:6-22, only accepts
 * device tensors; its tests create them with device='cuda'.)
 * ------------------------------------------------------------------------- */
int gemm_b200_sgemm_f32_host(const float* hA, const float* hB, float* hC,
                             int64_t M, int64_t N, int64_t K);
int gemm_b200_gemm_bf16_host(const void* hA, const void* hB, void* hC,
                             int64_t M, int64_t N, int64_t K, int b_layout, int out_dtype);
/* Frees the cached workspace of the current device. */
int gemm_b200_release_workspace(void);

/* -------------------------------------------------------------------------
 * Library state
 * ------------------------------------------------------------------------- */
/* Reads (and clears) the device-side status word that bounded waits write when
 * they give up.  Synchronises `stream`.  0 = clean, GEMM_B200_ERR_TIMEOUT
 * otherwise; `detail`, if not NULL, receives {code, block, role, stage}.
 * The word is per device and sticky: once a wait has given up, every later
 * tensor-core kernel on that device skips its work (its C is garbage) while the
 * launching calls keep returning GEMM_B200_OK, until this function has been
 * called.  Call it wherever a result is consumed.  The host-buffer entry points
 * call it themselves before returning. */
int gemm_b200_check_status(void* stream, int32_t detail[4]);
/* Self-test of the bounded-wait machinery: launches one warp that waits `limit_us` microseconds
 * (1 .. 100000) on a barrier nothing arrives on, then records the give-up in the status word and
 * returns normally (writing 1 to *device_flag, an int in device memory).  A following
 * gemm_b200_check_status() must report GEMM_B200_ERR_TIMEOUT with role 4, stage 777, and clears
 * the status.  Nothing hangs: the kernel ends by itself after `limit_us`.  The reference has no
 * error path at all (naive/naive_1.cu:23 launches and returns). */
int gemm_b200_selftest_wait_timeout(int64_t limit_us, int* device_flag, void* stream);
const char* gemm_b200_last_error(void);
int gemm_b200_version(void);
/* 1 if device `dev` can run the tensor-core paths (compute capability 10.x). */
int gemm_b200_device_supported(int dev);
/* Number of kernels this library has launched in this process. */
int64_t gemm_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* GEMM_B200_H_ */
