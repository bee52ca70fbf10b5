// Host-side launchers of the sm_100a kernels.  Internal to the library: the public surfaces
// are include/bitsqz_llm.hpp (C++ interface of the reference) and include/bitsqz_llm_c.h
// (C ABI).  Every launcher enqueues work on `stream` and returns without synchronising.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace bsq {

// ---- NF4 / NF4_DQ over a flat array (bsq_quant.cu) ----------------------------------------
// d_deq_out (nullable): also write the dequantised values, which is what the reference's
// compress path feeds into its error-correction stage (src/bitsqz_llm.cu:506-511).
cudaError_t nf4_quantize(const float *d_x, uint64_t n, float *d_scales, uint8_t *d_data, float *d_deq_out, int sm_count,
                         cudaStream_t stream);
size_t nf4dq_scratch_bytes(uint64_t n);
cudaError_t nf4dq_quantize(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                           float *d_deq_out, void *d_scratch, int sm_count, cudaStream_t stream);
// Variant for callers that must not allocate: scratch is a fixed array inside the library.
uint64_t nf4dq_static_max_elements();
cudaError_t nf4dq_quantize_static(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                                  int sm_count, cudaStream_t stream);
cudaError_t nf4_dequantize(const float *d_scales, const uint8_t *d_data, uint64_t n, float *d_out, int sm_count,
                           cudaStream_t stream);
cudaError_t nf4dq_dequantize(const float *d_dq, const uint8_t *d_scale_codes, const uint8_t *d_data, uint64_t n,
                             float *d_out, int sm_count, cudaStream_t stream);
// Dequantise a rows x cols matrix and add a row-wise top-k list in one pass; d_scales (NF4) or d_dq + d_scale_codes (NF4_DQ).
cudaError_t nf4_dequantize_add_topk(const float *d_scales, const float *d_dq, const uint8_t *d_scale_codes, const uint8_t *d_data,
                                    uint32_t rows, uint32_t cols, const uint16_t *d_idx, const float *d_val, uint32_t k,
                                    float *d_out, unsigned *d_status, int sm_count, cudaStream_t stream);

// ---- per-row top-k (bsq_topk.cu) ------------------------------------------------------------
// k = (uint16)roundf(cols * ratio) clamped to cols, at least 1 for ratio > 0; -1 for a ratio
// outside [0, 1] (reference topk_cuda.cu:53-69).
int topk_num_columns(uint16_t cols, float ratio);

// Per row: the k entries of largest |x| ordered by (|x| descending, column ascending), NaN
// ranking below every number.  d_idx / d_val are [rows][k].  d_residual (nullable): receives
// the row with the selected entries set to +0.0f; may alias d_in (in-place separation).
// d_status: device word that receives kStatus* bits.
// d_bound (nullable device word) receives, where the shared-memory path runs (*bound_written says so), the bits of the
// largest k-th |x| over the rows: an upper bound of every |x| that is left in d_residual.
cudaError_t topk_rows(const float *d_in, float *d_residual, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                      float *d_val, unsigned *d_status, int sm_count, cudaStream_t stream, unsigned *d_bound = nullptr,
                      bool *bound_written = nullptr);

// dense[row, idx] += val for every entry; indices >= cols are skipped and reported in d_status.
cudaError_t topk_apply(const uint16_t *d_idx, const float *d_val, uint32_t rows, uint32_t cols, uint32_t k,
                       float *d_dense, unsigned *d_status, cudaStream_t stream);

// ---- fused front end of the no-SVD path (bsq_frontend.cu) -----------------------------------
// outlier separation + NF4 or NF4_DQ of the remainder, reading the input once from HBM (the
// NF4_DQ second pass re-reads it through L2).  Needs cols % 64 == 0, k <= 256 and a row that
// fits shared memory; frontend_supported() says whether a shape qualifies.
bool frontend_supported(uint32_t rows, uint32_t cols, uint32_t k);
size_t frontend_scratch_bytes(uint32_t rows, uint32_t cols);
// method: 11 = NF4 (d_scales_f32 used), 10 = NF4_DQ (d_dq, d_scale_codes used).
cudaError_t frontend_quantize(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                              float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                              void *d_scratch, unsigned *d_status, int sm_count, cudaStream_t stream,
                              cudaEvent_t *events = nullptr);   // events[3]: before pass 1, between, after pass 2

// ---- residual / error helpers ---------------------------------------------------------------
// e = a - b and *d_flag |= 1 when some |e| > FLT_EPSILON (reference src/bitsqz_llm.cu:164-184).
cudaError_t residual_error(const float *d_a, const float *d_b, uint64_t n, float *d_e, unsigned *d_flag, int sm_count,
                           cudaStream_t stream);

int device_sm_count();
// A block for a packed object that the caller will release with bitsqz_llm_free: page-locked from the library's pool
// when one can be had, plain heap memory otherwise (bsq_api.cu).
void *host_block_take(size_t bytes);
bool topk_rows_fit_smem(const void *d_in, const void *d_residual, uint32_t cols, uint32_t k);

// ---- randomized low-rank SVD and reconstruction (bsq_svd.cu, bsq_gemm.cu) -------------------
// Replaces svd_lowrank_cuda_initialize / svd_lowrank_cuda / svd_lowrank_cuda_release
// (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:541-581) and reconstruct_lowrank_cuda
// (modules/reconstruct_lowrank_cuda/src/reconstruct_lowrank_cuda.cu:153-171).
// C[M x N] = opA[M x K] * opB[K x N] in FP32 (bsq_gemm.cu).  a_kmajor: opA(i,kk) = A[i*lda+kk], else A[kk*lda+i];
// b_kmajor: opB(kk,j) = B[j*ldb+kk], else B[kk*ldb+j].  kscale (nullable) scales opA along K.  minuend (nullable):
// C = minuend - product, *flag |= 1 when some |C| > FLT_EPSILON.  workspace (nullable) enables a deterministic K split.
// Skinny products (N = 16..256, no fused epilogue) run on the tensor cores (bsq_gemm_tc.cu); `status` (nullable device
// word) receives kStatusBarrierTimeout if one of that kernel's bounded waits gives up.
cudaError_t gemm(bool a_kmajor, bool b_kmajor, const float *A, long lda, const float *B, long ldb, float *C, long ldc, int M,
                 int N, int K, const float *kscale, const float *minuend, long ldm, unsigned *flag, unsigned *status,
                 float *workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream, const unsigned *a_absmax_bits = nullptr,
                 float b_bound = 0.0f);
// The same with the kernel choice explicit: allow_tensor_cores = false keeps the product on the FP32 pipes.
cudaError_t gemm_select(bool allow_tensor_cores, bool a_kmajor, bool b_kmajor, const float *A, long lda, const float *B, long ldb,
                        float *C, long ldc, int M, int N, int K, const float *kscale, const float *minuend, long ldm,
                        unsigned *flag, unsigned *status, float *workspace, size_t workspace_bytes, int sm_count,
                        cudaStream_t stream, const unsigned *a_absmax_bits = nullptr, float b_bound = 0.0f);
// (a_absmax_bits: device word with the bits of an upper bound of |A|, b_bound: an upper bound of |B| known on the host,
// 0 = none -- with a bound on |A| the 256-column products split their operands into FP16 halves, bsq_gemm_tc.cuh)

struct SvdWorkspace;
// sums `count` floats at `buf` over all ranks, enqueued on `stream`
typedef cudaError_t (*SvdAllReduce)(void *ctx, float *buf, size_t count, cudaStream_t stream);
SvdWorkspace *svd_workspace_create(int m, int n, int k, int niter, int sm_count);
SvdWorkspace *svd_workspace_create_sharded(int m_local, int n, int k, int niter, int sm_count, SvdAllReduce allreduce,
                                           void *allreduce_ctx, int m_total);
void svd_workspace_destroy(SvdWorkspace *ws);
// A row-major m x n -> U (m x k row-major), S (k, descending), V (n x k row-major).
// The random matrix is the first N x k normals of cuRAND's XORWOW sequence of `seed`, starting `offset` values in.
cudaError_t svd_lowrank(SvdWorkspace *ws, const float *d_A, float *d_U, float *d_S, float *d_V,
                        unsigned long long seed, unsigned *d_status, cudaStream_t stream, unsigned long long offset = 0,
                        const unsigned *d_abs_bound = nullptr);
// (d_abs_bound, nullable: device word with the bits of an upper bound of |A|, e.g. from topk_rows; without it the call
// makes a pass over A for the largest |A| where it needs one.)
// Optional timing of a call's products with the big matrix (kind 0) and, row-sharded, its all-reduces (kind 1).
cudaError_t svd_workspace_profile(SvdWorkspace *ws, bool on);
int svd_workspace_spans(SvdWorkspace *ws, float *ms, int *kinds, int capacity);
// For calls made with d_status == nullptr: waits for the stream and returns an error if a bounded wait gave up.
cudaError_t svd_workspace_finish(SvdWorkspace *ws, cudaStream_t stream);
// out = (U diag(S)) V^T, row-major m x n.  d_minuend (nullable): write minuend - out instead and
// OR 1 into *d_flag when some |difference| > FLT_EPSILON.
// d_status (nullable): device word that receives kStatusBarrierTimeout if a bounded wait of the product kernel gives up
// (the output is then incomplete).
// d_workspace (nullable, reconstruct_workspace_bytes, 128-byte aligned): room for V and U diag(S) split once into the
// tensor cores' operand format, shared by all tiles; without it every tile splits its pieces itself.
size_t reconstruct_workspace_bytes(int m, int n, int k);
cudaError_t reconstruct_lowrank(const float *d_U, const float *d_S, const float *d_V, int m, int n, int k,
                                const float *d_minuend, float *d_out, unsigned *d_flag, unsigned *d_status, float *d_workspace,
                                size_t workspace_bytes, int sm_count, cudaStream_t stream);

}  // namespace bsq
