// extern "C" surface of the library (include/bitsqz_llm_c.h): thin forwards onto the C++
// interface and onto the stage launchers.  No logic lives here beyond argument translation.
#include <bitsqz_llm.hpp>
#include <bitsqz_llm_c.h>

#include "bsq_internal.hpp"

using namespace bsq;

static inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }
static inline int rc(cudaError_t e) {
    if (e != cudaSuccess) cudaGetLastError();
    return e == cudaSuccess ? 0 : 1;
}

extern "C" {

int bsq_compress_initialize(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio,
                            float error_correction_topk_ratio, int svd_ranks, int svd_niters, int svd_uv_format,
                            int svd_s_format, int quantization_only_format, int input_location) {
    return bitsqz_llm_compress_initialize(num_rows, num_columns, outlier_topk_ratio, error_correction_topk_ratio,
                                          svd_ranks, svd_niters, (quantization_method_t)svd_uv_format,
                                          (quantization_method_t)svd_s_format,
                                          (quantization_method_t)quantization_only_format,
                                          (bitsqz_llm_input_location_t)input_location);
}
void bsq_compress_release(void) { bitsqz_llm_compress_release(); }
int bsq_decompress_initialize(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio,
                              float error_correction_topk_ratio, int svd_ranks, int svd_uv_format, int svd_s_format,
                              int quantization_only_format) {
    return bitsqz_llm_decompress_initialize(num_rows, num_columns, outlier_topk_ratio, error_correction_topk_ratio,
                                            svd_ranks, (quantization_method_t)svd_uv_format,
                                            (quantization_method_t)svd_s_format,
                                            (quantization_method_t)quantization_only_format);
}
void bsq_decompress_release(void) { bitsqz_llm_decompress_release(); }
int bsq_compress(const float *row_major_matrix, struct bitsqz_llm_array **out, void *profile) {
    return bitsqz_llm_compress(row_major_matrix, out, static_cast<bitsqz_llm_compress_profile_t *>(profile));
}
int bsq_decompress(const struct bitsqz_llm_array *compressed, float *d_dst, uint32_t dst_num_elements) {
    return bitsqz_llm_decompress(compressed, d_dst, dst_num_elements);
}
uint64_t bsq_get_packed_size(const struct bitsqz_llm_array *compressed) { return bitsqz_llm_get_packed_size(compressed); }
struct bitsqz_llm_array *bsq_load_from_buffer(const void *buffer, uint64_t buffer_size) {
    return load_bitsqz_llm_from_buffer(buffer, buffer_size);
}
void bsq_free(struct bitsqz_llm_array *compressed) { bitsqz_llm_free(compressed); }

int bsq_topk_num_columns(uint16_t num_columns, float topk_ratio) { return topk_num_columns(num_columns, topk_ratio); }
int bsq_topk_rows(const float *d_in, float *d_residual, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                  float *d_val, uint32_t *d_status, void *stream) {
    return rc(topk_rows(d_in, d_residual, rows, cols, k, d_idx, d_val, d_status, device_sm_count(), as_stream(stream)));
}
int bsq_topk_apply(const uint16_t *d_idx, const float *d_val, uint32_t rows, uint32_t cols, uint32_t k, float *d_dense,
                   uint32_t *d_status, void *stream) {
    return rc(topk_apply(d_idx, d_val, rows, cols, k, d_dense, d_status, as_stream(stream)));
}

int bsq_nf4_quantize(const float *d_x, uint64_t n, float *d_scales, uint8_t *d_data, float *d_deq_out, void *stream) {
    if (!d_x || !n || !d_scales || !d_data) return 1;
    return rc(nf4_quantize(d_x, n, d_scales, d_data, d_deq_out, device_sm_count(), as_stream(stream)));
}
size_t bsq_nf4dq_scratch_bytes(uint64_t n) { return nf4dq_scratch_bytes(n); }
int bsq_nf4dq_quantize(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                       float *d_deq_out, void *d_scratch, void *stream) {
    if (!d_x || !n || !d_dq || !d_scale_codes || !d_data || !d_scratch) return 1;
    return rc(nf4dq_quantize(d_x, n, d_dq, d_scale_codes, d_data, d_deq_out, d_scratch, device_sm_count(), as_stream(stream)));
}
uint64_t bsq_nf4dq_quantize_static_max_elements(void) { return nf4dq_static_max_elements(); }
int bsq_nf4dq_quantize_static(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                              void *stream) {
    if (!d_x || !d_dq || !d_scale_codes || !d_data) return 1;
    if (n == 0 || n > nf4dq_static_max_elements()) return 1;      // beyond the built-in scratch: use bsq_nf4dq_quantize
    return rc(nf4dq_quantize_static(d_x, n, d_dq, d_scale_codes, d_data, device_sm_count(), as_stream(stream)));
}
int bsq_nf4_dequantize(const float *d_scales, const uint8_t *d_data, uint64_t n, float *d_out, void *stream) {
    if (!d_scales || !d_data || !n || !d_out) return 1;
    return rc(nf4_dequantize(d_scales, d_data, n, d_out, device_sm_count(), as_stream(stream)));
}
int bsq_nf4dq_dequantize(const float *d_dq, const uint8_t *d_scale_codes, const uint8_t *d_data, uint64_t n,
                         float *d_out, void *stream) {
    if (!d_dq || !d_scale_codes || !d_data || !n || !d_out) return 1;
    return rc(nf4dq_dequantize(d_dq, d_scale_codes, d_data, n, d_out, device_sm_count(), as_stream(stream)));
}

int bsq_dequantize_add_topk(int method, const float *d_scales_f32, const float *d_dq, const uint8_t *d_scale_codes,
                            const uint8_t *d_data, uint32_t rows, uint32_t cols, const uint16_t *d_idx, const float *d_val,
                            uint32_t k, float *d_out, uint32_t *d_status, void *stream) {
    if (method != 10 && method != 11) return 1;
    return rc(nf4_dequantize_add_topk(method == 11 ? d_scales_f32 : nullptr, method == 10 ? d_dq : nullptr,
                                      method == 10 ? d_scale_codes : nullptr, d_data, rows, cols, d_idx, d_val, k, d_out, d_status,
                                      device_sm_count(), as_stream(stream)));
}

int bsq_frontend_supported(uint32_t rows, uint32_t cols, uint32_t k) { return frontend_supported(rows, cols, k) ? 1 : 0; }
size_t bsq_frontend_scratch_bytes(uint32_t rows, uint32_t cols) { return frontend_scratch_bytes(rows, cols); }
int bsq_frontend_quantize(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                          float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                          void *d_scratch, uint32_t *d_status, void *stream) {
    return rc(frontend_quantize(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data,
                                d_scratch, d_status, device_sm_count(), as_stream(stream)));
}

int bsq_frontend_quantize_timed(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                                float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                                void *d_scratch, uint32_t *d_status, void *stream, float *ms_pass) {
    if (!ms_pass) return 1;
    cudaEvent_t ev[3] = {nullptr, nullptr, nullptr};
    for (auto &e : ev)
        if (cudaEventCreate(&e) != cudaSuccess) return 1;
    int r = rc(frontend_quantize(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data,
                                 d_scratch, d_status, device_sm_count(), as_stream(stream), ev));
    r |= rc(cudaEventSynchronize(ev[2]));
    if (r == 0) {
        r |= rc(cudaEventElapsedTime(&ms_pass[0], ev[0], ev[1]));
        r |= rc(cudaEventElapsedTime(&ms_pass[1], ev[1], ev[2]));
    }
    for (auto &e : ev) cudaEventDestroy(e);
    return r;
}

int bsq_residual_error(const float *d_a, const float *d_b, uint64_t n, float *d_e, uint32_t *d_flag, void *stream) {
    return rc(residual_error(d_a, d_b, n, d_e, d_flag, device_sm_count(), as_stream(stream)));
}

int bsq_svd_lowrank(const float *d_A, int m, int n, int k, int niter, unsigned long long seed, float *d_U, float *d_S,
                    float *d_V, void *stream) {
    if (!d_A || !d_U || !d_S || !d_V || m <= 0 || n <= 0 || k <= 0 || niter < 0) return 1;
    SvdWorkspace *ws = svd_workspace_create(m, n, k, niter, device_sm_count());
    if (!ws) return 1;
    const cudaError_t e = svd_lowrank(ws, d_A, d_U, d_S, d_V, seed, nullptr, as_stream(stream));
    const cudaError_t s = svd_workspace_finish(ws, as_stream(stream));  // the workspace dies with this call
    svd_workspace_destroy(ws);
    return rc(e) | rc(s);
}
int bsq_svd_lowrank_at(const float *d_A, int m, int n, int k, int niter, unsigned long long seed, unsigned long long offset,
                       float *d_U, float *d_S, float *d_V, void *stream) {
    if (!d_A || !d_U || !d_S || !d_V || m <= 0 || n <= 0 || k <= 0 || niter < 0) return 1;
    SvdWorkspace *ws = svd_workspace_create(m, n, k, niter, device_sm_count());
    if (!ws) return 1;
    const cudaError_t e = svd_lowrank(ws, d_A, d_U, d_S, d_V, seed, nullptr, as_stream(stream), offset);
    const cudaError_t s = svd_workspace_finish(ws, as_stream(stream));
    svd_workspace_destroy(ws);
    return rc(e) | rc(s);
}
int bsq_gemm(int a_kmajor, int b_kmajor, const float *d_A, long lda, const float *d_B, long ldb, float *d_C, long ldc, int M,
             int N, int K, float *d_workspace, size_t workspace_bytes, int allow_tensor_cores, uint32_t *d_status, void *stream) {
    if (!d_A || !d_B || !d_C || M <= 0 || N <= 0 || K <= 0) return 1;
    return rc(gemm_select(allow_tensor_cores != 0, a_kmajor != 0, b_kmajor != 0, d_A, lda, d_B, ldb, d_C, ldc, M, N, K, nullptr,
                          nullptr, 0, nullptr, d_status, d_workspace, workspace_bytes, device_sm_count(), as_stream(stream)));
}
int bsq_gemm_bounded(int a_kmajor, int b_kmajor, const float *d_A, long lda, const float *d_B, long ldb, float *d_C, long ldc, int M,
                     int N, int K, float *d_workspace, size_t workspace_bytes, const uint32_t *d_a_absmax_bits, uint32_t *d_status,
                     void *stream) {
    if (!d_A || !d_B || !d_C || !d_a_absmax_bits || M <= 0 || N <= 0 || K <= 0) return 1;
    return rc(gemm_select(true, a_kmajor != 0, b_kmajor != 0, d_A, lda, d_B, ldb, d_C, ldc, M, N, K, nullptr, nullptr, 0, nullptr,
                          d_status, d_workspace, workspace_bytes, device_sm_count(), as_stream(stream), d_a_absmax_bits));
}
int bsq_reconstruct(const float *d_U, const float *d_S, const float *d_V, int m, int n, int k, const float *d_minuend,
                    float *d_out, uint32_t *d_flag, uint32_t *d_status, void *stream) {
    if (!d_U || !d_S || !d_V || !d_out || m <= 0 || n <= 0 || k <= 0) return 1;
    if (d_minuend && !d_flag) return 1;
    return rc(reconstruct_lowrank(d_U, d_S, d_V, m, n, k, d_minuend, d_out, d_flag, d_status, nullptr, 0, device_sm_count(), as_stream(stream)));
}

const char *bsq_build_info(void) { return "bitsqz_llm sm_100a " __DATE__; }

}  // extern "C"
