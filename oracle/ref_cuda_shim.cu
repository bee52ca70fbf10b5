// TEST INFRASTRUCTURE ONLY.  C-linkage doors onto the reference's own CUDA build (its
// five .cu files compiled unmodified, from where they lie in the reference tree, into
// oracle/_ref/libref_cuda.so for sm_100).  It is the parity oracle on a GPU box for the
// stages that have no CPU twin in the reference (per-row top-k, randomized SVD,
// reconstruct, the whole pipeline).  This file holds no arithmetic of its own.
#include <bitsqz_llm.hpp>
#include <quantization_cuda/quantization_cuda.cuh>
#include <reconstruct_lowrank_cuda/reconstruct_lowrank_cuda.cuh>
#include <svd_lowrank_cuda/svd_lowrank_cuda.cuh>
#include <topk_cuda.cuh>

#include <cstdint>
#include <exception>

extern "C" {

// ---- public API (include/bitsqz_llm.hpp:95-141) -----------------------------------
int ref_compress_initialize(uint16_t rows, uint16_t cols, float outlier, float err, int ranks, int niters,
                            int uv, int s, int q, int loc) {
    return bitsqz_llm_compress_initialize(rows, cols, outlier, err, ranks, niters,
                                          (quantization_method_t)uv, (quantization_method_t)s,
                                          (quantization_method_t)q, (bitsqz_llm_input_location_t)loc);
}
void ref_compress_release(void) { bitsqz_llm_compress_release(); }
int ref_decompress_initialize(uint16_t rows, uint16_t cols, float outlier, float err, int ranks, int uv, int s, int q) {
    return bitsqz_llm_decompress_initialize(rows, cols, outlier, err, ranks, (quantization_method_t)uv,
                                            (quantization_method_t)s, (quantization_method_t)q);
}
void ref_decompress_release(void) { bitsqz_llm_decompress_release(); }
int ref_compress(const float *x, bitsqz_llm_array_t **out, bitsqz_llm_compress_profile_t *prof) {
    return bitsqz_llm_compress(x, out, prof);
}
int ref_decompress(const bitsqz_llm_array_t *c, float *d_dst, uint32_t n) { return bitsqz_llm_decompress(c, d_dst, n); }
uint64_t ref_get_packed_size(const bitsqz_llm_array_t *c) { return bitsqz_llm_get_packed_size(c); }
bitsqz_llm_array_t *ref_load_from_buffer(const void *b, uint64_t n) { return load_bitsqz_llm_from_buffer(b, n); }
void ref_free(bitsqz_llm_array_t *c) { bitsqz_llm_free(c); }

// ---- top-k module (modules/topk_cuda/include/topk_cuda.cuh:47-107) ------------------
int ref_topk_num_columns(uint16_t cols, float ratio) {
    try { return topk_compute_num_topk_columns(cols, ratio); } catch (const std::exception &) { return -1; }
}

// topk_extraction (separation == 0) or topk_separation (separation != 0) on a device matrix
int ref_topk_rows(float *d_x, uint16_t rows, uint16_t cols, uint16_t k, int separation, uint16_t *d_idx, float *d_val) {
    TopkCUDAContext ctx{};
    try {
        topk_initialize(&ctx, rows, cols);
        topk_array_t arr{};
        topk_bind_array(&arr, rows, cols, k, d_idx, d_val);
        if (separation) topk_separation(&ctx, d_x, &arr); else topk_extraction(&ctx, d_x, &arr);
        topk_release(&ctx);
        return 0;
    } catch (const std::exception &) { topk_release(&ctx); return 1; }
}

int ref_topk_apply(const uint16_t *d_idx, const float *d_val, uint16_t rows, uint16_t cols, uint16_t k, float *d_dense) {
    TopkCUDAContext ctx{};
    try {
        topk_initialize(&ctx, rows, cols);
        topk_array_t arr{};
        topk_bind_array(&arr, rows, cols, k, const_cast<uint16_t *>(d_idx), const_cast<float *>(d_val));
        topk_apply(&ctx, &arr, d_dense);
        topk_release(&ctx);
        return 0;
    } catch (const std::exception &) { topk_release(&ctx); return 1; }
}

// ---- quantiser module (quantization_cuda.cuh:58-112) -------------------------------
int ref_quant_compress(int method, const float *d_x, uint64_t n, float *d_scales_f32, uint8_t *d_scales_u8,
                       float *d_dq, uint8_t *d_data) {
    QuantizationCUDAContext ctx{};
    try {
        quantization_cuda_initialize(&ctx, n);
        quantization_cuda_array_t arr{};
        if (method == NF4) quantization_cuda_bind_nf4_array(&arr, n, d_scales_f32, d_data);
        else quantization_cuda_bind_nf4_dq_array(&arr, n, d_dq, d_scales_u8, d_data);
        quantization_cuda_compress(&ctx, d_x, &arr);
        quantization_cuda_release(&ctx);
        return 0;
    } catch (const std::exception &) { quantization_cuda_release(&ctx); return 1; }
}

int ref_quant_decompress(int method, float *d_scales_f32, uint8_t *d_scales_u8, float *d_dq, uint8_t *d_data,
                         uint64_t n, float *d_out) {
    QuantizationCUDAContext ctx{};
    try {
        quantization_cuda_initialize(&ctx, n);
        quantization_cuda_array_t arr{};
        if (method == NF4) quantization_cuda_bind_nf4_array(&arr, n, d_scales_f32, d_data);
        else quantization_cuda_bind_nf4_dq_array(&arr, n, d_dq, d_scales_u8, d_data);
        quantization_cuda_decompress(&ctx, &arr, d_out);
        quantization_cuda_release(&ctx);
        return 0;
    } catch (const std::exception &) { quantization_cuda_release(&ctx); return 1; }
}

// ---- randomized SVD (svd_lowrank_cuda.cuh:54-68) ------------------------------------
int ref_svd_initialize(int m, int n, int q, int niter, unsigned long long warmup_seed) {
    try { svd_lowrank_cuda_initialize(m, n, q, niter, warmup_seed); return 0; } catch (const std::exception &) { return 1; }
}
int ref_svd_run(const float *d_A, float *d_U, float *d_S, float *d_V, unsigned long long seed) {
    try { svd_lowrank_cuda(d_A, d_U, d_S, d_V, seed); return 0; } catch (const std::exception &) { return 1; }
}
void ref_svd_release(void) { svd_lowrank_cuda_release(); }

// ---- reconstruct (reconstruct_lowrank_cuda.cuh:64-78) -------------------------------
int ref_reconstruct(const float *d_U, const float *d_S, const float *d_V, int m, int n, int k, float *d_out) {
    ReconstructLowrankCUDAContext ctx{};
    try {
        reconstruct_lowrank_cuda_initialize(&ctx, m, n, k);
        reconstruct_lowrank_cuda(&ctx, d_U, d_S, d_V, d_out);
        reconstruct_lowrank_cuda_release(&ctx);
        return 0;
    } catch (const std::exception &) { reconstruct_lowrank_cuda_release(&ctx); return 1; }
}

}  // extern "C"
