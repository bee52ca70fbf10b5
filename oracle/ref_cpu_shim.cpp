// TEST INFRASTRUCTURE ONLY.  C-linkage doors onto the reference's own CPU quantiser
// (legacy_modules/quantization/src/impl/nf4_impl.cpp and nf4_dq_impl.cpp), which is
// compiled unmodified, from where it lies in the reference tree, into oracle/_ref.
// This file holds no arithmetic: it calls the reference's functions and copies their
// results into caller buffers so that ctypes can reach them.
#include <quantization/impl/nf4_dq_impl.hpp>
#include <quantization/impl/nf4_impl.hpp>

#include <cstdint>
#include <cstring>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// nf4_compress (nf4_impl.cpp:92): scales[ceil(n/64)], data[ceil(n/2)]
int ref_nf4_quantize(const float *x, unsigned long long n, float *scales, uint8_t *data) {
    nf4_array_t *arr = nullptr;
    if (nf4_compress(x, n, &arr) != 0 || arr == nullptr) return 1;
    std::memcpy(scales, arr->block_scales, arr->num_blocks * sizeof(float));
    std::memcpy(data, arr->data, (n + 1) / 2);
    free_nf4_array(arr);
    return 0;
}

// nf4_compress + nf4_decompress round trip (what tests/quantization_cuda/test_nf4_cuda.cu compares)
int ref_nf4_roundtrip(const float *x, unsigned long long n, float *out) {
    nf4_array_t *arr = nullptr;
    if (nf4_compress(x, n, &arr) != 0 || arr == nullptr) return 1;
    const int rc = nf4_decompress(arr, out);
    free_nf4_array(arr);
    return rc;
}

// nf4_dq_compress (nf4_dq_impl.cpp:227)
int ref_nf4dq_quantize(const float *x, unsigned long long n, float *dq, uint8_t *scale_codes, uint8_t *data) {
    nf4_dq_array_t *arr = nullptr;
    if (nf4_dq_compress(x, n, &arr) != 0 || arr == nullptr) return 1;
    *dq = arr->dq_scale;
    std::memcpy(scale_codes, arr->block_scales, arr->num_blocks);
    std::memcpy(data, arr->data, (n + 1) / 2);
    free_nf4_dq_array(arr);
    return 0;
}

int ref_nf4dq_roundtrip(const float *x, unsigned long long n, float *out) {
    nf4_dq_array_t *arr = nullptr;
    if (nf4_dq_compress(x, n, &arr) != 0 || arr == nullptr) return 1;
    const int rc = nf4_dq_decompress(arr, out);
    free_nf4_dq_array(arr);
    return rc;
}

// decompress from raw parts (nf4_impl.cpp:137, nf4_dq_impl.cpp:243)
int ref_nf4_dequantize(const float *scales, const uint8_t *data, unsigned long long n, float *out) {
    nf4_array_t *arr = allocate_nf4_array(n, DEFAULT_NF4_BLOCK_SIZE);
    if (!arr) return 1;
    std::memcpy(arr->block_scales, scales, arr->num_blocks * sizeof(float));
    std::memcpy(arr->data, data, (n + 1) / 2);
    const int rc = nf4_decompress(arr, out);
    free_nf4_array(arr);
    return rc;
}

int ref_nf4dq_dequantize(float dq, const uint8_t *scale_codes, const uint8_t *data, unsigned long long n, float *out) {
    nf4_dq_array_t *arr = allocate_nf4_dq_array(n, DEFAULT_NF4_DQ_BLOCK_SIZE);
    if (!arr) return 1;
    arr->dq_scale = dq;
    std::memcpy(arr->block_scales, scale_codes, arr->num_blocks);
    std::memcpy(arr->data, data, (n + 1) / 2);
    const int rc = nf4_dq_decompress(arr, out);
    free_nf4_dq_array(arr);
    return rc;
}

int ref_cpu_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// OpenMP threads for the calls that follow (a launcher may have exported OMP_NUM_THREADS=1 to the process)
void ref_cpu_set_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

}  // extern "C"
