// bitsqz_llm -- public C++ interface of the compress/decompress hot path.
//
// This header declares exactly the interface of the reference library
// (include/bitsqz_llm.hpp:17-141 of DandinPower/BitSqueeze-LLM): the same enum values,
// the same struct layouts (24-byte sections, 200-byte array header, 56-byte profile) and
// the same nine C++-linkage functions, so that the shared library built from this
// repository exports the same mangled symbols and existing callers relink unchanged.
// The layouts are pinned by the static_asserts at the bottom of this file.
#pragma once

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32)
#  if defined(BITSQZ_LLM_EXPORTS)
#    define BITSQZ_LLM_API __declspec(dllexport)
#  else
#    define BITSQZ_LLM_API __declspec(dllimport)
#  endif
#else
#  define BITSQZ_LLM_API
#endif

// Storage format of one section.  Only quantization_NONE, NF4 and NF4_DQ are accepted by
// the initialisers (reference: src/bitsqz_llm.cu:144-146); the other enumerators exist so
// that the integer values stay those of the reference (include/bitsqz_llm.hpp:17-33).
#ifndef BITSQZ_LLM_QUANTIZATION_METHOD_T_DEFINED
#define BITSQZ_LLM_QUANTIZATION_METHOD_T_DEFINED
typedef enum {
    quantization_NONE = -1,                     // keep the section in FP32
    quantization_INVALID = quantization_NONE,   // older spelling of the same value
    Q8_0 = 0, Q4_0 = 1, Q2_K = 2, BF16 = 3, FP16 = 4, FP8 = 5, FP4 = 6,
    MXFP8 = 7, MXFP4 = 8, NVFP4 = 9,
    NF4_DQ = 10,                                // NF4 codes, E4M3 block scales, one FP32 scale
    NF4 = 11,                                   // NF4 codes, FP32 block scales
    Q2_K_FAST = 12,
} quantization_method_t;
#endif

// What a section's bytes are (reference include/bitsqz_llm.hpp:36-41).
typedef enum {
    BITSQZ_SECTION_NONE = 0,    // absent
    BITSQZ_SECTION_FP32 = 1,    // raw little-endian floats
    BITSQZ_SECTION_QUANT = 2,   // 48-byte quantiser header + block scales + nibbles
    BITSQZ_SECTION_TOPK = 3,    // 8-byte header + u16 column indices + f32 values
} bitsqz_section_storage_t;

// Where the matrix handed to bitsqz_llm_compress lives (reference :43-46).
typedef enum {
    BITSQZ_LLM_INPUT_HOST = 0,
    BITSQZ_LLM_INPUT_DEVICE = 1,
} bitsqz_llm_input_location_t;

// One entry of the section table (reference :48-53).  `offset` is relative to `payload`.
typedef struct {
    uint64_t offset;
    uint64_t size;
    uint8_t storage;            // bitsqz_section_storage_t
    uint8_t reserved[7];
} bitsqz_section_t;

// Header of a compressed matrix (reference :55-83).  compress/load return this struct and
// its payload as ONE heap block: payload == (uint8_t *)this + sizeof(bitsqz_llm_array_t),
// and copying bitsqz_llm_get_packed_size() bytes from `this` serialises the object.
typedef struct bitsqz_llm_array {
    uint16_t num_rows;
    uint16_t num_columns;
    uint32_t num_elements;

    float outlier_topk_ratio;
    float error_correction_topk_ratio;

    int16_t svd_ranks;          // as configured (< 1: no SVD)
    int16_t svd_niters;
    int16_t effective_rank;     // clamp(svd_ranks, 1, min(rows, cols)), or 0 without SVD
    int16_t reserved0;

    quantization_method_t svd_uv_format;
    quantization_method_t svd_s_format;
    quantization_method_t quantization_only_format;
    int32_t reserved1;

    uint32_t flags;             // bit0 SVD sections, bit1 outlier top-k, bit2 error top-k

    bitsqz_section_t section_u;
    bitsqz_section_t section_s;
    bitsqz_section_t section_v;
    bitsqz_section_t section_direct;
    bitsqz_section_t section_outlier_topk;
    bitsqz_section_t section_error_topk;

    void *payload;
} bitsqz_llm_array_t;

// Per-stage wall time of one compress call in milliseconds (reference :85-93).  The
// misspelt member name is part of the interface.
typedef struct {
    double topk_separation_latency_ms;
    double svd_lowrank_cuda_latency_ms;
    double quantization_compress_latency_ms;
    double reconsturct_quantization_decompress_latency_ms;
    double reconstruct_svd_latency_ms;
    double error_extraction_latency_ms;
    double other_latency_ms;
} bitsqz_llm_compress_profile_t;

// All functions return 0 on success and 1 on any failure, never throw, and act on the
// calling thread's current CUDA device.  Each device has one compress runtime and one
// decompress runtime; an initialiser replaces the runtime of its kind on that device.

// Reference: include/bitsqz_llm.hpp:95-105, src/bitsqz_llm.cu:785-885.
BITSQZ_LLM_API int bitsqz_llm_compress_initialize(
    uint16_t num_rows, uint16_t num_columns,
    float outlier_topk_ratio, float error_correction_topk_ratio,
    int svd_ranks, int svd_niters,
    quantization_method_t svd_uv_format, quantization_method_t svd_s_format,
    quantization_method_t quantization_only_format,
    bitsqz_llm_input_location_t input_location);

// Reference: :107, src/bitsqz_llm.cu:887-889.
BITSQZ_LLM_API void bitsqz_llm_compress_release();

// Reference: :109-117, src/bitsqz_llm.cu:891-975.
BITSQZ_LLM_API int bitsqz_llm_decompress_initialize(
    uint16_t num_rows, uint16_t num_columns,
    float outlier_topk_ratio, float error_correction_topk_ratio,
    int svd_ranks,
    quantization_method_t svd_uv_format, quantization_method_t svd_s_format,
    quantization_method_t quantization_only_format);

// Reference: :119, src/bitsqz_llm.cu:977-979.
BITSQZ_LLM_API void bitsqz_llm_decompress_release();

// Reference: :121-124, src/bitsqz_llm.cu:981-1302.  `*out` must be null on entry.
BITSQZ_LLM_API int bitsqz_llm_compress(
    const float *row_major_matrix_float_data,
    bitsqz_llm_array_t **out,
    bitsqz_llm_compress_profile_t *profile);

// Reference: :126-130.
inline int bitsqz_llm_compress(const float *row_major_matrix_float_data, bitsqz_llm_array_t **out) {
    return bitsqz_llm_compress(row_major_matrix_float_data, out, nullptr);
}

// Reference: :132-135, src/bitsqz_llm.cu:1304-1393.  `d_dst` is device memory.
BITSQZ_LLM_API int bitsqz_llm_decompress(
    const bitsqz_llm_array_t *compressed, float *d_dst, uint32_t dst_num_elements);

// Reference: :137, src/bitsqz_llm.cu:1395-1415.
BITSQZ_LLM_API uint64_t bitsqz_llm_get_packed_size(const bitsqz_llm_array_t *compressed);

// Reference: :139, src/bitsqz_llm.cu:1417-1450.
BITSQZ_LLM_API bitsqz_llm_array_t *load_bitsqz_llm_from_buffer(const void *buffer, uint64_t buffer_size);

// Reference: :141, src/bitsqz_llm.cu:1452-1455.
BITSQZ_LLM_API void bitsqz_llm_free(bitsqz_llm_array_t *compressed);

// Not part of the reference's bitsqz_llm.hpp: the column-count helper of its top-k module
// (modules/topk_cuda/include/topk_cuda.cuh:47), which its own integration tests and walkthrough call next to the
// functions above; exported under the same C++ name.  k = (uint16_t)roundf(num_columns * topk_ratio), at most
// num_columns, at least 1 for a positive ratio.
BITSQZ_LLM_API uint16_t topk_compute_num_topk_columns(uint16_t num_columns, float topk_ratio);

static_assert(sizeof(bitsqz_section_t) == 24, "section entry is 24 bytes");
static_assert(sizeof(bitsqz_llm_array_t) == 200, "array header is 200 bytes");
static_assert(offsetof(bitsqz_llm_array_t, flags) == 40, "flags at byte 40");
static_assert(offsetof(bitsqz_llm_array_t, section_u) == 48, "section table starts at byte 48");
static_assert(offsetof(bitsqz_llm_array_t, section_error_topk) == 168, "last section at byte 168");
static_assert(offsetof(bitsqz_llm_array_t, payload) == 192, "payload pointer at byte 192");
static_assert(sizeof(bitsqz_llm_compress_profile_t) == 56, "profile is seven doubles");
