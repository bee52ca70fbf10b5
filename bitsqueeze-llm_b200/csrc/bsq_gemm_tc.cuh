// Device helpers shared by the tensor-core product kernels (bsq_gemm_tc.cu, bsq_gemm_tma.cu): tcgen05 instruction and
// descriptor wrappers, the TF32 split, and the layout of the operand images that a product's second operand is split
// into beforehand.
#pragma once

#include <cuda_fp16.h>

#include "bsq_device.cuh"
#include "bsq_gemm.hpp"

namespace bsq {
namespace {

constexpr int TM = 128;          // output rows per CTA (UMMA M)
constexpr int TK = 16;           // K per shared-memory stage (two k-steps of 8)
constexpr int NT = 256;          // threads: all stage operands, one issues the MMAs, two per accumulator row in the epilogue
constexpr int DEPTH = 3;         // chunks of K in flight in registers per thread
constexpr int STAGES = 2;        // operand stages in shared memory (three measured slower: less L1 left for the loads)

__device__ __forceinline__ uint64_t smem_desc(unsigned addr_bytes, unsigned lbo_bytes, unsigned sbo_bytes) {
    // start address, leading / stride byte offsets in 16-byte units; version 1 (bits 46-47); no swizzle
    return (uint64_t)((addr_bytes >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

__device__ __forceinline__ void mma_tf32(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, bool accumulate) {
    const unsigned acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void mma_f16(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, bool accumulate) {
    const unsigned acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// 16 consecutive accumulator columns of this thread's row (lane) of tensor memory
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// 32-byte global accesses (sm_100): a thread of the epilogue owns a row of the tile, so every access of a warp goes to 32
// different lines; whole 32-byte sectors halve the number of memory instructions (and of entries in the load/store
// queue, where the epilogue warps were seen to stall) against 16-byte accesses that use half a sector each.
__device__ __forceinline__ void ld_global_v8(const float *p, float4 &a, float4 &b) {
    asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=f"(a.x), "=f"(a.y), "=f"(a.z), "=f"(a.w), "=f"(b.x), "=f"(b.y), "=f"(b.z), "=f"(b.w)
                 : "l"(p));
}
__device__ __forceinline__ void st_global_v8(float *p, const float4 &a, const float4 &b) {
    asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(a.x), "f"(a.y), "f"(a.z), "f"(a.w), "f"(b.x),
                 "f"(b.y), "f"(b.z), "f"(b.w)
                 : "memory");
}
// Round to TF32 (10 mantissa bits), ties away from zero, by integer arithmetic on the bit pattern: two full-rate
// instructions (add half of the last kept place, clear the 13 low bits; a carry out of the mantissa bumps the exponent
// as it should).  Same result as cvt.rna.tf32.f32 for every finite value.
__device__ __forceinline__ float tf32_rna(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}

// x = hi + lo + e with hi, lo exactly representable in TF32 and |e| <= 2^-22 |x|
__device__ __forceinline__ void split_store(float4 v, float4 *hi, float4 *lo) {
    const float4 h = make_float4(tf32_rna(v.x), tf32_rna(v.y), tf32_rna(v.z), tf32_rna(v.w));
    *hi = h;
    *lo = make_float4(tf32_rna(__fsub_rn(v.x, h.x)), tf32_rna(__fsub_rn(v.y, h.y)), tf32_rna(__fsub_rn(v.z, h.z)),
                      tf32_rna(__fsub_rn(v.w, h.w)));
}

// The FP16 form of the split: x * s = hi + lo' / 2^11 (+ e, |e| <= 2^-22 |x * s|) with hi = fp16(x * s) and
// lo' = fp16((x * s - hi) * 2^11), s a power of two that brings the operand's largest magnitude into [2^14, 2^15):
// hi carries 11 significant bits and lo' the next 11, like the two TF32 halves, and lo' has hi's magnitude, so both sit
// in FP16's range (elements below 2^-28 of the largest lose bits, an absolute error below FP32's on the largest).
// hi * hi goes into one accumulator, lo' * hi + hi * lo' into the other, which the epilogue scales by 2^-11.
constexpr float kSplit16LoScale = 2048.0f;
// The scale from the bits of the operand's largest |x|: 2^(14 - exponent), kept within 2^+-60 so that the product of
// two scales and its reciprocal stay finite (an operand of zeros, or one that holds Inf / NaN, gets 1: zeros stay
// zeros, and the non-finite values go through the conversion as they are).
__device__ __forceinline__ float split16_scale(unsigned absmax_bits) {
    if (absmax_bits == 0u || absmax_bits >= 0x7f800000u) return 1.0f;
    const int e = (int)(absmax_bits >> 23) - 127;
    return exp2f((float)min(max(14 - e, -60), 60));
}
// eight consecutive k of one row: two 16-byte units (hi, lo).  hi is taken as a float first, by the integer rounding
// of tf32_rna (FP16 has TF32's 10 mantissa bits, so the value converts exactly wherever FP16 is normal), which leaves
// one conversion instruction per pair of halves (cvt.rn.f16x2.f32) instead of three conversions per element.
__device__ __forceinline__ void split16_store8(const float4 &a, const float4 &b, float s, uint4 *hi, uint4 *lo, float lo_scale = kSplit16LoScale) {
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    float h[8], l[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float xs = v[i] * s;
        h[i] = tf32_rna(xs);
        l[i] = (xs - h[i]) * lo_scale;
    }
    auto pack = [](float p, float q) {
        const __half2 r = __floats2half2_rn(p, q);
        return *reinterpret_cast<const unsigned *>(&r);
    };
    *hi = make_uint4(pack(h[0], h[1]), pack(h[2], h[3]), pack(h[4], h[5]), pack(h[6], h[7]));
    *lo = make_uint4(pack(l[0], l[1]), pack(l[2], l[3]), pack(l[4], l[5]), pack(l[6], l[7]));
}

// A B image is dense (nobody stores into it with a pattern that could conflict): core matrices of 8 columns x 16 B
// follow one another along N every 128 B (SBO) and along K every extent * 16 B (LBO).
__host__ __device__ constexpr unsigned image_half_units(int extent) { return (unsigned)(TK / 4) * (unsigned)extent; }
__device__ __forceinline__ unsigned image_unit_index(int kc, int r, int extent) { return (unsigned)kc * (unsigned)extent + (unsigned)r; }
// 16-byte units from one chunk's image to the next, and from one tile column's images to the next
__host__ __device__ constexpr size_t image_units(int n_tile) { return 2 * (size_t)image_half_units(n_tile); }


}  // namespace
}  // namespace bsq
