// Device-side building blocks shared by the sm_100a kernels: the NF4 encoder tables, E4M3
// scale coding, bounded mbarrier waits and 1-D bulk (TMA) copies between HBM and shared
// memory.  Everything that must agree bit-for-bit with the reference's CPU arithmetic uses
// explicitly rounded intrinsics (__fmul_rn, __fdiv_rn) so that the compiler can never fuse
// a multiply into a neighbouring add.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace bsq {

constexpr int kBlockElems = 64;          // NF4 block: 64 consecutive elements of the flat array
constexpr float kE4M3Max = 448.0f;
constexpr unsigned kFullMask = 0xffffffffu;

// Status word a kernel ORs into when it gives up on something instead of trapping.
enum : unsigned {
    kStatusBarrierTimeout = 1u << 0,     // an mbarrier / grid-barrier wait ran out of tries
    kStatusBadIndex = 1u << 1,           // an index read from a payload was out of range
    kStatusCholesky = 1u << 2,           // non-positive pivot in the k x k Cholesky
};

// ---- NF4 -------------------------------------------------------------------------------
// The 16 levels (reference quantization_cuda.cu:20-37, nf4_impl.cpp:3-20).
static __device__ __constant__ float c_nf4_levels[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

// Bucket table of the encoder.  The reference's scan (first level of minimal |v - L[i]|,
// quantization_cuda.cu:43-58) is, for every v below 2^23+1, the step function "number of
// thresholds <= v" over 15 thresholds.  v is mapped to one of 32 buckets by two FMAs (see
// nf4_bucket); bucket b holds at most one threshold c_nf4_bucket_thr[b] (NaN if none: v >= NaN is false for
// every v, so the code stays a nibble even for v = +Inf, whose neighbour in the packed byte it would otherwise spoil) and
// c_nf4_bucket_base[b] thresholds lie in lower buckets.  oracle/check_nf4_fast_encoder.c
// builds this table and proves code == scan for every finite |v| < 2^23.
static __device__ __constant__ unsigned c_nf4_bucket_thr[32] = {
    0x7fc00000u, 0x7fc00000u, 0xbf591cd8u, 0x7fc00000u, 0x7fc00000u, 0x7fc00000u, 0xbf1c5270u, 0x7fc00000u,
    0xbeeb847fu, 0x7fc00000u, 0xbeadea76u, 0x7fc00000u, 0xbe703cecu, 0xbe0d38bbu, 0x7fc00000u, 0xbd3a7870u,
    0x3d22fb00u, 0x3df64863u, 0x7fc00000u, 0x3e5067e1u, 0x3e9582d5u, 0x7fc00000u, 0x3ec753fau, 0x3f006d04u,
    0x7fc00000u, 0x3f248db0u, 0x7fc00000u, 0x7fc00000u, 0x7fc00000u, 0x3f5c89dau, 0x7fc00000u, 0x7fc00000u};
static __device__ __constant__ int c_nf4_bucket_base[32] = {
    0, 0, 0, 1, 1, 1, 1, 2, 2, 3, 3, 4, 4, 5, 6, 6, 7, 8, 9, 9, 10, 11, 11, 12, 13, 13, 14, 14, 14, 14, 15, 15};

// Literal restatement of the reference scan; only reached for |v| >= 2^23.
static __device__ __noinline__ unsigned nf4_code_scan(float v) {
    if (!isfinite(v)) v = 0.0f;
    int best = 0;
    float best_err = fabsf(__fsub_rn(v, c_nf4_levels[0]));
    for (int i = 1; i < 16; ++i) {
        const float err = fabsf(__fsub_rn(v, c_nf4_levels[i]));
        if (err < best_err) { best_err = err; best = i; }
    }
    return (unsigned)best;
}

// Per-lane copy of the bucket table: lane b keeps bucket b, a warp shuffle is the lookup.
struct Nf4Lut {
    float thr;
    int base;
    float level;    // lane c (c < 16) keeps level c for dequantisation
    __device__ __forceinline__ void load() {
        const int lane = threadIdx.x & 31;
        thr = __uint_as_float(c_nf4_bucket_thr[lane]);
        base = c_nf4_bucket_base[lane];
        level = c_nf4_levels[lane & 15];
    }
    // All 32 lanes of the warp must call this together.  v must satisfy |v| < 2^23.
    __device__ __forceinline__ unsigned encode(float v) const {
        const float u = __saturatef(fmaf(v, 0.5f, 0.5f));
        const int b = __float_as_int(fmaf(u, 31.0f, 12582912.0f));    // low 5 bits = bucket
        const float t = __shfl_sync(kFullMask, thr, b);
        const int c = __shfl_sync(kFullMask, base, b);
        return (unsigned)(c + (v >= t ? 1 : 0));
    }
    __device__ __forceinline__ float decode(unsigned code) const {
        return __shfl_sync(kFullMask, level, (int)code);
    }
};

// Non-finite inputs count as zero (reference quantization_cuda.cu:39-41).
__device__ __forceinline__ float sanitize(float x) {
    return ((__float_as_uint(x) & 0x7fffffffu) < 0x7f800000u) ? x : 0.0f;
}

// ---- E4M3 block-scale code (reference quantization_cuda.cu:64-128, nf4_dq_impl.cpp:83-129)
__device__ __forceinline__ unsigned e4m3_encode(float x) {
    if (!isfinite(x)) x = (x < 0.0f) ? -kE4M3Max : kE4M3Max;
    const unsigned sign = (__float_as_uint(x) >> 31) & 1u;
    float ax = fabsf(x);
    if (ax == 0.0f) return sign << 7;
    if (ax > kE4M3Max) ax = kE4M3Max;
    int e2 = 0;
    const float frac = frexpf(ax, &e2);
    int efield = e2 - 1 + 7;
    if (efield <= 0) {
        int m = __float2int_rn(__fmul_rn(ax, 512.0f));
        if (m > 7) m = 7;
        return (sign << 7) | (unsigned)(m & 7);
    }
    int m = __float2int_rn(__fmul_rn(__fsub_rn(__fmul_rn(frac, 2.0f), 1.0f), 8.0f));
    if (m > 7) { m = 0; efield += 1; }
    if (efield >= 16) { efield = 15; m = 7; }
    return (sign << 7) | ((unsigned)(efield & 0xF) << 3) | (unsigned)(m & 7);
}

__device__ __forceinline__ float e4m3_decode(unsigned c) {
    const unsigned sign = (c >> 7) & 1u, efield = (c >> 3) & 0xFu, m = c & 7u;
    // (1 + m/8) * 2^(e-7) and (m/8) * 2^-6 are exact in FP32, so bit assembly is exact too
    const float r = efield ? __uint_as_float(((efield + 120u) << 23) | (m << 20)) : __fmul_rn((float)m, 0.001953125f);
    return sign ? -r : r;
}

// dq = max/448, 1.0 when that is 0 or not finite (nf4_dq_impl.cpp:149-159,183-184)
__device__ __forceinline__ float dq_from_max(float gmax) {
    if (gmax == 0.0f || !isfinite(gmax)) return 1.0f;
    const float dq = __fdiv_rn(gmax, kE4M3Max);
    return dq == 0.0f ? 1.0f : dq;
}

// Effective block scale of NF4_DQ and its E4M3 code (nf4_dq_impl.cpp:203-209)
__device__ __forceinline__ float dq_block_scale(float absmax_or_one, float dq, unsigned *code_out) {
    const unsigned code = e4m3_encode(__fdiv_rn(absmax_or_one, dq));
    *code_out = code;
    float s = __fmul_rn(dq, e4m3_decode(code));
    if (s == 0.0f || !isfinite(s)) s = 1.0f;
    return s;
}

// ---- shared-memory barriers and bulk copies ------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void *p) {
    return (unsigned)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `kMbarSpinLimit` polls, records the failure in *status and
// returns false.  try_wait itself blocks for a hardware-chosen interval per call, so the
// limit corresponds to seconds, far beyond any legitimate copy.
constexpr unsigned kMbarSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, unsigned parity, unsigned *status) {
    for (unsigned i = 0; i < kMbarSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    if (status) atomicOr(status, kStatusBarrierTimeout);
    return false;
}

// CTA-wide wait for a bulk copy: only warp 0 polls the barrier (a polling warp burns issue slots
// whether 1 or 32 of its lanes spin), everybody else parks at the CTA barrier.  Returns false, for
// all threads alike, if the wait gave up.
__device__ __forceinline__ bool cta_wait_copy(uint64_t *bar, unsigned parity, unsigned *status) {
    bool ok = true;
    if (threadIdx.x < 32) ok = mbar_wait_bounded(bar, parity, status);
    return __syncthreads_and(ok) != 0;
}

// Order generic-proxy accesses to shared memory before later async-proxy (bulk copy) ones.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// HBM -> shared, completion counted in bytes on `bar`.  src, dst 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// shared -> HBM, tracked by the bulk async-group of the issuing thread.
__device__ __forceinline__ void bulk_s2g(void *dst_gmem, const void *src_smem, unsigned bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until the issuing thread's bulk stores have finished READING shared memory
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... until at most the newest of them is still reading (two staging buffers in turn)
__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- small warp helpers -----------------------------------------------------------------
__device__ __forceinline__ float group16_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 1));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 2));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 4));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 8));
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
    v = group16_max(v);
    return fmaxf(v, __shfl_xor_sync(kFullMask, v, 16));
}
__device__ __forceinline__ float abs4max(const float4 &a) {
    return fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w)));
}
__device__ __forceinline__ float4 sanitize4(const float4 &a) {
    return make_float4(sanitize(a.x), sanitize(a.y), sanitize(a.z), sanitize(a.w));
}

}  // namespace bsq
