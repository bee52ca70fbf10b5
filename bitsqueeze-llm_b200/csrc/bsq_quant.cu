// NF4 / NF4_DQ blockwise quantiser and dequantiser over a flat FP32 array (sm_100a).
//
// Replaces the reference kernels nf4_compress_kernel, compute_block_absmax_kernel,
// cub::DeviceReduce::Max, store_dq_scale_kernel, nf4_dq_compress_kernel,
// nf4_decompress_kernel and nf4_dq_decompress_kernel
// (modules/quantization_cuda/src/quantization_cuda.cu:130-341, launched from :564-663).
//
// Work decomposition: a warp takes a batch of 1024 consecutive elements = 16 blocks of 64.
// In each of 4 iterations a lane owns 8 consecutive elements (two 128-bit loads, one 32-bit
// store of 8 nibbles), so a block is 8 adjacent lanes and its absmax is 3 shuffles.  The
// per-block scale work (IEEE reciprocal, E4M3 coding) is done once per block by lanes 0..15
// and handed to the owning lanes by shuffle.  Codes come from the bucket-table encoder in
// bsq_device.cuh.  HBM-bound: 4 B read + 0.5 B + (4 or 1)/64 B written per element.
#include "bsq_device.cuh"
#include "bsq_internal.hpp"

#include <mutex>

namespace bsq {
namespace {

// Scratch of nf4dq_quantize_static(): global-max word (16 bytes) + one float per 64-element
// block, for at most kStaticMaxElems elements.  Lives in the module image of every device that
// loads the library, from load to exit.
constexpr uint64_t kStaticMaxElems = 1ull << 24;
static __device__ __align__(256) unsigned char g_static_scratch[16 + (kStaticMaxElems / 64) * sizeof(float)];

constexpr int kBatch = 1024;
constexpr int kThreads = 256;

struct Lane8 {
    float v[8];
};

__device__ __forceinline__ Lane8 load8(const float *x, uint64_t e, uint64_t n, bool vec) {
    Lane8 r;
    if (vec && e + 8 <= n) {
        const float4 a = __ldcs(reinterpret_cast<const float4 *>(x + e));
        const float4 b = __ldcs(reinterpret_cast<const float4 *>(x + e) + 1);
        r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
        r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) r.v[j] = (e + j < n) ? x[e + j] : 0.0f;
    }
    return r;
}

__device__ __forceinline__ float absmax8(const Lane8 &r) {
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(sanitize(r.v[j])));
    return m;
}

__device__ __forceinline__ float group8_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 1));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 2));
    v = fmaxf(v, __shfl_xor_sync(kFullMask, v, 4));
    return v;
}

// Lane l (< 16) receives the value that block l of the batch holds: block j = 4*it + g lives
// in am[it] of lanes 8g..8g+7.
__device__ __forceinline__ float gather_block_value(const float (&am)[4], int lane) {
    float s = 0.0f;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const float t = __shfl_sync(kFullMask, am[it], (lane & 3) * 8);
        if ((lane >> 2) == it) s = t;
    }
    return s;
}

// ---- NF4_DQ pass 1: per-block absmax (1.0 for an all-zero block) and the global maximum ----
__global__ void __launch_bounds__(kThreads) absmax_flat_kernel(const float *__restrict__ x, uint64_t n, bool vec,
                                                               float *__restrict__ absmax_out,
                                                               unsigned *__restrict__ gmax_bits) {
    const int lane = threadIdx.x & 31;
    const uint64_t warp = (uint64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const uint64_t nwarps = (uint64_t)gridDim.x * (kThreads / 32);
    const uint64_t nb = (n + 63) / 64;
    float run = 0.0f;
    for (uint64_t base = warp * kBatch; base < n; base += nwarps * kBatch) {
        float am[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const Lane8 r = load8(x, base + it * 256 + lane * 8, n, vec);
            am[it] = group8_max(absmax8(r));
        }
        float s = gather_block_value(am, lane);
        s = s > 0.0f ? s : 1.0f;
        const uint64_t blk = base / 64 + lane;
        if (lane < 16 && blk < nb) {
            absmax_out[blk] = s;
            run = fmaxf(run, s);
        }
    }
    run = warp_max(run);
    if (lane == 0 && run > 0.0f) atomicMax(gmax_bits, __float_as_uint(run));
}

// ---- encode: NF4 (DQ == false: computes its own absmax) or NF4_DQ pass 2 -----------------
template <bool DQ, bool WRITE_DEQ>
__global__ void __launch_bounds__(kThreads)
    encode_flat_kernel(const float *x, uint64_t n, bool vec, const float *__restrict__ absmax_in,
                       const unsigned *__restrict__ gmax_bits, float *__restrict__ scales_f32,
                       uint8_t *__restrict__ scale_codes, float *__restrict__ dq_out, uint8_t *__restrict__ data,
                       float *deq_out) {   // deq_out may alias x (in-place write-back)
    const int lane = threadIdx.x & 31;
    const uint64_t warp = (uint64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const uint64_t nwarps = (uint64_t)gridDim.x * (kThreads / 32);
    const uint64_t nb = (n + 63) / 64;
    Nf4Lut lut;
    lut.load();
    float dq = 1.0f;
    if (DQ) {
        dq = dq_from_max(__uint_as_float(*gmax_bits));
        if (warp == 0 && lane == 0) *dq_out = dq;
    }
    for (uint64_t base = warp * kBatch; base < n; base += nwarps * kBatch) {
        Lane8 r[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) r[it] = load8(x, base + it * 256 + lane * 8, n, vec);

        const uint64_t blk = base / 64 + lane;
        const bool owns_block = lane < 16 && blk < nb;
        float scale = 1.0f, blk_absmax = 0.0f;
        if (!DQ) {
            float am[4];
#pragma unroll
            for (int it = 0; it < 4; ++it) am[it] = group8_max(absmax8(r[it]));
            blk_absmax = gather_block_value(am, lane);
            scale = blk_absmax > 0.0f ? blk_absmax : 1.0f;
            if (owns_block) scales_f32[blk] = scale;
        } else {
            if (owns_block) {
                blk_absmax = absmax_in[blk];
                unsigned code;
                scale = dq_block_scale(blk_absmax, dq, &code);
                scale_codes[blk] = (uint8_t)code;
            }
        }
        const float inv = __fdiv_rn(1.0f, scale);
        // A scaled value leaves the encoder's exact range (|v| < 2^23) only in two corners: a DQ
        // block that fell back to scale 1.0 while holding a huge element, and a block whose scale
        // is so small (denormal) that 1/scale overflows; such blocks take the literal scan.
        const unsigned slow_blocks = __ballot_sync(kFullMask, !(__fmul_rn(blk_absmax, inv) < 8388608.0f));

#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int j = it * 4 + (lane >> 3);
            const float invb = __shfl_sync(kFullMask, inv, j);
            const uint64_t e = base + it * 256 + lane * 8;
            unsigned c[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) c[q] = lut.encode(__fmul_rn(sanitize(r[it].v[q]), invb));
            if ((slow_blocks >> j) & 1u) {
#pragma unroll
                for (int q = 0; q < 8; ++q) c[q] = nf4_code_scan(__fmul_rn(sanitize(r[it].v[q]), invb));
            }
            if (WRITE_DEQ) {
                const float sb = __shfl_sync(kFullMask, scale, j);
                float d[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) d[q] = __fmul_rn(sb, lut.decode(c[q]));
                if (vec && e + 8 <= n) {
                    reinterpret_cast<float4 *>(deq_out + e)[0] = make_float4(d[0], d[1], d[2], d[3]);
                    reinterpret_cast<float4 *>(deq_out + e)[1] = make_float4(d[4], d[5], d[6], d[7]);
                } else {
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        if (e + q < n) deq_out[e + q] = d[q];
                }
            }
            if (e + 8 <= n) {
                const unsigned w = ((c[0] << 4) | c[1]) | (((c[2] << 4) | c[3]) << 8) | (((c[4] << 4) | c[5]) << 16) |
                                   (((c[6] << 4) | c[7]) << 24);
                if (vec) {
                    *reinterpret_cast<unsigned *>(data + e / 2) = w;
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q) data[e / 2 + q] = (uint8_t)(w >> (8 * q));
                }
            } else if (e < n) {
#pragma unroll
                for (int q = 0; q < 8; q += 2) {
                    if (e + q < n) {
                        const unsigned lo = (e + q + 1 < n) ? c[q + 1] : 0u;   // odd tail: low nibble 0
                        data[(e + q) / 2] = (uint8_t)((c[q] << 4) | lo);
                    }
                }
            }
        }
    }
}

// ---- decode ----------------------------------------------------------------------------------
// Optional (idx non-null): a row-wise top-k list to add onto the decoded rows x cols matrix in the same pass.
struct TopkList {
    const uint16_t *idx;
    const float *val;
    unsigned cols, k;
    unsigned *status;
};
template <bool DQ>
__global__ void __launch_bounds__(kThreads)
    decode_flat_kernel(const float *__restrict__ scales_f32, const uint8_t *__restrict__ scale_codes,
                       const float *__restrict__ dq_in, const uint8_t *__restrict__ data, uint64_t n, bool vec,
                       float *out, TopkList add) {
    const int lane = threadIdx.x & 31;
    const uint64_t warp = (uint64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    const uint64_t nwarps = (uint64_t)gridDim.x * (kThreads / 32);
    const uint64_t nb = (n + 63) / 64;
    Nf4Lut lut;
    lut.load();
    float dq = 1.0f;
    if (DQ) {
        dq = *dq_in;
        if (dq == 0.0f || !isfinite(dq)) dq = 1.0f;   // quantization_cuda.cu:325-328
    }
    for (uint64_t base = warp * kBatch; base < n; base += nwarps * kBatch) {
        const uint64_t blk = base / 64 + lane;
        float scale = 1.0f;
        if (lane < 16 && blk < nb) {
            scale = DQ ? __fmul_rn(dq, e4m3_decode(scale_codes[blk])) : scales_f32[blk];
            if (scale == 0.0f || !isfinite(scale)) scale = 1.0f;
        }
        unsigned w[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const uint64_t e = base + it * 256 + lane * 8;
            if (vec && e + 8 <= n) {
                w[it] = __ldcs(reinterpret_cast<const unsigned *>(data + e / 2));
            } else {
                w[it] = 0;
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (e + 2 * q < n) w[it] |= (unsigned)data[e / 2 + q] << (8 * q);
            }
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const uint64_t e = base + it * 256 + lane * 8;
            const float sb = __shfl_sync(kFullMask, scale, it * 4 + (lane >> 3));
            float d[8];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const unsigned byte = (w[it] >> (8 * q)) & 0xFFu;
                d[2 * q] = __fmul_rn(sb, lut.decode(byte >> 4));
                d[2 * q + 1] = __fmul_rn(sb, lut.decode(byte & 0xFu));
            }
            if (vec && e + 8 <= n) {
                __stcs(reinterpret_cast<float4 *>(out + e), make_float4(d[0], d[1], d[2], d[3]));
                __stcs(reinterpret_cast<float4 *>(out + e) + 1, make_float4(d[4], d[5], d[6], d[7]));
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (e + q < n) out[e + q] = d[q];
            }
        }
        if (add.idx) {
            // dense[row, idx] += value (topk_cuda.cuh:83-86) for the entries that fall into the kBatch elements this
            // warp has just written: the row(s) of the batch, k entries each, a few per lane
            __syncwarp();                                     // the warp's stores are ordered before its reads below
            const uint64_t last = (base + kBatch <= n ? base + kBatch : n) - 1;
            for (uint64_t r = base / add.cols; r <= last / add.cols; ++r) {
                for (unsigned j = lane; j < add.k; j += 32) {
                    const unsigned c = add.idx[r * add.k + j];
                    if (c < add.cols) {
                        const uint64_t pos = r * add.cols + c;
                        if (pos >= base && pos <= last) out[pos] = out[pos] + add.val[r * add.k + j];
                    } else if (add.status) {
                        atomicOr(add.status, kStatusBadIndex);
                    }
                }
            }
        }
    }
}

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int grid_for(uint64_t n, int sm_count) {
    const uint64_t batches = (n + kBatch - 1) / kBatch;
    const uint64_t blocks = (batches + (kThreads / 32) - 1) / (kThreads / 32);
    const uint64_t cap = (uint64_t)sm_count * 8;      // 8 resident CTAs of 256 threads per SM
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace

cudaError_t nf4_quantize(const float *d_x, uint64_t n, float *d_scales, uint8_t *d_data, float *d_deq_out, int sm_count,
                         cudaStream_t stream) {
    const bool vec = aligned(d_x, 16) && aligned(d_data, 4) && (!d_deq_out || aligned(d_deq_out, 16));
    const int grid = grid_for(n, sm_count);
    if (d_deq_out)
        encode_flat_kernel<false, true><<<grid, kThreads, 0, stream>>>(d_x, n, vec, nullptr, nullptr, d_scales, nullptr,
                                                                         nullptr, d_data, d_deq_out);
    else
        encode_flat_kernel<false, false><<<grid, kThreads, 0, stream>>>(d_x, n, vec, nullptr, nullptr, d_scales, nullptr,
                                                                          nullptr, d_data, nullptr);
    return cudaGetLastError();
}

size_t nf4dq_scratch_bytes(uint64_t n) { return (size_t)((n + 63) / 64) * sizeof(float) + 16; }

cudaError_t nf4dq_quantize(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                           float *d_deq_out, void *d_scratch, int sm_count, cudaStream_t stream) {
    // scratch layout: [0,16) global-max word (+ padding), then one float per block
    unsigned *gmax = static_cast<unsigned *>(d_scratch);
    float *absmax = reinterpret_cast<float *>(static_cast<uint8_t *>(d_scratch) + 16);
    const bool vec = aligned(d_x, 16) && aligned(d_data, 4) && (!d_deq_out || aligned(d_deq_out, 16));
    const int grid = grid_for(n, sm_count);
    cudaError_t err = cudaMemsetAsync(gmax, 0, 16, stream);
    if (err != cudaSuccess) return err;
    absmax_flat_kernel<<<grid, kThreads, 0, stream>>>(d_x, n, vec, absmax, gmax);
    if (d_deq_out)
        encode_flat_kernel<true, true><<<grid, kThreads, 0, stream>>>(d_x, n, vec, absmax, gmax, nullptr, d_scale_codes,
                                                                        d_dq, d_data, d_deq_out);
    else
        encode_flat_kernel<true, false><<<grid, kThreads, 0, stream>>>(d_x, n, vec, absmax, gmax, nullptr, d_scale_codes,
                                                                         d_dq, d_data, nullptr);
    return cudaGetLastError();
}

uint64_t nf4dq_static_max_elements() { return kStaticMaxElems; }

// NF4_DQ quantiser that allocates nothing: its scratch is the file-scope array above.  The device
// address of that array is looked up once per device (cudaGetSymbolAddress, with that device
// current) the first time the function runs there; that first call should therefore come before
// any stream capture.  All calls on a device share the array: work from two calls that overlaps
// on the GPU (different streams) races on it.  Stale contents are harmless: the global-max word is
// cleared at the start of every call and every block maximum that is read was written by the same call.
cudaError_t nf4dq_quantize_static(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                                  int sm_count, cudaStream_t stream) {
    static std::mutex mu;
    static void *scratch_of_device[64] = {};
    if (n == 0 || n > kStaticMaxElems) return cudaErrorInvalidValue;
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> g(mu);
        if (!scratch_of_device[dev]) {
            void *p = nullptr;
            err = cudaGetSymbolAddress(&p, g_static_scratch);     // host code must not pass the symbol itself
            if (err != cudaSuccess) return err;
            scratch_of_device[dev] = p;
        }
        scratch = scratch_of_device[dev];
    }
    return nf4dq_quantize(d_x, n, d_dq, d_scale_codes, d_data, nullptr, scratch, sm_count, stream);
}

cudaError_t nf4_dequantize(const float *d_scales, const uint8_t *d_data, uint64_t n, float *d_out, int sm_count,
                           cudaStream_t stream) {
    const bool vec = aligned(d_data, 4) && aligned(d_out, 16);
    decode_flat_kernel<false><<<grid_for(n, sm_count), kThreads, 0, stream>>>(d_scales, nullptr, nullptr, d_data, n, vec,
                                                                                d_out, TopkList{});
    return cudaGetLastError();
}

cudaError_t nf4dq_dequantize(const float *d_dq, const uint8_t *d_scale_codes, const uint8_t *d_data, uint64_t n,
                             float *d_out, int sm_count, cudaStream_t stream) {
    const bool vec = aligned(d_data, 4) && aligned(d_out, 16);
    decode_flat_kernel<true><<<grid_for(n, sm_count), kThreads, 0, stream>>>(nullptr, d_scale_codes, d_dq, d_data, n, vec,
                                                                               d_out, TopkList{});
    return cudaGetLastError();
}

// Dequantise a rows x cols matrix and add its row-wise top-k list in the same pass (quantization_cuda_decompress
// followed by topk_apply in the reference, src/bitsqz_llm.cu:1304-1393).  d_scales: FP32 block scales (NF4) or null;
// d_dq + d_scale_codes: NF4_DQ or null.
cudaError_t nf4_dequantize_add_topk(const float *d_scales, const float *d_dq, const uint8_t *d_scale_codes, const uint8_t *d_data,
                                    uint32_t rows, uint32_t cols, const uint16_t *d_idx, const float *d_val, uint32_t k,
                                    float *d_out, unsigned *d_status, int sm_count, cudaStream_t stream) {
    if (!d_data || !d_out || !d_idx || !d_val || rows == 0 || cols == 0 || k == 0) return cudaErrorInvalidValue;
    if ((d_scales != nullptr) == (d_dq != nullptr && d_scale_codes != nullptr)) return cudaErrorInvalidValue;
    const uint64_t n = (uint64_t)rows * cols;
    const bool vec = aligned(d_data, 4) && aligned(d_out, 16);
    const TopkList add{d_idx, d_val, cols, k, d_status};
    if (d_scales)
        decode_flat_kernel<false><<<grid_for(n, sm_count), kThreads, 0, stream>>>(d_scales, nullptr, nullptr, d_data, n, vec, d_out, add);
    else
        decode_flat_kernel<true><<<grid_for(n, sm_count), kThreads, 0, stream>>>(nullptr, d_scale_codes, d_dq, d_data, n, vec, d_out, add);
    return cudaGetLastError();
}

}  // namespace bsq
