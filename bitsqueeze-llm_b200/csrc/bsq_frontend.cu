// Fused front end of the no-SVD compress path: per-row outlier separation followed by NF4 or
// NF4_DQ of the remainder, without ever writing the zeroed matrix to HBM (sm_100a).
//
// The reference runs, for this path, a device-to-device copy of the whole input, the top-k
// module (three kernels around a full segmented sort) and the quantiser (one kernel for NF4,
// four for NF4_DQ), each separated by a device synchronisation
// (src/bitsqz_llm.cu:1036-1056,1183-1195; modules/topk_cuda/src/topk_cuda_utils.cuh:275-295;
// modules/quantization_cuda/src/quantization_cuda.cu:564-624).  Here a CTA brings one row into
// shared memory with a bulk (TMA) copy, selects and zeroes its outliers there (bsq_topk.cuh)
// and then
//   * NF4:    computes the 64-element block scales and the nibbles from the same shared-memory
//             row and streams them out -- one kernel, input read once;
//   * NF4_DQ: writes only the block maxima (4 B per 64 elements) and folds them into one global
//             maximum; a second kernel, launched right behind, re-reads the rows (newest first,
//             so that most of them are still in L2), re-applies the zeroing from the k column
//             indices of the row, and encodes against dq * e4m3(absmax / dq).
// Rows must be a multiple of 64 long, so that NF4 blocks never straddle rows.
#include "bsq_internal.hpp"
#include "bsq_topk.cuh"

namespace bsq {

bool topk_rows_fit_smem(const void *d_in, const void *d_residual, uint32_t cols, uint32_t k);

namespace {

// One chunk = up to 4 iterations of the CTA over the row; a warp then covers 8 blocks of 64
// elements (16 lanes x float4 each) and lanes 0..7 own one block each for the scale work.
constexpr int kChunkIters = 4;

// Block absmax (1.0 for an all-zero block) of a shared-memory row -> absmax_out[block of the row].
// Returns this thread's running maximum over the blocks it owns.
template <int NT>
__device__ __forceinline__ float row_block_absmax(const float *row, unsigned cols, float *absmax_out) {
    const int tid = threadIdx.x, lane = tid & 31;
    const unsigned f4 = cols >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    float run = 0.0f;
    const unsigned iters = (f4 + NT - 1) / NT;               // every lane runs every iteration (shuffles)
    for (unsigned f = 0; f < iters; ++f) {
        const unsigned i = f * NT + tid;
        const bool valid = i < f4;
        float m = valid ? abs4max(sanitize4(row4[i])) : 0.0f;
        m = group16_max(m);
        if (valid && (lane & 15) == 0) {
            const float s = m > 0.0f ? m : 1.0f;
            absmax_out[i >> 4] = s;
            run = fmaxf(run, s);
        }
    }
    return run;
}

// Encode a shared-memory row.  DQ: scales come from absmax_in (per block of the row) and dq;
// the E4M3 codes go to scale_codes_out.  !DQ: scales are computed here and go to scales_out.
// Nibbles are written to codes_smem (cols/2 bytes).
template <int NT, bool DQ>
__device__ __forceinline__ void row_encode(const float *row, unsigned cols, const Nf4Lut &lut, float dq,
                                           const float *absmax_in, float *scales_out, uint8_t *scale_codes_out,
                                           uint16_t *codes_smem) {
    const int tid = threadIdx.x, lane = tid & 31, warp_base = tid & ~31;
    const unsigned f4 = cols >> 2;
    const unsigned iters = (f4 + NT - 1) / NT;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    for (unsigned f0 = 0; f0 < iters; f0 += kChunkIters) {
        float4 a[kChunkIters];
        float am[kChunkIters];
#pragma unroll
        for (int fi = 0; fi < kChunkIters; ++fi) {
            const unsigned i = (f0 + fi) * NT + tid;
            const bool valid = (f0 + fi) < iters && i < f4;
            a[fi] = valid ? sanitize4(row4[i]) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (!DQ) am[fi] = group16_max(abs4max(a[fi]));
        }
        // lane j < 8 owns block (fi = j >> 1, half = j & 1) of this warp's chunk
        const int ofi = lane >> 1, ohalf = lane & 1;
        const unsigned oi4 = (f0 + ofi) * NT + warp_base + ohalf * 16;      // first float4 of the owned block
        const bool owns = lane < 8 && (f0 + ofi) < iters && oi4 < f4;
        float blk_absmax = 0.0f, scale = 1.0f;
        if (!DQ) {
            float sgather = 0.0f;
#pragma unroll
            for (int fi = 0; fi < kChunkIters; ++fi) {
                const float t = __shfl_sync(kFullMask, am[fi], ohalf * 16);
                if (ofi == fi) sgather = t;
            }
            blk_absmax = sgather;
            scale = blk_absmax > 0.0f ? blk_absmax : 1.0f;
            if (owns) scales_out[oi4 >> 4] = scale;
        } else if (owns) {
            blk_absmax = absmax_in[oi4 >> 4];
            unsigned code;
            scale = dq_block_scale(blk_absmax, dq, &code);
            scale_codes_out[oi4 >> 4] = (uint8_t)code;
        }
        const float inv = __fdiv_rn(1.0f, scale);
        const unsigned slow_blocks = __ballot_sync(kFullMask, !(__fmul_rn(blk_absmax, inv) < 8388608.0f));
#pragma unroll
        for (int fi = 0; fi < kChunkIters; ++fi) {
            const int j = fi * 2 + (lane >> 4);
            const float invb = __shfl_sync(kFullMask, inv, j);
            const float v[4] = {a[fi].x, a[fi].y, a[fi].z, a[fi].w};
            unsigned c[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) c[q] = lut.encode(__fmul_rn(v[q], invb));
            if ((slow_blocks >> j) & 1u) {
#pragma unroll
                for (int q = 0; q < 4; ++q) c[q] = nf4_code_scan(__fmul_rn(v[q], invb));
            }
            const unsigned i = (f0 + fi) * NT + tid;
            if ((f0 + fi) < iters && i < f4)
                codes_smem[i] = (uint16_t)(((c[0] << 4) | c[1]) | (((c[2] << 4) | c[3]) << 8));
        }
    }
}

struct FrontSmemLayout {
    size_t codes_off, scratch_off, total;
};
__host__ __device__ inline FrontSmemLayout front_layout(unsigned cols) {
    FrontSmemLayout l;
    l.codes_off = (size_t)cols * 4;
    l.scratch_off = l.codes_off + (((size_t)cols / 2 + 15) & ~(size_t)15);
    l.total = l.scratch_off + sizeof(TopkScratch);
    return l;
}

// Pass 1.  DQ == false: complete NF4 encode.  DQ == true: block maxima + global maximum only.
template <int NT, bool DQ>
__global__ void __launch_bounds__(NT)
    frontend_pass1_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                          uint16_t *__restrict__ out_idx, float *__restrict__ out_val, float *__restrict__ scales_f32,
                          uint8_t *__restrict__ data, float *__restrict__ absmax_scratch, unsigned *gmax_bits,
                          unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const FrontSmemLayout lay = front_layout(cols);
    float *row = reinterpret_cast<float *>(smem_raw);
    uint16_t *codes = reinterpret_cast<uint16_t *>(smem_raw + lay.codes_off);
    TopkScratch &s = *reinterpret_cast<TopkScratch *>(smem_raw + lay.scratch_off);
    __shared__ __align__(8) uint64_t bar;
    const int tid = threadIdx.x;
    const unsigned bytes = cols * 4u, blocks_per_row = cols >> 6;
    Nf4Lut lut;
    lut.load();
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    unsigned phase = 0;
    float run = 0.0f;
    for (unsigned r = blockIdx.x; r < rows; r += gridDim.x) {
        if (tid == 0) {
            mbar_expect_tx(&bar, bytes);
            bulk_g2s(row, in + (size_t)r * cols, bytes, &bar);
        }
        if (!mbar_wait_bounded(&bar, phase, status)) return;
        phase ^= 1u;
        if (k > 0) topk_row<NT>(row, cols, k, s, out_idx + (size_t)r * k, out_val + (size_t)r * k, true);
        if (DQ) {
            run = fmaxf(run, row_block_absmax<NT>(row, cols, absmax_scratch + (size_t)r * blocks_per_row));
            fence_proxy_async_smem();
        } else {
            row_encode<NT, false>(row, cols, lut, 1.0f, nullptr, scales_f32 + (size_t)r * blocks_per_row, nullptr, codes);
            fence_proxy_async_smem();
            __syncthreads();
            if (tid == 0) {
                bulk_s2g(data + (size_t)r * (cols / 2), codes, cols / 2);
                bulk_commit();
                bulk_wait_read_all();
            }
        }
        __syncthreads();
    }
    if (DQ) {
        run = warp_max(run);
        if ((tid & 31) == 0 && run > 0.0f) atomicMax(gmax_bits, __float_as_uint(run));
    } else if (tid == 0) {
        bulk_wait_all();
    }
}

// Pass 2 of NF4_DQ: rows newest-first, zeroing re-applied from the row's k column indices.
template <int NT>
__global__ void __launch_bounds__(NT)
    frontend_pass2_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                          const uint16_t *__restrict__ idx, const float *__restrict__ absmax_scratch,
                          const unsigned *__restrict__ gmax_bits, float *__restrict__ dq_out,
                          uint8_t *__restrict__ scale_codes, uint8_t *__restrict__ data, unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const FrontSmemLayout lay = front_layout(cols);
    float *row = reinterpret_cast<float *>(smem_raw);
    uint16_t *codes = reinterpret_cast<uint16_t *>(smem_raw + lay.codes_off);
    __shared__ __align__(8) uint64_t bar;
    const int tid = threadIdx.x;
    const unsigned bytes = cols * 4u, blocks_per_row = cols >> 6;
    Nf4Lut lut;
    lut.load();
    const float dq = dq_from_max(__uint_as_float(*gmax_bits));
    if (blockIdx.x == 0 && tid == 0) *dq_out = dq;
    if (tid == 0) {
        mbar_init(&bar, 1);
        mbar_fence_init();
    }
    __syncthreads();
    unsigned phase = 0;
    for (unsigned rr = blockIdx.x; rr < rows; rr += gridDim.x) {
        const unsigned r = rows - 1u - rr;
        if (tid == 0) {
            mbar_expect_tx(&bar, bytes);
            bulk_g2s(row, in + (size_t)r * cols, bytes, &bar);
        }
        if (!mbar_wait_bounded(&bar, phase, status)) return;
        phase ^= 1u;
        if (k > 0) {
            for (unsigned j = tid; j < k; j += NT) {
                const unsigned c = idx[(size_t)r * k + j];
                if (c < cols) row[c] = 0.0f;
            }
            __syncthreads();
        }
        row_encode<NT, true>(row, cols, lut, dq, absmax_scratch + (size_t)r * blocks_per_row, nullptr,
                             scale_codes + (size_t)r * blocks_per_row, codes);
        fence_proxy_async_smem();
        __syncthreads();
        if (tid == 0) {
            bulk_s2g(data + (size_t)r * (cols / 2), codes, cols / 2);
            bulk_commit();
            bulk_wait_read_all();
        }
        __syncthreads();
    }
    if (tid == 0) bulk_wait_all();
}

int front_threads(uint32_t cols) { return cols <= 4096 ? 256 : (cols <= 16384 ? 512 : 1024); }

template <typename K>
cudaError_t persistent_grid(K kernel, int threads, size_t smem, int sm_count, unsigned rows, unsigned *grid_out) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    int per_sm = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    if (err != cudaSuccess) return err;
    if (per_sm < 1) per_sm = 1;
    unsigned grid = (unsigned)sm_count * (unsigned)per_sm;
    *grid_out = grid > rows ? rows : grid;
    return cudaSuccess;
}

template <int NT>
cudaError_t launch_front(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                         float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                         void *d_scratch, unsigned *d_status, int sm_count, cudaStream_t stream, cudaEvent_t *events) {
    const size_t smem = front_layout(cols).total;
    unsigned *gmax = static_cast<unsigned *>(d_scratch);
    float *absmax = reinterpret_cast<float *>(static_cast<uint8_t *>(d_scratch) + 16);
    unsigned grid = 0;
    cudaError_t err;
    if (method == 11) {
        err = persistent_grid(frontend_pass1_kernel<NT, false>, NT, smem, sm_count, rows, &grid);
        if (err != cudaSuccess) return err;
        if (events) cudaEventRecord(events[0], stream);
        frontend_pass1_kernel<NT, false><<<grid, NT, smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, d_scales_f32,
                                                                      d_data, nullptr, nullptr, d_status);
        if (events) { cudaEventRecord(events[1], stream); cudaEventRecord(events[2], stream); }
        return cudaGetLastError();
    }
    err = cudaMemsetAsync(gmax, 0, 16, stream);
    if (err != cudaSuccess) return err;
    err = persistent_grid(frontend_pass1_kernel<NT, true>, NT, smem, sm_count, rows, &grid);
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[0], stream);
    frontend_pass1_kernel<NT, true><<<grid, NT, smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, nullptr, nullptr,
                                                                 absmax, gmax, d_status);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[1], stream);
    err = persistent_grid(frontend_pass2_kernel<NT>, NT, smem, sm_count, rows, &grid);
    if (err != cudaSuccess) return err;
    frontend_pass2_kernel<NT><<<grid, NT, smem, stream>>>(d_in, rows, cols, k, d_idx, absmax, gmax, d_dq, d_scale_codes,
                                                          d_data, d_status);
    if (events) cudaEventRecord(events[2], stream);
    return cudaGetLastError();
}

}  // namespace

bool frontend_supported(uint32_t rows, uint32_t cols, uint32_t k) {
    if (rows == 0 || cols == 0 || cols % 64 != 0 || k > (uint32_t)kCandCap) return false;
    if (k > (uint32_t)front_threads(cols)) return false;
    return front_layout(cols).total <= 200 * 1024;
}

size_t frontend_scratch_bytes(uint32_t rows, uint32_t cols) { return 16 + (size_t)rows * (cols / 64) * sizeof(float); }

cudaError_t frontend_quantize(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                              float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                              void *d_scratch, unsigned *d_status, int sm_count, cudaStream_t stream,
                              cudaEvent_t *events) {
    if (!frontend_supported(rows, cols, k) || (method != 10 && method != 11)) return cudaErrorInvalidValue;
    if (!d_in || !d_data || (k > 0 && (!d_idx || !d_val))) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(d_in) % 16) || (reinterpret_cast<uintptr_t>(d_data) % 16)) return cudaErrorInvalidValue;
    if (method == 10 && (!d_dq || !d_scale_codes || !d_scratch)) return cudaErrorInvalidValue;
    if (method == 11 && !d_scales_f32) return cudaErrorInvalidValue;
    switch (front_threads(cols)) {
        case 256:
            return launch_front<256>(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data,
                                     d_scratch, d_status, sm_count, stream, events);
        case 512:
            return launch_front<512>(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data,
                                     d_scratch, d_status, sm_count, stream, events);
        default:
            return launch_front<1024>(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes,
                                      d_data, d_scratch, d_status, sm_count, stream, events);
    }
}

}  // namespace bsq
