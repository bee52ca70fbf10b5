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

#ifdef BSQ_TRACE
__device__ long long g_trace[2][8][16];
#define BSQ_T(kern, slot) do { if (blockIdx.x == 5 && threadIdx.x == 0 && trace_it < 8) g_trace[kern][trace_it][slot] = clock64(); } while (0)
#else
#define BSQ_T(kern, slot) do { } while (0)
#endif

namespace {

// Shared-memory layout of one CTA: the row, its nibbles, one float per 64-element block, scratch.
struct FrontSmemLayout {
    size_t codes_off, blk_off, scratch_off, total;
};
__host__ __device__ inline FrontSmemLayout front_layout(unsigned cols) {
    FrontSmemLayout l;
    l.codes_off = (size_t)cols * 4;
    l.blk_off = l.codes_off + (((size_t)cols / 2 + 15) & ~(size_t)15);
    l.scratch_off = l.blk_off + (((size_t)(cols / 64) * 4 + 15) & ~(size_t)15);
    l.total = l.scratch_off + sizeof(TopkScratch);
    return l;
}

// Block maxima of the row after outlier zeroing.  m4[f] are the float4 maxima taken BEFORE the
// zeroing (row_thread_max); only float4s marked dirty are read again.  `special` rows (Inf/NaN
// somewhere) are recomputed with non-finite values counted as zero, and a block that holds one
// gets its maximum NEGATED as a marker for the encoder.  blk_out[b] = absmax, or 1.0 for a block
// of zeros (quantization_cuda.cu:217-219).  Returns this thread's running maximum of |blk_out|.
template <int NT, int IT>
__device__ __forceinline__ float row_block_absmax(const float *row, unsigned cols, const unsigned (&m4)[IT],
                                                  const TopkScratch &s, bool special, float *blk_out) {
    const int tid = threadIdx.x, lane = tid & 31;
    const unsigned f4 = cols >> 2;
    const uint4 *row4 = reinterpret_cast<const uint4 *>(row);
    float run = 0.0f;
#pragma unroll
    for (int f = 0; f < IT; ++f) {
        if ((unsigned)f * NT >= f4) break;                   // uniform over the CTA
        const unsigned i = f * NT + tid;
        const bool valid = i < f4;
        unsigned m = m4[f];
        bool nonfinite = false;
        if (valid && (special || ((s.dirty[i >> 5] >> (i & 31u)) & 1u))) {
            const uint4 a = row4[i];
            const unsigned e[4] = {a.x & 0x7fffffffu, a.y & 0x7fffffffu, a.z & 0x7fffffffu, a.w & 0x7fffffffu};
            m = 0;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (e[q] < 0x7f800000u) m = max(m, e[q]);
                else nonfinite = true;
            }
        }
        // maximum over the 16 lanes of the block (bit patterns of non-negative floats order as
        // integers): one warp-reduce instruction per half warp
        m = __reduce_max_sync((lane & 16) ? 0xffff0000u : 0x0000ffffu, m);
        const unsigned nf = special ? __ballot_sync(kFullMask, nonfinite) : 0u;
        if (valid && (lane & 15) == 0) {
            const float am = __uint_as_float(m);
            const float v = am > 0.0f ? am : 1.0f;
            const bool marked = ((nf >> (lane & 16)) & 0xFFFFu) != 0;
            blk_out[i >> 4] = marked ? -v : v;
            run = fmaxf(run, v);
        }
    }
    return run;
}

// Per block of the row: scale -> (1/scale) for the encoder, kept in blk[] (shared memory).  A
// negative value marks a block that must take the literal scan (non-finite elements, or a scaled
// value that can leave the exact range of the table encoder).
//   DQ: blk_in holds the (possibly negated) block maxima from pass 1; writes the E4M3 codes.
//  !DQ: blk holds the maxima on entry; writes the FP32 scales.
template <int NT, bool DQ>
__device__ __forceinline__ void row_block_scales(unsigned cols, float dq, const float *blk_in, float *blk,
                                                 float *scales_out, uint8_t *scale_codes_out) {
    const unsigned nblk = cols >> 6;
    for (unsigned b = threadIdx.x; b < nblk; b += NT) {
        const float raw = DQ ? blk_in[b] : blk[b];
        const float am = fabsf(raw);
        float scale;
        if (DQ) {
            unsigned code;
            scale = dq_block_scale(am, dq, &code);
            scale_codes_out[b] = (uint8_t)code;
        } else {
            scale = am;
            scales_out[b] = scale;
        }
        const float inv = __fdiv_rn(1.0f, scale);
        const bool slow = raw < 0.0f || !(__fmul_rn(am, inv) < 8388608.0f);
        blk[b] = slow ? -inv : inv;
    }
}

// Nibbles of the row into codes_smem (cols/2 bytes); blk[] holds +-1/scale per block.
template <int NT>
__device__ __forceinline__ void row_encode(const float *row, unsigned cols, const Nf4Lut &lut, const float *blk,
                                           uint16_t *codes_smem) {
    const int tid = threadIdx.x;
    const unsigned f4 = cols >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
#pragma unroll 4
    for (unsigned i0 = 0; i0 < f4; i0 += NT) {               // every lane runs every iteration (shuffles)
        const unsigned i = i0 + tid;
        const bool valid = i < f4;
        const float4 a = valid ? row4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float invs = valid ? blk[i >> 4] : 1.0f;
        const float inv = fabsf(invs);
        unsigned c0 = lut.encode(__fmul_rn(a.x, inv));
        unsigned c1 = lut.encode(__fmul_rn(a.y, inv));
        unsigned c2 = lut.encode(__fmul_rn(a.z, inv));
        unsigned c3 = lut.encode(__fmul_rn(a.w, inv));
        if (invs < 0.0f) {                                   // rare: literal scan on sanitised values
            c0 = nf4_code_scan(__fmul_rn(sanitize(a.x), inv));
            c1 = nf4_code_scan(__fmul_rn(sanitize(a.y), inv));
            c2 = nf4_code_scan(__fmul_rn(sanitize(a.z), inv));
            c3 = nf4_code_scan(__fmul_rn(sanitize(a.w), inv));
        }
        if (valid) codes_smem[i] = (uint16_t)((c0 << 4) | c1 | (c2 << 12) | (c3 << 8));
    }
}

// Pass 1.  DQ == false: complete NF4 encode.  DQ == true: block maxima + global maximum only.
template <int NT, int IT, bool DQ>
__global__ void __launch_bounds__(NT, 1536 / NT)
    frontend_pass1_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                          uint16_t *__restrict__ out_idx, float *__restrict__ out_val, float *__restrict__ scales_f32,
                          uint8_t *__restrict__ data, float *__restrict__ absmax_scratch, unsigned *gmax_bits,
                          unsigned *row_counter, unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const FrontSmemLayout lay = front_layout(cols);
    float *row = reinterpret_cast<float *>(smem_raw);
    uint16_t *codes = reinterpret_cast<uint16_t *>(smem_raw + lay.codes_off);
    float *blk = reinterpret_cast<float *>(smem_raw + lay.blk_off);
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
    float run = 0.0f, hint = 0.0f;
    int trace_it = -1;
    (void)trace_it;
    __shared__ unsigned next_row;
    if (tid == 0) next_row = atomicAdd(row_counter, 1u);
    __syncthreads();
    for (;;) {
        const unsigned r = next_row;                         // rows are handed out dynamically
        if (r >= rows) break;
        ++trace_it;
        BSQ_T(0, 0);
        if (tid == 0) {
            mbar_expect_tx(&bar, bytes);
            bulk_g2s(row, in + (size_t)r * cols, bytes, &bar);
        }
        if (!cta_wait_copy(&bar, phase, status)) return;
        phase ^= 1u;
        BSQ_T(0, 1);
        unsigned m4[IT];
        const unsigned gb = row_thread_max<NT, IT>(row, cols, m4);
        const bool special = __syncthreads_or(gb >= 0x7f800000u) != 0;
        if (tid == 0) next_row = atomicAdd(row_counter, 1u);   // published by the barriers below
        BSQ_T(0, 2);
        if (k > 0) {
            hint = topk_row<NT, IT>(row, cols, k, s, out_idx + (size_t)r * k, out_val + (size_t)r * k, true, gb, m4, special,
                                hint);
            BSQ_T(0, 3);
        } else {
            for (int i = tid; i < 256; i += NT) s.dirty[i] = 0;
            __syncthreads();
        }
        if (DQ) {
            run = fmaxf(run, row_block_absmax<NT, IT>(row, cols, m4, s, special, absmax_scratch + (size_t)r * blocks_per_row));
            fence_proxy_async_smem();
            BSQ_T(0, 4);
        } else {
            row_block_absmax<NT, IT>(row, cols, m4, s, special, blk);
            __syncthreads();
            row_block_scales<NT, false>(cols, 1.0f, nullptr, blk, scales_f32 + (size_t)r * blocks_per_row, nullptr);
            __syncthreads();
            row_encode<NT>(row, cols, lut, blk, codes);
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
__global__ void __launch_bounds__(NT, 2048 / NT)
    frontend_pass2_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                          const uint16_t *__restrict__ idx, const float *__restrict__ absmax_scratch,
                          const unsigned *__restrict__ gmax_bits, float *__restrict__ dq_out,
                          uint8_t *__restrict__ scale_codes, uint8_t *__restrict__ data, unsigned *row_counter,
                          unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const FrontSmemLayout lay = front_layout(cols);
    float *row = reinterpret_cast<float *>(smem_raw);
    uint16_t *codes = reinterpret_cast<uint16_t *>(smem_raw + lay.codes_off);
    float *blk = reinterpret_cast<float *>(smem_raw + lay.blk_off);
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
    int trace_it = -1;
    (void)trace_it;
    __shared__ unsigned next_row;
    if (tid == 0) next_row = atomicAdd(row_counter, 1u);
    __syncthreads();
    for (;;) {
        const unsigned rr = next_row;
        if (rr >= rows) break;
        const unsigned r = rows - 1u - rr;                   // newest rows of pass 1 first
        ++trace_it;
        BSQ_T(1, 0);
        if (tid == 0) {
            mbar_expect_tx(&bar, bytes);
            bulk_g2s(row, in + (size_t)r * cols, bytes, &bar);
        }
        // scale work does not need the row: do it while the copy is in flight
        row_block_scales<NT, true>(cols, dq, absmax_scratch + (size_t)r * blocks_per_row, blk, nullptr,
                                   scale_codes + (size_t)r * blocks_per_row);
        BSQ_T(1, 1);
        if (!cta_wait_copy(&bar, phase, status)) return;
        phase ^= 1u;
        BSQ_T(1, 2);
        for (unsigned j = tid; j < k; j += NT) {
            const unsigned c = idx[(size_t)r * k + j];
            if (c < cols) row[c] = 0.0f;
        }
        __syncthreads();
        // every thread has read next_row by now; the barriers below publish the new value
        if (tid == 0) next_row = atomicAdd(row_counter, 1u);
        BSQ_T(1, 3);
        row_encode<NT>(row, cols, lut, blk, codes);
        fence_proxy_async_smem();
        __syncthreads();
        BSQ_T(1, 4);
        if (tid == 0) {
            bulk_s2g(data + (size_t)r * (cols / 2), codes, cols / 2);
            bulk_commit();
            bulk_wait_read_all();
        }
        __syncthreads();
        BSQ_T(1, 5);
    }
    if (tid == 0) bulk_wait_all();
}

int front_threads(uint32_t cols) { return cols <= 4096 ? 256 : (cols <= 16384 ? 512 : 1024); }

template <typename K>
cudaError_t persistent_grid(K kernel, int threads, size_t smem, int sm_count, unsigned rows, unsigned *grid_out) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (err != cudaSuccess) return err;
    int per_sm = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    if (err != cudaSuccess) return err;
    if (per_sm < 1) per_sm = 1;
    unsigned grid = (unsigned)sm_count * (unsigned)per_sm;
    *grid_out = grid > rows ? rows : grid;
    return cudaSuccess;
}

template <int NT, int IT>
cudaError_t launch_front(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                         float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                         void *d_scratch, unsigned *d_status, int sm_count, cudaStream_t stream, cudaEvent_t *events) {
    const size_t smem = front_layout(cols).total;
    // scratch words: [0] global maximum, [1] row counter of pass 1, [2] row counter of pass 2
    unsigned *gmax = static_cast<unsigned *>(d_scratch);
    float *absmax = reinterpret_cast<float *>(static_cast<uint8_t *>(d_scratch) + 16);
    unsigned grid = 0;
    cudaError_t err = cudaMemsetAsync(gmax, 0, 16, stream);
    if (err != cudaSuccess) return err;
    if (method == 11) {
        err = persistent_grid(frontend_pass1_kernel<NT, IT, false>, NT, smem, sm_count, rows, &grid);
        if (err != cudaSuccess) return err;
        if (events) cudaEventRecord(events[0], stream);
        frontend_pass1_kernel<NT, IT, false><<<grid, NT, smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, d_scales_f32,
                                                                      d_data, nullptr, nullptr, gmax + 1, d_status);
        if (events) { cudaEventRecord(events[1], stream); cudaEventRecord(events[2], stream); }
        return cudaGetLastError();
    }
    err = persistent_grid(frontend_pass1_kernel<NT, IT, true>, NT, smem, sm_count, rows, &grid);
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[0], stream);
    frontend_pass1_kernel<NT, IT, true><<<grid, NT, smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, nullptr, nullptr,
                                                                 absmax, gmax, gmax + 1, d_status);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[1], stream);
    err = persistent_grid(frontend_pass2_kernel<NT>, NT, smem, sm_count, rows, &grid);
    if (err != cudaSuccess) return err;
    frontend_pass2_kernel<NT><<<grid, NT, smem, stream>>>(d_in, rows, cols, k, d_idx, absmax, gmax, d_dq, d_scale_codes,
                                                          d_data, gmax + 2, d_status);
    if (events) cudaEventRecord(events[2], stream);
    return cudaGetLastError();
}

}  // namespace

#ifdef BSQ_TRACE
extern "C" int bsq_trace_read(long long *dst, long long *dst_topk) {
    if (cudaMemcpyFromSymbol(dst, g_trace, sizeof(g_trace)) != cudaSuccess) return 1;
    return cudaMemcpyFromSymbol(dst_topk, g_trace_topk, sizeof(g_trace_topk)) == cudaSuccess ? 0 : 1;
}
#endif

bool frontend_supported(uint32_t rows, uint32_t cols, uint32_t k) {
    if (rows == 0 || cols == 0 || cols % 64 != 0 || k > (uint32_t)kCandCap) return false;
    if (k > (uint32_t)front_threads(cols) || cols > 4u * (uint32_t)front_threads(cols) * kMaxRowIters) return false;
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
    if (!d_scratch || (method == 10 && (!d_dq || !d_scale_codes))) return cudaErrorInvalidValue;
    if (method == 11 && !d_scales_f32) return cudaErrorInvalidValue;
    const int nt = front_threads(cols);
    const bool few = cols <= 16u * (uint32_t)nt;              // at most 4 float4 per thread
#define BSQ_LAUNCH(NT_)                                                                                              \
    (few ? launch_front<NT_, 4>(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data,  \
                                d_scratch, d_status, sm_count, stream, events)                                        \
         : launch_front<NT_, 8>(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data,  \
                                d_scratch, d_status, sm_count, stream, events))
    switch (nt) {
        case 256: return BSQ_LAUNCH(256);
        case 512: return BSQ_LAUNCH(512);
        default: return BSQ_LAUNCH(1024);
    }
#undef BSQ_LAUNCH
}

}  // namespace bsq
