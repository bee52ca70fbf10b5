// Fused front end of the no-SVD compress path: per-row outlier separation followed by NF4 or
// NF4_DQ of the remainder, without ever writing the zeroed matrix to HBM (sm_100a).
//
// The reference runs, for this path, a device-to-device copy of the whole input, the top-k module
// (three kernels around a full segmented sort) and the quantiser (one kernel for NF4, four for
// NF4_DQ), each separated by a device synchronisation (src/bitsqz_llm.cu:1036-1056,1183-1195;
// modules/topk_cuda/src/topk_cuda_utils.cuh:275-295; modules/quantization_cuda/src/
// quantization_cuda.cu:564-624).  Here a group of G warps (bsq_rowgroup.cuh) brings one row into
// shared memory with a bulk (TMA) copy, selects and zeroes its outliers there and then
//   * NF4:    computes the 64-element block scales and the nibbles from the same shared-memory row
//             and streams them out -- one kernel, input read once;
//   * NF4_DQ: writes only the block maxima (4 B per 64 elements) and folds them into one global
//             maximum; a second kernel, launched right behind, re-reads the rows (newest first, so
//             that most of them are still in L2), re-applies the zeroing from the row's k column
//             indices, and encodes against dq * e4m3(absmax / dq).
// Rows are a multiple of 64 long, so NF4 blocks never straddle rows.  Rows are handed to the groups
// through an atomic counter; every wait on a copy is bounded and reports through the status word.
#include "bsq_internal.hpp"
#include "bsq_rowgroup.cuh"

#include <cstdlib>

namespace bsq {
namespace {

// Shared memory of one group: row | nibbles | one float per block | control.
struct GroupLayout {
    size_t codes_off, blk_off, ctl_off, total;
};
__host__ __device__ inline GroupLayout group_layout(unsigned cols, bool with_codes) {
    GroupLayout l;
    l.codes_off = (size_t)cols * 4;
    l.blk_off = l.codes_off + (with_codes ? (((size_t)cols / 2 + 15) & ~(size_t)15) : 0);
    l.ctl_off = l.blk_off + (((size_t)(cols / 64) * 4 + 15) & ~(size_t)15);
    l.total = (l.ctl_off + sizeof(GroupCtl) + 127) & ~(size_t)127;
    return l;
}

// Fetch the next row for the group (lane 0 asks the global counter) and start its copy.
// Returns the row index, uniform over the group (>= rows: no work left).
template <int G>
__device__ __forceinline__ unsigned group_next_row(const RowGroup<G> &g, GroupCtl &c, unsigned *row_counter) {
    if (g.lane == 0) c.next_row = atomicAdd(row_counter, 1u);
    g.sync();
    const unsigned r = c.next_row;
    g.sync();
    return r;
}

template <int G>
__device__ __forceinline__ bool group_wait_copy(GroupCtl &c, unsigned parity, unsigned *status) {
    return mbar_wait_bounded(reinterpret_cast<uint64_t *>(&c.bar), parity, status);
}

// Pass 1.  DQ == false: complete NF4 encode.  DQ == true: selection + block maxima + global maximum.
template <int G, bool DQ>
__global__ void __launch_bounds__(512)
    frontend_pass1_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                          uint16_t *__restrict__ out_idx, float *__restrict__ out_val, float *__restrict__ scales_f32,
                          uint8_t *__restrict__ data, float *__restrict__ absmax_scratch, unsigned *gmax_bits,
                          unsigned *row_counter, unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const RowGroup<G> g;
    const GroupLayout lay = group_layout(cols, !DQ);
    unsigned char *base = smem_raw + (size_t)g.gid * lay.total;
    float *row = reinterpret_cast<float *>(base);
    uint16_t *codes = reinterpret_cast<uint16_t *>(base + lay.codes_off);
    float *blk = reinterpret_cast<float *>(base + lay.blk_off);
    GroupCtl &c = *reinterpret_cast<GroupCtl *>(base + lay.ctl_off);
    uint64_t *bar = reinterpret_cast<uint64_t *>(&c.bar);
    const unsigned bytes = cols * 4u, blocks_per_row = cols >> 6;
    Nf4Lut lut;
    lut.load();
    if (g.lane == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    g.sync();
    unsigned phase = 0;
    float run = 0.0f, hint = 0.0f;
    for (;;) {
        const unsigned r = group_next_row<G>(g, c, row_counter);
        if (r >= rows) break;
        if (g.lane == 0) {
            mbar_expect_tx(bar, bytes);
            bulk_g2s(row, in + (size_t)r * cols, bytes, bar);
        }
        if (!group_wait_copy<G>(c, phase, status)) break;
        phase ^= 1u;
        bool special = false;
        if (k > 0) {
            hint = group_topk_row<G>(g, c, row, cols, k, out_idx + (size_t)r * k, out_val + (size_t)r * k, true, hint,
                                     &special);
        } else {
            float acc = 0.0f;
            const float4 *row4 = reinterpret_cast<const float4 *>(row);
            for (unsigned i = g.lane; i < (cols >> 2); i += RowGroup<G>::L) acc = absmax3_nan(acc, absmax4_nan(row4[i]), 0.0f);
            special = g.any(!(acc < __int_as_float(0x7f800000)), c);
        }
        if (DQ) {
            run = fmaxf(run, group_block_absmax<G>(g, row, cols, special, absmax_scratch + (size_t)r * blocks_per_row));
            fence_proxy_async_smem();
        } else {
            group_block_absmax<G>(g, row, cols, special, blk);
            g.sync();
            const bool slow = g.any(
                group_block_scales<G, false>(g, cols, 1.0f, nullptr, blk, scales_f32 + (size_t)r * blocks_per_row, nullptr), c);
            g.sync();
            group_encode<G>(g, row, cols, lut, blk, codes, slow);
            fence_proxy_async_smem();
            g.sync();
            if (g.lane == 0) {
                bulk_s2g(data + (size_t)r * (cols / 2), codes, cols / 2);
                bulk_commit();
                bulk_wait_read_all();
            }
        }
        g.sync();
    }
    if (DQ) {
        run = warp_max(run);
        if ((g.lane & 31) == 0 && run > 0.0f) atomicMax(gmax_bits, __float_as_uint(run));
    } else if (g.lane == 0) {
        bulk_wait_all();
    }
}

// Pass 2 of NF4_DQ: rows newest-first, zeroing re-applied from the row's k column indices.
template <int G>
__global__ void __launch_bounds__(512)
    frontend_pass2_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                          const uint16_t *__restrict__ idx, const float *__restrict__ absmax_scratch,
                          const unsigned *__restrict__ gmax_bits, float *__restrict__ dq_out,
                          uint8_t *__restrict__ scale_codes, uint8_t *__restrict__ data, unsigned *row_counter,
                          unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const RowGroup<G> g;
    const GroupLayout lay = group_layout(cols, true);
    unsigned char *base = smem_raw + (size_t)g.gid * lay.total;
    float *row = reinterpret_cast<float *>(base);
    uint16_t *codes = reinterpret_cast<uint16_t *>(base + lay.codes_off);
    float *blk = reinterpret_cast<float *>(base + lay.blk_off);
    GroupCtl &c = *reinterpret_cast<GroupCtl *>(base + lay.ctl_off);
    uint64_t *bar = reinterpret_cast<uint64_t *>(&c.bar);
    const unsigned bytes = cols * 4u, blocks_per_row = cols >> 6;
    Nf4Lut lut;
    lut.load();
    const float dq = dq_from_max(__uint_as_float(*gmax_bits));
    if (blockIdx.x == 0 && threadIdx.x == 0) *dq_out = dq;
    if (g.lane == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
    }
    g.sync();
    unsigned phase = 0;
    for (;;) {
        const unsigned rr = group_next_row<G>(g, c, row_counter);
        if (rr >= rows) break;
        const unsigned r = rows - 1u - rr;                   // newest rows of pass 1 first
        if (g.lane == 0) {
            mbar_expect_tx(bar, bytes);
            bulk_g2s(row, in + (size_t)r * cols, bytes, bar);
        }
        // the scale work does not need the row: do it while the copy is in flight
        const bool slow = g.any(group_block_scales<G, true>(g, cols, dq, absmax_scratch + (size_t)r * blocks_per_row, blk,
                                                            nullptr, scale_codes + (size_t)r * blocks_per_row), c);
        if (!group_wait_copy<G>(c, phase, status)) break;
        phase ^= 1u;
        for (unsigned j = g.lane; j < k; j += RowGroup<G>::L) {
            const unsigned col = idx[(size_t)r * k + j];
            if (col < cols) row[col] = 0.0f;
        }
        g.sync();
        group_encode<G>(g, row, cols, lut, blk, codes, slow);
        fence_proxy_async_smem();
        g.sync();
        if (g.lane == 0) {
            bulk_s2g(data + (size_t)r * (cols / 2), codes, cols / 2);
            bulk_commit();
            bulk_wait_read_all();
        }
        g.sync();
    }
    if (g.lane == 0) bulk_wait_all();
}

// Launch geometry: G warps per row so that a group never holds more than 16 KiB of row, as many
// groups per CTA as fit half of the SM's shared memory, two CTAs per SM.
struct FrontGeometry {
    int G, groups, threads;
    size_t smem;
};
FrontGeometry front_geometry(uint32_t cols, bool with_codes) {
    FrontGeometry f;
    f.G = cols <= 4096 ? 2 : (cols <= 8192 ? 4 : 8);      // measured on 4096-column rows: 2 warps per row is best
    if (const char *e = getenv("BSQ_FRONT_G")) {             // tuning override: warps per row
        const int v = atoi(e);
        if ((v == 1 || v == 2 || v == 4 || v == 8) && cols <= 4096u * (unsigned)v * 8u) f.G = v;
    }
    const size_t per_group = group_layout(cols, with_codes).total;
    int groups = (int)((110 * 1024) / per_group);
    groups = groups < 1 ? 1 : groups;
    const int max_by_threads = 512 / (32 * f.G), max_by_barriers = 15;      // kernels are built for <= 512 threads
    if (groups > max_by_threads) groups = max_by_threads;
    if (groups > max_by_barriers) groups = max_by_barriers;
    f.groups = groups;
    f.threads = groups * 32 * f.G;
    f.smem = per_group * groups;
    return f;
}

template <typename K>
cudaError_t persistent_grid(K kernel, int threads, size_t smem, int sm_count, unsigned rows, int groups, unsigned *grid_out) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (err != cudaSuccess) return err;
    int per_sm = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
    if (err != cudaSuccess) return err;
    if (per_sm < 1) per_sm = 1;
    unsigned grid = (unsigned)sm_count * (unsigned)per_sm;
    const unsigned needed = (rows + groups - 1) / groups;
    *grid_out = grid > needed ? needed : grid;
    return cudaSuccess;
}

template <int G>
cudaError_t launch_front(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                         float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                         void *d_scratch, unsigned *d_status, int sm_count, cudaStream_t stream, cudaEvent_t *events) {
    // scratch words: [0] global maximum, [1] row counter of pass 1, [2] row counter of pass 2
    unsigned *gmax = static_cast<unsigned *>(d_scratch);
    float *absmax = reinterpret_cast<float *>(static_cast<uint8_t *>(d_scratch) + 16);
    unsigned grid = 0;
    cudaError_t err = cudaMemsetAsync(gmax, 0, 16, stream);
    if (err != cudaSuccess) return err;
    if (method == 11) {
        const FrontGeometry f = front_geometry(cols, true);
        err = persistent_grid(frontend_pass1_kernel<G, false>, f.threads, f.smem, sm_count, rows, f.groups, &grid);
        if (err != cudaSuccess) return err;
        if (events) cudaEventRecord(events[0], stream);
        frontend_pass1_kernel<G, false><<<grid, f.threads, f.smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, d_scales_f32,
                                                                              d_data, nullptr, nullptr, gmax + 1, d_status);
        if (events) { cudaEventRecord(events[1], stream); cudaEventRecord(events[2], stream); }
        return cudaGetLastError();
    }
    const FrontGeometry f1 = front_geometry(cols, false), f2 = front_geometry(cols, true);
    err = persistent_grid(frontend_pass1_kernel<G, true>, f1.threads, f1.smem, sm_count, rows, f1.groups, &grid);
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[0], stream);
    frontend_pass1_kernel<G, true><<<grid, f1.threads, f1.smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, nullptr, nullptr,
                                                                           absmax, gmax, gmax + 1, d_status);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[1], stream);
    err = persistent_grid(frontend_pass2_kernel<G>, f2.threads, f2.smem, sm_count, rows, f2.groups, &grid);
    if (err != cudaSuccess) return err;
    frontend_pass2_kernel<G><<<grid, f2.threads, f2.smem, stream>>>(d_in, rows, cols, k, d_idx, absmax, gmax, d_dq,
                                                                     d_scale_codes, d_data, gmax + 2, d_status);
    if (events) cudaEventRecord(events[2], stream);
    return cudaGetLastError();
}

}  // namespace

bool frontend_supported(uint32_t rows, uint32_t cols, uint32_t k) {
    if (rows == 0 || cols == 0 || cols % 64 != 0 || k > (uint32_t)kCandCap || cols > 32768u) return false;
    return group_layout(cols, true).total <= 110 * 1024;
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
#define BSQ_FRONT(G_)                                                                                               \
    launch_front<G_>(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data, d_scratch, \
                     d_status, sm_count, stream, events)
    switch (front_geometry(cols, true).G) {
        case 1: return BSQ_FRONT(1);
        case 2: return BSQ_FRONT(2);
        case 4: return BSQ_FRONT(4);
        default: return BSQ_FRONT(8);
    }
#undef BSQ_FRONT
}

}  // namespace bsq
