// Fused front end of the no-SVD compress path: per-row outlier separation followed by NF4 or
// NF4_DQ of the remainder, without ever writing the zeroed matrix to HBM (sm_100a).
//
// The reference runs, for this path, a device-to-device copy of the whole input, the top-k module
// (three kernels around a full segmented sort) and the quantiser (one kernel for NF4, four for
// NF4_DQ), each separated by a device synchronisation (src/bitsqz_llm.cu:1036-1056,1183-1195;
// modules/topk_cuda/src/topk_cuda_utils.cuh:275-295; modules/quantization_cuda/src/
// quantization_cuda.cu:564-624).  Here a group of G warps streams one row from global memory
// (bsq_rowstream.cuh: 8 float4 per lane in flight, nothing of the row kept in shared memory):
//   * NF4_DQ, kernel 1 (frontend_select_kernel): one sweep selects the row's outliers and gets the
//     64-element block maxima of what remains (4 B per block written), folded into one global maximum;
//   * NF4_DQ, kernel 2 (frontend_encode_kernel), launched right behind: re-reads the rows newest first,
//     so that most of them are still in L2, encodes against dq * e4m3(absmax / dq), patches the
//     row's k selected columns to the code of 0.0 and sends the nibbles out by a bulk store;
//   * NF4 (frontend_nf4_kernel): both steps back to back on one row in one kernel (the second read
//     of the row comes from L1 / L2).
// Rows are a multiple of 64 long, so NF4 blocks never straddle rows.  Rows are handed to the groups
// through an atomic counter whose next value is requested one row ahead.
#include "bsq_internal.hpp"
#include "bsq_rowstream.cuh"

#include <cstdlib>
#include <mutex>
#include <vector>

namespace bsq {
namespace {

// Shared memory of one group: control | one word per block | selection bitmap | nibble staging buffers.
struct StreamLayout {
    size_t blk_off, bitmap_off, codes_off, codes_stride, total;
};
__host__ __device__ inline StreamLayout stream_layout(unsigned cols, int code_buffers) {
    StreamLayout l;
    l.blk_off = (sizeof(GroupCtl) + 15) & ~(size_t)15;
    l.bitmap_off = l.blk_off + (((size_t)(cols / 64) * 4 + 15) & ~(size_t)15);
    l.codes_off = l.bitmap_off + (((size_t)((cols + 31) / 32) * 4 + 15) & ~(size_t)15);
    l.codes_stride = ((size_t)cols / 2 + 15) & ~(size_t)15;
    l.total = (l.codes_off + l.codes_stride * code_buffers + 127) & ~(size_t)127;
    return l;
}

// Row hand-out: a group's first row is its own number among the grid's groups (no atomic: all groups starting at once
// on one counter would queue up for microseconds); further rows come from a global counter, offset by the number of
// groups.  Lane 0 keeps the value it asked for one row ago (`pending`), publishes it and asks for the next, so that
// the latency of the global atomic never shows; also clears the row flags.  Returns the row (uniform; >= rows: no
// work left).
template <int G>
__device__ __forceinline__ unsigned first_row_of_group(const RowGroup<G> &g) {
    return blockIdx.x * (blockDim.x / RowGroup<G>::L) + g.gid;
}
template <int G>
__device__ __forceinline__ unsigned stream_next_row(const RowGroup<G> &g, GroupCtl &c, unsigned *row_counter, unsigned &pending,
                                                    unsigned rows) {
    if (g.lane == 0) {
        c.next_row = pending;
        c.flags = 0;
        if (pending < rows) pending = gridDim.x * (blockDim.x / RowGroup<G>::L) + atomicAdd(row_counter, 1u);
    }
    g.sync();
    return c.next_row;
}

// The selection bound that the last launch on this scratch area left behind (a group's first row otherwise has to
// work one out with a sweep of its own, and a group sees only three or four rows of a 4096-row matrix).  Any value
// is safe: the bound only says where to look for candidates, a row that finds fewer than k above it (or too many)
// works out its own; the pairs written never depend on it.
__device__ __forceinline__ float carried_hint(const unsigned *hint_word) {
    const float h = __uint_as_float(*hint_word);
    return (h > 0.0f && h < __int_as_float(0x7f800000)) ? h : 0.0f;
}

// NF4_DQ kernel 1: selection + block maxima + global maximum.
template <int G>
__global__ void __launch_bounds__(256, 4)
    frontend_select_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                           uint16_t *__restrict__ out_idx, float *__restrict__ out_val, float *__restrict__ absmax_scratch,
                           unsigned *gmax_bits, unsigned *row_counter, unsigned *hint_word) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const RowGroup<G> g;
    const StreamLayout lay = stream_layout(cols, 0);
    unsigned char *base = smem_raw + (size_t)g.gid * lay.total;
    GroupCtl &c = *reinterpret_cast<GroupCtl *>(base);
    unsigned *blk = reinterpret_cast<unsigned *>(base + lay.blk_off);
    unsigned *bitmap = reinterpret_cast<unsigned *>(base + lay.bitmap_off);
    const unsigned blocks_per_row = cols >> 6;
    unsigned pending = first_row_of_group<G>(g);
    float run = 0.0f, hint = k > 0 ? carried_hint(hint_word) : 0.0f;
    bool fresh = false;                                      // the row before has left the control block clean
    for (;;) {
        const unsigned r = stream_next_row<G>(g, c, row_counter, pending, rows);
        if (r >= rows) break;
        hint = stream_select_absmax<G>(g, c, blk, bitmap, GlobalRow{in + (size_t)r * cols}, cols, k, out_idx + (size_t)r * k,
                                       out_val + (size_t)r * k, hint, absmax_scratch + (size_t)r * blocks_per_row, &run, fresh,
                                       true, true);
        fresh = true;
    }
    if (g.lane == 0 && hint > 0.0f) *hint_word = __float_as_uint(hint);      // whichever group writes last: all are usable
    run = warp_max(run);
    if ((g.lane & 31) == 0 && run > 0.0f) atomicMax(gmax_bits, __float_as_uint(run));
}

// Encode one row whose +-1/scale per block is in blkf[] and send it out; `codes` is the staging buffer of this row,
// `first` the row's first chunk and `sel` its selected columns, both loaded earlier.
template <int G, class Row>
__device__ __forceinline__ void encode_and_store(const RowGroup<G> &g, GroupCtl &c, const Row &row, unsigned cols,
                                                 const float4 (&first)[kChunk], const Nf4Lut &lut, const float *blkf,
                                                 uint16_t *codes, const SelectedCols<G> &sel, uint8_t *dst) {
    stream_encode<G>(g, row, cols, first, lut, blkf, codes, (c.flags & kFlagSlow) != 0);
    stream_patch_selected<G>(g, codes, sel, cols);
    fence_proxy_async_smem();
    g.sync();
    if (g.lane == 0) {
        bulk_s2g(dst, codes, cols / 2);
        bulk_commit();
    }
}

// NF4_DQ kernel 2: rows newest-first.
template <int G>
__global__ void __launch_bounds__(256, 4)
    frontend_encode_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k,
                           const uint16_t *__restrict__ idx, const float *__restrict__ absmax_scratch,
                           const unsigned *__restrict__ gmax_bits, float *__restrict__ dq_out,
                           uint8_t *__restrict__ scale_codes, uint8_t *__restrict__ data, unsigned *row_counter) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const RowGroup<G> g;
    const StreamLayout lay = stream_layout(cols, 2);
    unsigned char *base = smem_raw + (size_t)g.gid * lay.total;
    GroupCtl &c = *reinterpret_cast<GroupCtl *>(base);
    float *blkf = reinterpret_cast<float *>(base + lay.blk_off);
    const unsigned blocks_per_row = cols >> 6;
    Nf4Lut lut;
    lut.load();
    const float dq = dq_from_max(__uint_as_float(*gmax_bits));
    if (blockIdx.x == 0 && threadIdx.x == 0) *dq_out = dq;
    unsigned buf = 0;
    unsigned pending = first_row_of_group<G>(g);
    for (;;) {
        if (g.lane == 0) bulk_wait_read_1();                 // the store issued two rows ago has left its staging buffer
        const unsigned rr = stream_next_row<G>(g, c, row_counter, pending, rows);
        if (rr >= rows) break;
        const unsigned r = rows - 1u - rr;                   // newest rows of kernel 1 first
        // everything the row needs from global memory is asked for at once: its data, its columns, its block maxima
        const GlobalRow row{in + (size_t)r * cols};
        float4 first[kChunk];
        load_first_chunk<G>(g, row, cols >> 2, first);
        SelectedCols<G> sel;
        load_selected<G>(g, idx + (size_t)r * k, k, sel);
        if (group_block_scales<G, true>(g, cols, dq, absmax_scratch + (size_t)r * blocks_per_row, blkf, nullptr,
                                        scale_codes + (size_t)r * blocks_per_row))
            atomicOr(&c.flags, kFlagSlow);
        g.sync();
        uint16_t *codes = reinterpret_cast<uint16_t *>(base + lay.codes_off + buf * lay.codes_stride);
        encode_and_store<G>(g, c, row, cols, first, lut, blkf, codes, sel, data + (size_t)r * (cols / 2));
        buf ^= 1u;
    }
    if (g.lane == 0) bulk_wait_all();
}

// NF4: selection, block scales and nibbles of a row in one go.
template <int G>
__global__ void __launch_bounds__(256, 2)
    frontend_nf4_kernel(const float *__restrict__ in, unsigned rows, unsigned cols, unsigned k, uint16_t *__restrict__ out_idx,
                        float *__restrict__ out_val, float *__restrict__ scales_f32, uint8_t *__restrict__ data,
                        unsigned *row_counter, unsigned *hint_word) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const RowGroup<G> g;
    const StreamLayout lay = stream_layout(cols, 2);
    unsigned char *base = smem_raw + (size_t)g.gid * lay.total;
    GroupCtl &c = *reinterpret_cast<GroupCtl *>(base);
    unsigned *blk = reinterpret_cast<unsigned *>(base + lay.blk_off);
    float *blkf = reinterpret_cast<float *>(blk);
    unsigned *bitmap = reinterpret_cast<unsigned *>(base + lay.bitmap_off);
    const unsigned blocks_per_row = cols >> 6;
    Nf4Lut lut;
    lut.load();
    unsigned buf = 0;
    unsigned pending = first_row_of_group<G>(g);
    float run = 0.0f, hint = k > 0 ? carried_hint(hint_word) : 0.0f;
    for (;;) {
        if (g.lane == 0) bulk_wait_read_1();
        const unsigned r = stream_next_row<G>(g, c, row_counter, pending, rows);
        if (r >= rows) break;
        const GlobalRow row{in + (size_t)r * cols};
        hint = stream_select_absmax<G>(g, c, blk, bitmap, row, cols, k, out_idx + (size_t)r * k, out_val + (size_t)r * k, hint,
                                       nullptr, &run);
        if (group_block_scales<G, false>(g, cols, 1.0f, nullptr, blkf, scales_f32 + (size_t)r * blocks_per_row, nullptr))
            atomicOr(&c.flags, kFlagSlow);
        g.sync();
        uint16_t *codes = reinterpret_cast<uint16_t *>(base + lay.codes_off + buf * lay.codes_stride);
        float4 first[kChunk];
        load_first_chunk<G>(g, row, cols >> 2, first);
        SelectedCols<G> sel;
        load_selected<G>(g, out_idx + (size_t)r * k, k, sel);    // written by this group before its last sync
        encode_and_store<G>(g, c, row, cols, first, lut, blkf, codes, sel, data + (size_t)r * (cols / 2));
        buf ^= 1u;
    }
    if (g.lane == 0 && hint > 0.0f) *hint_word = __float_as_uint(hint);
    if (g.lane == 0) bulk_wait_all();
}

// Launch geometry: G warps per row, 256 threads per CTA, as many CTAs per SM as registers and shared memory allow.
struct FrontGeometry {
    int G, groups, threads;
    size_t smem;
};
FrontGeometry front_geometry(uint32_t cols, int code_buffers) {
    FrontGeometry f;
    f.G = cols <= 2048 ? 2 : (cols <= 8192 ? 4 : 8);        // measured on 4096-column rows: 4 warps per row is best
    static const int forced_g = [] {                         // tuning override, read once: warps per row
        const char *e = getenv("BSQ_FRONT_G");
        const int v = e ? atoi(e) : 0;
        return (v == 1 || v == 2 || v == 4 || v == 8) ? v : 0;
    }();
    if (forced_g) f.G = forced_g;
    f.threads = 256;
    f.groups = f.threads / (32 * f.G);
    f.smem = stream_layout(cols, code_buffers).total * f.groups;
    return f;
}

// CTAs that fill the device for `kernel` with this much dynamic shared memory.  The attribute call and the occupancy
// query cost microseconds of host time each, a tenth of what the stage itself takes, so their answer is kept per
// (device, kernel, shared-memory size).
template <typename K>
cudaError_t persistent_grid(K kernel, int threads, size_t smem, int sm_count, unsigned rows, int groups, unsigned *grid_out) {
    struct Known {
        int device;
        const void *kernel;
        size_t smem;
        int per_sm;
    };
    static std::mutex lock;
    static std::vector<Known> known;
    int device = 0, per_sm = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    {
        std::lock_guard<std::mutex> hold(lock);
        for (const Known &e : known)
            if (e.device == device && e.kernel == reinterpret_cast<const void *>(kernel) && e.smem == smem) per_sm = e.per_sm;
    }
    if (per_sm == 0) {
        size_t largest = smem;                               // the attribute is only ever raised: sizes asked for earlier stay valid
        {
            std::lock_guard<std::mutex> hold(lock);
            for (const Known &e : known)
                if (e.device == device && e.kernel == reinterpret_cast<const void *>(kernel) && e.smem > largest) largest = e.smem;
        }
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)largest);
        if (err != cudaSuccess) return err;
        err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem);
        if (err != cudaSuccess) return err;
        if (per_sm < 1) per_sm = 1;
        std::lock_guard<std::mutex> hold(lock);
        known.push_back({device, reinterpret_cast<const void *>(kernel), smem, per_sm});
    }
    unsigned grid = (unsigned)sm_count * (unsigned)per_sm;
    const unsigned needed = (rows + groups - 1) / groups;
    *grid_out = grid > needed ? needed : grid;
    return cudaSuccess;
}

template <int G>
cudaError_t launch_front(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                         float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                         void *d_scratch, int sm_count, cudaStream_t stream, cudaEvent_t *events) {
    // scratch words: [0] global maximum, [1] row counter of kernel 1, [2] row counter of kernel 2 (cleared per call),
    // [3] the selection bound carried from call to call (never cleared; see carried_hint)
    unsigned *gmax = static_cast<unsigned *>(d_scratch);
    float *absmax = reinterpret_cast<float *>(static_cast<uint8_t *>(d_scratch) + 16);
    unsigned grid = 0;
    cudaError_t err = cudaMemsetAsync(gmax, 0, 12, stream);
    if (err != cudaSuccess) return err;
    if (method == 11) {
        const FrontGeometry f = front_geometry(cols, 2);
        err = persistent_grid(frontend_nf4_kernel<G>, f.threads, f.smem, sm_count, rows, f.groups, &grid);
        if (err != cudaSuccess) return err;
        if (events) cudaEventRecord(events[0], stream);
        frontend_nf4_kernel<G><<<grid, f.threads, f.smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_data,
                                                                    gmax + 1, gmax + 3);
        if (events) { cudaEventRecord(events[1], stream); cudaEventRecord(events[2], stream); }
        return cudaGetLastError();
    }
    const FrontGeometry f1 = front_geometry(cols, 0), f2 = front_geometry(cols, 2);
    err = persistent_grid(frontend_select_kernel<G>, f1.threads, f1.smem, sm_count, rows, f1.groups, &grid);
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[0], stream);
    frontend_select_kernel<G><<<grid, f1.threads, f1.smem, stream>>>(d_in, rows, cols, k, d_idx, d_val, absmax, gmax, gmax + 1,
                                                                     gmax + 3);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    if (events) cudaEventRecord(events[1], stream);
    err = persistent_grid(frontend_encode_kernel<G>, f2.threads, f2.smem, sm_count, rows, f2.groups, &grid);
    if (err != cudaSuccess) return err;
    frontend_encode_kernel<G><<<grid, f2.threads, f2.smem, stream>>>(d_in, rows, cols, k, d_idx, absmax, gmax, d_dq,
                                                                      d_scale_codes, d_data, gmax + 2);
    if (events) cudaEventRecord(events[2], stream);
    return cudaGetLastError();
}

}  // namespace

bool frontend_supported(uint32_t rows, uint32_t cols, uint32_t k) {
    if (rows == 0 || cols == 0 || cols % 64 != 0 || k > (uint32_t)kCandCap || cols > 65472u) return false;
    return front_geometry(cols, 2).smem <= 200 * 1024;
}

size_t frontend_scratch_bytes(uint32_t rows, uint32_t cols) { return 16 + (size_t)rows * (cols / 64) * sizeof(float); }

cudaError_t frontend_quantize(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                              float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                              void *d_scratch, unsigned *d_status, int sm_count, cudaStream_t stream,
                              cudaEvent_t *events) {
    (void)d_status;                                          // these kernels wait on nothing
    if (!frontend_supported(rows, cols, k) || (method != 10 && method != 11)) return cudaErrorInvalidValue;
    if (!d_in || !d_data || (k > 0 && (!d_idx || !d_val))) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(d_in) % 16) || (reinterpret_cast<uintptr_t>(d_data) % 16)) return cudaErrorInvalidValue;
    if (!d_scratch || (method == 10 && (!d_dq || !d_scale_codes))) return cudaErrorInvalidValue;
    if (method == 11 && !d_scales_f32) return cudaErrorInvalidValue;
#define BSQ_FRONT(G_)                                                                                               \
    launch_front<G_>(method, d_in, rows, cols, k, d_idx, d_val, d_scales_f32, d_dq, d_scale_codes, d_data, d_scratch, \
                     sm_count, stream, events)
    switch (front_geometry(cols, 2).G) {
        case 1: return BSQ_FRONT(1);
        case 2: return BSQ_FRONT(2);
        case 4: return BSQ_FRONT(4);
        default: return BSQ_FRONT(8);
    }
#undef BSQ_FRONT
}

}  // namespace bsq
