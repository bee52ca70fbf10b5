// Per-row ordered top-k of |x| (outlier separation and error-correction extraction), the
// scatter-add that undoes it, and the residual/any-nonzero helper (sm_100a).
//
// Replaces build_sort_inputs_kernel + cub::DeviceSegmentedRadixSort::SortPairsDescending +
// gather_topk_kernel + zero_selected_entries_kernel and scatter_add_topk_kernel
// (modules/topk_cuda/src/topk_cuda_utils.cuh:51-149,254-295; entry points
// modules/topk_cuda/src/topk_cuda.cu:186-233), and subtract_kernel / has_nonzero_kernel
// (src/bitsqz_llm.cu:164-184).  The reference sorts every row completely to keep ~1 % of it;
// here a row is read once from HBM into shared memory by a bulk (TMA) copy, selected and
// sorted there (bsq_topk.cuh), and only the k pairs -- and, for separation, the row with the
// selected entries zeroed -- are written back.  HBM-bound: 4 B read per element, 6k B written
// per row (+ 4 B per element when the zeroed copy is wanted).
#include "bsq_internal.hpp"
#include "bsq_rowgroup.cuh"
#include "bsq_topk.cuh"

#include <math.h>

namespace bsq {
namespace {

// ---- rows that fit shared memory: cols % 4 == 0, k <= kCandCap, 16-byte aligned rows ----------
// One group of G warps per row (bsq_rowgroup.cuh); a CTA holds several groups, rows are dealt out
// round-robin over all groups of the grid.
template <int G>
__global__ void __launch_bounds__(512)
    topk_rows_group_kernel(const float *__restrict__ in, float *residual, unsigned rows, unsigned cols, unsigned k,
                           uint16_t *__restrict__ out_idx, float *__restrict__ out_val, unsigned *status, unsigned group_bytes,
                           unsigned ctl_off, unsigned *bound) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const RowGroup<G> g;
    unsigned char *base = smem_raw + (size_t)g.gid * group_bytes;
    float *row = reinterpret_cast<float *>(base);
    GroupCtl &c = *reinterpret_cast<GroupCtl *>(base + ctl_off);
    uint64_t *bar = reinterpret_cast<uint64_t *>(&c.bar);
    const unsigned bytes = cols * 4u;
    const unsigned groups_per_cta = blockDim.x / RowGroup<G>::L;
    if (g.lane == 0) {
        mbar_init(bar, 1);
        mbar_fence_init();
        c.wait_failed = 0;
    }
    g.sync();
    unsigned phase = 0;
    float hint = 0.0f;
    const unsigned row_step = gridDim.x * groups_per_cta;
    bool next_loading = false;                               // uniform over the group: the copy of row r is already on its way
    for (unsigned r = blockIdx.x * groups_per_cta + g.gid; r < rows; r += row_step) {
        if (g.lane == 0 && !next_loading) {
            mbar_expect_tx(bar, bytes);
            bulk_g2s(row, in + (size_t)r * cols, bytes, bar);
        }
        next_loading = false;
        // the outcome of the wait must be the same for every lane of the group (they meet at group barriers below):
        // a lane whose wait ran out says so, and all lanes read the same flag after a group barrier
        if (!mbar_wait_bounded(bar, phase, status)) c.wait_failed = 1;
        g.sync();
        if (c.wait_failed) break;
        phase ^= 1u;
        bool special = false;
        // Extraction only (no zeroed copy wanted): once the candidates and their values are out of the row, the next
        // row's copy starts into the same buffer while this row's candidates are still ranked and written out.
        auto row_free = [&]() {
            if (r + row_step < rows) {
                fence_proxy_async_smem();
                g.sync();
                if (g.lane == 0) {
                    mbar_expect_tx(bar, bytes);
                    bulk_g2s(row, in + (size_t)(r + row_step) * cols, bytes, bar);
                }
                next_loading = true;
            }
        };
        hint = group_topk_row<G>(g, c, row, cols, k, out_idx + (size_t)r * k, out_val + (size_t)r * k, residual != nullptr,
                                 hint, &special, row_free);
        if (bound && g.lane == 0) atomicMax(bound, c.kth_bits);          // (published before the function's last group sync)
        fence_proxy_async_smem();
        g.sync();
        if (residual != nullptr && g.lane == 0) {
            bulk_s2g(residual + (size_t)r * cols, row, bytes);
            bulk_commit();
            bulk_wait_read_all();
        }
        g.sync();
    }
    if (g.lane == 0) bulk_wait_all();
}

// ---- any shape: row stays in global memory (L2), k up to cols -----------------------------------
constexpr int kGenericThreads = 256;
constexpr int kGenericSortCap = 2048;

struct GenericSmem {
    TopkScratch s;
    unsigned long long list[kGenericSortCap];
};

// CTA-wide bitonic sort (descending) of n2 (power of two, <= kGenericSortCap) composites.
__device__ void block_bitonic_desc(unsigned long long *a, unsigned n2) {
    for (unsigned size = 2; size <= n2; size <<= 1) {
        for (unsigned stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (unsigned t = threadIdx.x; t < n2 / 2; t += blockDim.x) {
                const unsigned i = 2 * t - (t & (stride - 1));      // lower index of the pair
                const unsigned j = i + stride;
                const bool desc = (i & size) == 0;
                const unsigned long long x = a[i], y = a[j];
                if (desc ? (x < y) : (x > y)) { a[i] = y; a[j] = x; }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kGenericThreads)
    topk_rows_generic_kernel(const float *in, float *residual, unsigned rows, unsigned cols, unsigned k,
                             uint16_t *__restrict__ out_idx, float *__restrict__ out_val) {
    __shared__ GenericSmem g;
    TopkScratch &s = g.s;
    const int tid = threadIdx.x;
    for (unsigned r = blockIdx.x; r < rows; r += gridDim.x) {
        const float *row = in + (size_t)r * cols;
        uint16_t *oi = out_idx + (size_t)r * k;
        float *ov = out_val + (size_t)r * k;
        // radix select over the 48-bit composite, most significant byte first
        unsigned long long prefix = 0;
        unsigned need = k;
        for (int pass = 0; pass < 6; ++pass) {
            const int shift = 40 - 8 * pass;
            for (int i = tid; i < 256; i += kGenericThreads) s.hist[i] = 0;
            __syncthreads();
            for (unsigned c = tid; c < cols; c += kGenericThreads) {
                const unsigned long long comp = topk_composite(row[c], c);
                if (pass == 0 || (comp >> (shift + 8)) == (prefix >> (shift + 8)))
                    atomicAdd(&s.hist[(unsigned)(comp >> shift) & 0xFFu], 1u);
            }
            __syncthreads();
            if (tid < 32) hist_select_warp(s, need);
            __syncthreads();
            prefix |= (unsigned long long)s.sel_bin << shift;
            need = s.sel_need;
        }
        if (k <= kGenericSortCap) {
            unsigned n2 = 2;
            while (n2 < k) n2 <<= 1;
            for (unsigned i = tid; i < n2; i += kGenericThreads) g.list[i] = 0ull;
            if (tid == 0) s.count = 0;
            __syncthreads();
            for (unsigned c = tid; c < cols; c += kGenericThreads) {
                const unsigned long long comp = topk_composite(row[c], c);
                if (comp >= prefix) {
                    const unsigned pos = atomicAdd(&s.count, 1u);
                    if (pos < kGenericSortCap) g.list[pos] = comp;
                }
            }
            block_bitonic_desc(g.list, n2);
            for (unsigned j = tid; j < k; j += kGenericThreads) {
                const unsigned col = 0xFFFFu - (unsigned)(g.list[j] & 0xFFFFull);
                oi[j] = (uint16_t)col;
                ov[j] = row[col];
            }
        } else {
            // very large k: rank every selected element by counting the composites above it
            for (unsigned c = tid; c < cols; c += kGenericThreads) {
                const unsigned long long comp = topk_composite(row[c], c);
                if (comp < prefix) continue;
                unsigned rank = 0;
                for (unsigned d = 0; d < cols; ++d) rank += topk_composite(row[d], d) > comp ? 1u : 0u;
                oi[rank] = (uint16_t)c;
                ov[rank] = row[c];
            }
        }
        __syncthreads();
        if (residual != nullptr) {
            float *dst = residual + (size_t)r * cols;
            if (dst != row) {
                for (unsigned c = tid; c < cols; c += kGenericThreads) dst[c] = row[c];
                __syncthreads();
            }
            for (unsigned j = tid; j < k; j += kGenericThreads) dst[oi[j]] = 0.0f;
        }
        __syncthreads();
    }
}

// ---- scatter-add ----------------------------------------------------------------------------------
__global__ void topk_apply_kernel(const uint16_t *__restrict__ idx, const float *__restrict__ val, unsigned rows,
                                  unsigned cols, unsigned k, float *dense, unsigned *status) {
    const size_t total = (size_t)rows * k;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        const unsigned r = (unsigned)(e / k);
        const unsigned c = idx[e];
        if (c < cols) dense[(size_t)r * cols + c] += val[e];
        else if (status) atomicOr(status, kStatusBadIndex);
    }
}

// ---- e = a - b, flag |= any(|e| > FLT_EPSILON) ----------------------------------------------------
__global__ void __launch_bounds__(256)
    residual_error_kernel(const float *__restrict__ a, const float *__restrict__ b, uint64_t n, bool vec,
                          float *__restrict__ e, unsigned *flag) {
    bool any = false;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t t0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        const uint64_t n4 = n / 4;
        for (uint64_t i = t0; i < n4; i += stride) {
            const float4 x = __ldcs(reinterpret_cast<const float4 *>(a) + i);
            const float4 y = __ldcs(reinterpret_cast<const float4 *>(b) + i);
            const float4 d = make_float4(__fsub_rn(x.x, y.x), __fsub_rn(x.y, y.y), __fsub_rn(x.z, y.z), __fsub_rn(x.w, y.w));
            any |= abs4max(d) > 1.1920928955078125e-07f;
            reinterpret_cast<float4 *>(e)[i] = d;
        }
        for (uint64_t i = n4 * 4 + t0; i < n; i += stride) {
            const float d = __fsub_rn(a[i], b[i]);
            any |= fabsf(d) > 1.1920928955078125e-07f;
            e[i] = d;
        }
    } else {
        for (uint64_t i = t0; i < n; i += stride) {
            const float d = __fsub_rn(a[i], b[i]);
            any |= fabsf(d) > 1.1920928955078125e-07f;
            e[i] = d;
        }
    }
    if (__any_sync(kFullMask, any) && (threadIdx.x & 31) == 0) atomicOr(flag, 1u);
}

}  // namespace

int device_sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
    return sms;
}

int topk_num_columns(uint16_t cols, float ratio) {
    if (cols == 0) return 0;
    if (!(ratio >= 0.0f && ratio <= 1.0f)) return -1;
    const float raw = (float)cols * ratio;
    uint16_t k = (uint16_t)roundf(raw);
    if (k > cols) k = cols;
    else if (k == 0 && ratio > 0.0f) k = 1;
    return k;
}

// Geometry of the group kernel: G warps per row (a group never holds more than 16 KiB of row per warp
// pair), as many groups per CTA as fit half of an SM's shared memory.
struct GroupGeometry {
    int G, groups, threads;
    unsigned group_bytes, ctl_off;
};
static GroupGeometry group_geometry(uint32_t cols) {
    GroupGeometry f;
    f.G = cols <= 4096 ? 2 : (cols <= 8192 ? 4 : 8);
    f.ctl_off = (cols * 4u + 15u) & ~15u;
    f.group_bytes = (f.ctl_off + (unsigned)sizeof(GroupCtl) + 127u) & ~127u;
    int groups = (int)((110u * 1024u) / f.group_bytes);
    if (groups < 1) groups = 1;
    if (groups > 512 / (32 * f.G)) groups = 512 / (32 * f.G);
    if (groups > 15) groups = 15;
    f.groups = groups;
    f.threads = groups * 32 * f.G;
    return f;
}

bool topk_rows_fit_smem(const void *d_in, const void *d_residual, uint32_t cols, uint32_t k) {
    if (cols % 4 != 0 || k == 0 || k > (uint32_t)kCandCap || cols > 24576u) return false;
    if (group_geometry(cols).group_bytes > 110u * 1024u) return false;
    if (reinterpret_cast<uintptr_t>(d_in) % 16 != 0) return false;
    if (d_residual && reinterpret_cast<uintptr_t>(d_residual) % 16 != 0) return false;
    return true;
}

template <int G>
static cudaError_t launch_group(const float *d_in, float *d_residual, uint32_t rows, uint32_t cols, uint32_t k,
                                uint16_t *d_idx, float *d_val, unsigned *d_status, int sm_count, cudaStream_t stream, unsigned *d_bound) {
    const GroupGeometry f = group_geometry(cols);
    const size_t smem = (size_t)f.group_bytes * f.groups;
    cudaError_t err = cudaFuncSetAttribute(topk_rows_group_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    err = cudaFuncSetAttribute(topk_rows_group_kernel<G>, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    if (err != cudaSuccess) return err;
    int per_sm = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, topk_rows_group_kernel<G>, f.threads, smem);
    if (err != cudaSuccess) return err;
    if (per_sm < 1) per_sm = 1;
    unsigned grid = (unsigned)sm_count * (unsigned)per_sm;
    const unsigned needed = (rows + f.groups - 1) / f.groups;
    if (grid > needed) grid = needed;
    topk_rows_group_kernel<G><<<grid, f.threads, smem, stream>>>(d_in, d_residual, rows, cols, k, d_idx, d_val, d_status,
                                                                  f.group_bytes, f.ctl_off, d_bound);
    return cudaGetLastError();
}

cudaError_t topk_rows(const float *d_in, float *d_residual, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                      float *d_val, unsigned *d_status, int sm_count, cudaStream_t stream, unsigned *d_bound, bool *bound_written) {
    if (bound_written) *bound_written = false;
    if (!d_in || rows == 0 || cols == 0 || cols > 65535u || k > cols) return cudaErrorInvalidValue;
    if (k == 0) {
        if (d_residual && d_residual != d_in)
            return cudaMemcpyAsync(d_residual, d_in, (size_t)rows * cols * 4, cudaMemcpyDeviceToDevice, stream);
        return cudaSuccess;
    }
    if (!d_idx || !d_val) return cudaErrorInvalidValue;
    if (topk_rows_fit_smem(d_in, d_residual, cols, k)) {
        if (d_bound) {
            const cudaError_t e = cudaMemsetAsync(d_bound, 0, sizeof(unsigned), stream);
            if (e != cudaSuccess) return e;
            if (bound_written) *bound_written = true;
        }
        switch (group_geometry(cols).G) {
            case 2: return launch_group<2>(d_in, d_residual, rows, cols, k, d_idx, d_val, d_status, sm_count, stream, d_bound);
            case 4: return launch_group<4>(d_in, d_residual, rows, cols, k, d_idx, d_val, d_status, sm_count, stream, d_bound);
            default: return launch_group<8>(d_in, d_residual, rows, cols, k, d_idx, d_val, d_status, sm_count, stream, d_bound);
        }
    }
    unsigned grid = (unsigned)sm_count * 8u;
    if (grid > rows) grid = rows;
    topk_rows_generic_kernel<<<grid, kGenericThreads, 0, stream>>>(d_in, d_residual, rows, cols, k, d_idx, d_val);
    return cudaGetLastError();
}

cudaError_t topk_apply(const uint16_t *d_idx, const float *d_val, uint32_t rows, uint32_t cols, uint32_t k,
                       float *d_dense, unsigned *d_status, cudaStream_t stream) {
    if (!d_dense || rows == 0 || cols == 0) return cudaErrorInvalidValue;
    if (k == 0) return cudaSuccess;
    if (!d_idx || !d_val) return cudaErrorInvalidValue;
    const size_t total = (size_t)rows * k;
    size_t grid = (total + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    topk_apply_kernel<<<(unsigned)grid, 256, 0, stream>>>(d_idx, d_val, rows, cols, k, d_dense, d_status);
    return cudaGetLastError();
}

cudaError_t residual_error(const float *d_a, const float *d_b, uint64_t n, float *d_e, unsigned *d_flag, int sm_count,
                           cudaStream_t stream) {
    if (!d_a || !d_b || !d_e || !d_flag || n == 0) return cudaErrorInvalidValue;
    const bool vec = ((reinterpret_cast<uintptr_t>(d_a) | reinterpret_cast<uintptr_t>(d_b) |
                       reinterpret_cast<uintptr_t>(d_e)) % 16) == 0;
    uint64_t grid = (n / 4 + 255) / 256;
    const uint64_t cap = (uint64_t)sm_count * 8;
    if (grid > cap) grid = cap;
    if (grid == 0) grid = 1;
    residual_error_kernel<<<(unsigned)grid, 256, 0, stream>>>(d_a, d_b, n, vec, d_e, d_flag);
    return cudaGetLastError();
}

}  // namespace bsq
