// Block-level routines for ordered per-row top-k on a row that sits in shared memory.
//
// Contract (reference modules/topk_cuda/src/topk_cuda_utils.cuh:51-93,254-295): the k entries
// with the largest key |x| (NaN ranks below every number, +0 == -0), emitted in the order
// (key descending, column ascending), values with their original sign and bits.
//
// Both routines work on a 48-bit "composite" per element,
//     composite = ukey << 16 | (0xFFFF - column),  ukey = NaN ? 0 : bits(|x|) + 1,
// whose descending order is exactly the reference order and which is unique per column, so
// "the k largest composites, sorted" is the whole specification.
//
//  * topk_fast(): the usual case (k small against cols, few ties).  Each thread takes the
//    maximum |x| of its share of the row; a two-round 256-bin histogram over those per-thread
//    maxima (8 exponent bits, then 8 mantissa bits) gives a bound L that at least k threads
//    reach, hence at least k elements.  Elements >= L are the candidates (about k of them);
//    one warp sorts them in registers with a bitonic network and emits the first k.  One
//    shared-memory atomic per THREAD instead of one per element.
//  * topk_exact(): always right, slower.  6 passes of 8-bit radix select over the composite
//    (most significant digit first) find the k-th largest composite; everything >= it is
//    gathered and sorted the same way.  Taken when the fast path sees more than kCandCap
//    candidates (heavy ties, rows of zeros) -- NaN needs no special case in either path.
#pragma once

#include "bsq_device.cuh"

#ifdef BSQ_TRACE
static __device__ long long g_trace_topk[16];
#define BSQ_TT(slot) do { if (blockIdx.x == 5 && threadIdx.x == 0) g_trace_topk[slot] = clock64(); } while (0)
#else
#define BSQ_TT(slot) do { } while (0)
#endif

namespace bsq {

constexpr int kCandCap = 256;              // candidate slots; also the largest k these routines take

struct TopkScratch {                       // per-CTA shared-memory scratch
    unsigned hist[256];
    unsigned long long cand[kCandCap];
    unsigned dirty[256];                   // one bit per float4 of the row: holds an entry that was zeroed
    unsigned count;                        // candidates appended
    unsigned kth_bits;                     // |x| bits of the k-th entry of the row just finished
    unsigned sel_bin;                      // histogram search result
    unsigned sel_need;
    unsigned sel_ok;
};

__device__ __forceinline__ unsigned long long topk_composite(float x, unsigned col) {
    const unsigned a = __float_as_uint(x) & 0x7fffffffu;
    const unsigned ukey = (a > 0x7f800000u) ? 0u : a + 1u;
    return ((unsigned long long)ukey << 16) | (unsigned long long)(0xFFFFu - col);
}

// Warp 0 only.  Finds the highest bin b with count(bins >= b) >= need and the number still
// needed inside b; publishes them in s.sel_bin / s.sel_need (sel_ok = 0 if the total is short).
__device__ __forceinline__ void hist_select_warp(TopkScratch &s, unsigned need) {
    const int lane = threadIdx.x & 31;
    unsigned c[8], sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { c[i] = s.hist[lane * 8 + i]; sum += c[i]; }
    unsigned suffix = sum;                                 // inclusive sum over lanes >= lane
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned t = __shfl_down_sync(kFullMask, suffix, d);
        if (lane + d < 32) suffix += t;
    }
    const unsigned ballot = __ballot_sync(kFullMask, suffix >= need);
    if (ballot == 0) {
        if (lane == 0) s.sel_ok = 0;
        return;
    }
    const int top = 31 - __clz((int)ballot);
    if (lane == top) {
        unsigned acc = suffix - sum;                       // count in higher lanes
        unsigned bin = 0, rem = need;
#pragma unroll
        for (int i = 7; i >= 0; --i) {
            if (acc + c[i] >= need) { bin = lane * 8 + i; rem = need - acc; break; }
            acc += c[i];
        }
        s.sel_bin = bin;
        s.sel_need = rem;
        s.sel_ok = 1;
    }
}

// Bitonic sort, descending, of SLOTS*32 composites held as a[slot] with element index
// slot*32 + lane.  One warp.
template <int SLOTS>
__device__ __forceinline__ void warp_bitonic_desc(unsigned long long (&a)[SLOTS]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int size = 2; size <= SLOTS * 32; size <<= 1) {
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (stride >= 32) {
                const int ss = stride >> 5;
#pragma unroll
                for (int slot = 0; slot < SLOTS; ++slot) {
                    if ((slot & ss) == 0) {
                        const int i = slot * 32 + lane;
                        const bool desc = (i & size) == 0;
                        const unsigned long long x = a[slot], y = a[slot | ss];
                        const bool swap = desc ? (x < y) : (x > y);
                        a[slot] = swap ? y : x;
                        a[slot | ss] = swap ? x : y;
                    }
                }
            } else {
#pragma unroll
                for (int slot = 0; slot < SLOTS; ++slot) {
                    const int i = slot * 32 + lane;
                    const bool desc = (i & size) == 0;
                    const bool lower = (lane & stride) == 0;
                    const unsigned long long x = a[slot];
                    const unsigned long long y = __shfl_xor_sync(kFullMask, x, stride);
                    const bool take_max = (desc == lower);
                    a[slot] = take_max ? (x > y ? x : y) : (x < y ? x : y);
                }
            }
        }
    }
}

// Warp 0 only: sort s.cand[0..count) and emit the first k as (column, value).  With
// `zero_selected` the chosen entries of the shared-memory row become +0.0f afterwards.
template <int SLOTS>
__device__ __forceinline__ void sort_emit_warp(TopkScratch &s, float *row, unsigned count, unsigned k,
                                               uint16_t *out_idx, float *out_val, bool zero_selected) {
    const int lane = threadIdx.x & 31;
    unsigned long long a[SLOTS];
#pragma unroll
    for (int slot = 0; slot < SLOTS; ++slot) {
        const unsigned i = slot * 32 + lane;
        a[slot] = i < count ? s.cand[i] : 0ull;
    }
    warp_bitonic_desc<SLOTS>(a);
#pragma unroll
    for (int slot = 0; slot < SLOTS; ++slot) {
        const unsigned r = slot * 32 + lane;
        if (r < k) {
            const unsigned col = 0xFFFFu - (unsigned)(a[slot] & 0xFFFFull);
            out_idx[r] = (uint16_t)col;
            out_val[r] = row[col];
            if (zero_selected) {
                row[col] = 0.0f;
                atomicOr(&s.dirty[col >> 7], 1u << ((col >> 2) & 31u));
            }
        }
    }
}

__device__ __forceinline__ void sort_emit_dispatch(TopkScratch &s, float *row, unsigned count, unsigned k,
                                                   uint16_t *out_idx, float *out_val, bool zero_selected) {
    if (count <= 64) sort_emit_warp<2>(s, row, count, k, out_idx, out_val, zero_selected);
    else if (count <= 128) sort_emit_warp<4>(s, row, count, k, out_idx, out_val, zero_selected);
    else sort_emit_warp<8>(s, row, count, k, out_idx, out_val, zero_selected);
}

// Exact path.  `row` may be any generic pointer (shared or global).  All threads of the CTA
// call it; k <= kCandCap; cols <= 65535.  Ends with a __syncthreads().
template <int NT>
__device__ __noinline__ void topk_exact(float *row, unsigned cols, unsigned k, TopkScratch &s, uint16_t *out_idx, float *out_val,
                           bool zero_selected) {
    const int tid = threadIdx.x;
    unsigned long long prefix = 0;
    unsigned need = k;
    for (int pass = 0; pass < 6; ++pass) {
        const int shift = 40 - 8 * pass;
        for (int i = tid; i < 256; i += NT) s.hist[i] = 0;
        __syncthreads();
        for (unsigned c = tid; c < cols; c += NT) {
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
    if (tid == 0) s.count = 0;
    __syncthreads();
    for (unsigned c = tid; c < cols; c += NT) {
        const unsigned long long comp = topk_composite(row[c], c);
        if (comp >= prefix) {
            const unsigned pos = atomicAdd(&s.count, 1u);
            if (pos < kCandCap) s.cand[pos] = comp;
        }
    }
    __syncthreads();
    if (tid < 32) sort_emit_dispatch(s, row, min(s.count, (unsigned)kCandCap), k, out_idx, out_val, zero_selected);
    __syncthreads();
}

// Per-thread maximum of the |x| bit patterns of a shared-memory row, float4 i = f * NT + tid.
// m4[f] keeps the maximum of each float4 (0 past the end of the row).  A result >= 0x7f800000
// means the thread saw an Inf or NaN.
constexpr int kMaxRowIters = 8;
template <int NT, int IT>
__device__ __forceinline__ unsigned row_thread_max(const float *row, unsigned cols, unsigned (&m4)[IT]) {
    const unsigned f4 = cols >> 2;
    const uint4 *row4 = reinterpret_cast<const uint4 *>(row);
    unsigned g = 0;
#pragma unroll
    for (int f = 0; f < IT; ++f) {
        const unsigned i = f * NT + threadIdx.x;
        unsigned m = 0;
        if (i < f4) {
            const uint4 a = row4[i];
            m = max(max(a.x & 0x7fffffffu, a.y & 0x7fffffffu), max(a.z & 0x7fffffffu, a.w & 0x7fffffffu));
        }
        m4[f] = m;
        g = max(g, m);
    }
    return g;
}

// Bound from a two-round histogram over the per-thread maxima: at least k threads, hence at least
// k elements, reach the returned value.  All threads call it; contains __syncthreads().
template <int NT>
__device__ __forceinline__ float topk_bound_hist(unsigned gb, unsigned k, TopkScratch &s) {
    const int tid = threadIdx.x;
    for (int i = tid; i < 256; i += NT) s.hist[i] = 0;
    __syncthreads();
    atomicAdd(&s.hist[gb >> 23], 1u);                      // round 1: exponent byte
    __syncthreads();
    if (tid < 32) hist_select_warp(s, k);
    __syncthreads();
    const unsigned b1 = s.sel_bin, need1 = s.sel_need;
    for (int i = tid; i < 256; i += NT) s.hist[i] = 0;     // warp 0 is done reading the histogram
    __syncthreads();
    if ((gb >> 23) == b1) atomicAdd(&s.hist[(gb >> 15) & 0xFFu], 1u);   // round 2: next 8 bits
    __syncthreads();
    if (tid < 32) hist_select_warp(s, need1);
    __syncthreads();
    return __uint_as_float((b1 << 23) | (s.sel_bin << 15));
}

// Append every element with |x| >= bound to s.cand (count in s.count, which the caller zeroed
// behind a barrier).  Only float4s whose maximum m4[f] reaches the bound are read again.
template <int NT, int IT>
__device__ __forceinline__ void topk_collect(const float *row, unsigned cols, const unsigned (&m4)[IT],
                                             float bound, TopkScratch &s) {
    const unsigned f4 = cols >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    const unsigned bb = __float_as_uint(bound);
#pragma unroll
    for (int f = 0; f < IT; ++f) {
        const unsigned i = f * NT + threadIdx.x;
        if (m4[f] >= bb && i < f4) {
            const float4 a = row4[i];
            const float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (fabsf(v[q]) >= bound) {
                    const unsigned pos = atomicAdd(&s.count, 1u);
                    if (pos < kCandCap) s.cand[pos] = topk_composite(v[q], i * 4 + q);
                }
            }
        }
    }
}

// Rank the `count` candidates by counting (composites are distinct), emit those of rank < k and,
// with zero_selected, zero them in the row.  P = 64, 128 or 256 >= count; NT / P threads share the
// comparisons of one candidate.  Leaves |x| of the k-th entry in s.kth_bits.  All threads call it;
// contains __syncthreads() and ends with one.
template <int NT, int P>
__device__ __forceinline__ void topk_rank_emit(float *row, unsigned count, unsigned k, TopkScratch &s, uint16_t *out_idx,
                                               float *out_val, bool zero_selected) {
    constexpr int PARTS = NT / P;
    const int tid = threadIdx.x;
    const unsigned j = tid % P, part = tid / P;
    if (PARTS > 1 && tid < P) s.hist[tid] = 0;             // hist doubles as the rank accumulator
    if (PARTS > 1) __syncthreads();
    unsigned rank = 0;
    const unsigned long long mine = j < count ? s.cand[j] : 0ull;
    if (j < count && part < (unsigned)PARTS) {
        for (unsigned i = part; i < count; i += PARTS) rank += s.cand[i] > mine ? 1u : 0u;
        if (PARTS > 1) atomicAdd(&s.hist[j], rank);
    }
    if (PARTS > 1) {
        __syncthreads();
        rank = s.hist[j];
    }
    if (tid < P && j < count && rank < k) {
        const unsigned col = 0xFFFFu - (unsigned)(mine & 0xFFFFull);
        const float v = row[col];
        out_idx[rank] = (uint16_t)col;
        out_val[rank] = v;
        if (rank == k - 1) s.kth_bits = __float_as_uint(v) & 0x7fffffffu;
        if (zero_selected) {
            row[col] = 0.0f;
            atomicOr(&s.dirty[col >> 7], 1u << ((col >> 2) & 31u));
        }
    }
    __syncthreads();
}

// Fast path with fallback.  `row` is a shared-memory row of `cols` floats, cols % 4 == 0,
// cols <= 4 * NT * IT, 16-byte aligned; k <= min(kCandCap, NT).  `gb` / `m4` come from
// row_thread_max(); `special` (uniform over the CTA) says that some thread saw Inf or NaN, which
// sends the row down the exact path.  `hint` (uniform) is a guess of the bound, normally a little
// below the k-th largest |x| of the row this CTA handled before (0 = no guess): any bound that
// at least k and at most kCandCap elements reach gives the exact answer, so a wrong guess only
// costs the histogram search.  Returns the guess for the next row.  All threads call it; the
// caller must have executed a __syncthreads() since the row was last written; ends with one.
template <int NT, int IT>
__device__ float topk_row(float *row, unsigned cols, unsigned k, TopkScratch &s, uint16_t *out_idx, float *out_val,
                          bool zero_selected, unsigned gb, const unsigned (&m4)[IT], bool special, float hint) {
    const int tid = threadIdx.x;
    for (int i = tid; i < 256; i += NT) s.dirty[i] = 0;
    if (tid == 0) s.count = 0;
    __syncthreads();
    if (special) {
        topk_exact<NT>(row, cols, k, s, out_idx, out_val, zero_selected);
        return 0.0f;
    }
    BSQ_TT(0);
    unsigned count = 0;
    bool have = false;
    if (hint > 0.0f) {
        topk_collect<NT, IT>(row, cols, m4, hint, s);
        __syncthreads();
        count = s.count;
        have = count >= k && count <= (unsigned)kCandCap;
        if (!have) {
            __syncthreads();
            if (tid == 0) s.count = 0;
        }
    }
    BSQ_TT(1);
    if (!have) {
        const float bound = topk_bound_hist<NT>(gb, k, s);          // its barriers also publish count = 0
        topk_collect<NT, IT>(row, cols, m4, bound, s);
        __syncthreads();
        count = s.count;
        if (count > (unsigned)kCandCap || count < k) {                // ties / zeros: exact path
            topk_exact<NT>(row, cols, k, s, out_idx, out_val, zero_selected);
            return 0.0f;
        }
    }
    BSQ_TT(2);
    if (count <= 64) topk_rank_emit<NT, 64>(row, count, k, s, out_idx, out_val, zero_selected);
    else if (count <= 128) topk_rank_emit<NT, 128>(row, count, k, s, out_idx, out_val, zero_selected);
    else topk_rank_emit<NT, 256>(row, count, k, s, out_idx, out_val, zero_selected);
    BSQ_TT(3);
    // next guess: 7/8 of this row's k-th largest magnitude
    return __uint_as_float(s.kth_bits) * 0.875f;
}

}  // namespace bsq
