// Pieces shared by the top-k kernels.
//
// Contract (reference modules/topk_cuda/src/topk_cuda_utils.cuh:51-93,254-295): per row the k entries
// with the largest key |x| (NaN ranks below every number, +0 == -0), emitted in the order (key
// descending, column ascending), values with their original sign and bits.
//
// Everything works on a 48-bit "composite" per element,
//     composite = ukey << 16 | (0xFFFF - column),  ukey = NaN ? 0 : bits(|x|) + 1,
// whose descending order is exactly the reference order and which is unique per column, so "the k
// largest composites, sorted" is the whole specification.
#pragma once

#include "bsq_device.cuh"

namespace bsq {

constexpr int kCandCap = 256;              // candidate slots; also the largest k these routines take

struct TopkScratch {                       // per-CTA shared-memory scratch of the generic kernel
    unsigned hist[256];
    unsigned count;                        // selected entries appended
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

}  // namespace bsq
