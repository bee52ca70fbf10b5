// Row-group routines: one group of G warps (G = 1, 2, 4 or 8; 32*G lanes) owns one matrix row that
// sits in shared memory and does everything for it -- top-k selection, zeroing, block maxima, NF4
// encoding -- without CTA-wide barriers.  A CTA holds several independent groups; groups only meet
// at a named barrier of their own.
//
// Why groups instead of a CTA per row: the selection and the encoder are instruction-issue bound,
// not bandwidth bound, and with a whole CTA on a row most instructions were per-thread fixed costs
// repeated by 8 warps, CTA barriers and single-warp sections.  Here a lane walks 32 float4 of the row
// with a handful of instructions each (3-input absolute maxima, one reduce instruction per 64-element
// block), and the k survivors are ranked by counting inside the group.
//
// Ordering contract of the selection (reference modules/topk_cuda/src/topk_cuda_utils.cuh:51-93,
// 254-295): the k entries of largest |x| (NaN below every number), by (|x| descending, column
// ascending); implemented on the 48-bit composite of bsq_topk.cuh.
#pragma once

#include "bsq_device.cuh"
#include "bsq_topk.cuh"

namespace bsq {

constexpr unsigned kFlagSpecial = 1u;      // GroupCtl::flags: the row holds Inf or NaN
constexpr unsigned kFlagSlow = 2u;         //                  some block of the row takes the literal scan
constexpr unsigned kFlagTie = 4u;          //                  two candidates share |x|: rank on the full composite

// control words of one group
struct GroupCtl {
    unsigned long long bar;        // mbarrier of the row copy
    unsigned count;                // candidates collected
    unsigned kth_bits;             // |x| bits of the k-th entry of the finished row
    unsigned next_row;             // row handed out by the global counter
    unsigned reduce;               // scratch for group-wide max / or
    unsigned nhits;                // float4 of the row whose maximum reached the bound (indices in hist[])
    unsigned flags;                // row state of the streaming routines (bsq_rowstream.cuh)
    unsigned wait_failed;          // a lane's bounded wait for the row copy ran out: the whole group stops
    unsigned seen[8];              // one bit per 32-bit rank already taken (tie detection, bsq_rowstream.cuh)
    unsigned hist[256];            // radix-select histogram of the exact path
    __align__(16) unsigned key[kCandCap];   // |x| bits of the candidates, zero beyond their number
    unsigned long long cand[kCandCap];
    float val[kCandCap];           // the candidates' values (group_topk_row: the row itself may be gone when they are emitted)
};

template <int G>
struct RowGroup {
    static constexpr int L = 32 * G;
    int lane;          // 0 .. L-1 within the group
    int gid;           // group index within the CTA

    __device__ __forceinline__ RowGroup() : lane(threadIdx.x % L), gid(threadIdx.x / L) {}

    __device__ __forceinline__ void sync() const {
        if (G == 1) __syncwarp();
        else asm volatile("bar.sync %0, %1;" ::"r"(gid + 1), "r"(L) : "memory");
    }
    // group-wide OR of a predicate (contains group syncs)
    __device__ __forceinline__ bool any(bool p, GroupCtl &c) const {
        if (G == 1) return __any_sync(kFullMask, p);
        if (lane == 0) c.reduce = 0;
        sync();
        if (__any_sync(kFullMask, p) && (lane & 31) == 0) atomicOr(&c.reduce, 1u);
        sync();
        const bool r = c.reduce != 0;
        sync();
        return r;
    }
    // group-wide maximum of unsigned values (contains group syncs)
    __device__ __forceinline__ unsigned max_bits(unsigned v, GroupCtl &c) const {
        v = __reduce_max_sync(kFullMask, v);
        if (G == 1) return v;
        if (lane == 0) c.reduce = 0u;
        sync();
        if ((lane & 31) == 0) atomicMax(&c.reduce, v);
        sync();
        const unsigned r = c.reduce;
        sync();
        return r;
    }
};

// max(|a|, |b|, |c|), NaN if any input is NaN
__device__ __forceinline__ float absmax3_nan(float a, float b, float c) {
    float d;
    asm("max.NaN.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float absmax4_nan(const float4 &a) {
    return absmax3_nan(absmax3_nan(a.x, a.y, a.z), a.w, 0.0f);
}

// A sweep over the row only notes WHICH float4 reach the bound (a few instructions on the rare
// hit); this turns the noted float4 into candidates, spread evenly over the lanes of the group.
// c.hist[] holds the float4 indices, c.nhits their number (more than 256: the caller falls back).
constexpr unsigned kHitCap = 256;
__device__ __forceinline__ void note_hit(unsigned i, GroupCtl &c) {
    const unsigned pos = atomicAdd(&c.nhits, 1u);
    if (pos < kHitCap) c.hist[pos] = i;
}
template <int G>
__device__ __forceinline__ void expand_hits(const RowGroup<G> &g, GroupCtl &c, const float *row, float bound) {
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    const unsigned n = min(c.nhits, kHitCap);
    for (unsigned e = g.lane; e < n; e += RowGroup<G>::L) {
        const unsigned i = c.hist[e];
        const float4 a = row4[i];
        const float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if (fabsf(v[q]) >= bound) {
                const unsigned pos = atomicAdd(&c.count, 1u);
                if (pos < (unsigned)kCandCap) {
                    c.key[pos] = __float_as_uint(v[q]) & 0x7fffffffu;
                    c.val[pos] = v[q];
                    c.cand[pos] = topk_composite(v[q], i * 4 + q);
                }
            }
        }
    }
}

// Rank the candidates by counting (composites are distinct), emit rank < k, zero them in the row when
// asked, publish |x| of the k-th.  Every lane of the group calls it; ends with a group sync.
template <int G>
__device__ __forceinline__ void group_rank_emit(const RowGroup<G> &g, GroupCtl &c, float *row, unsigned count, unsigned k,
                                                uint16_t *out_idx, float *out_val, bool zero_selected) {
    constexpr int L = RowGroup<G>::L;
    for (unsigned j0 = g.lane; j0 < count; j0 += 2 * L) {          // two candidates per lane and sweep
        const unsigned j1 = j0 + L;
        const unsigned long long m0 = c.cand[j0];
        const unsigned long long m1 = j1 < count ? c.cand[j1] : ~0ull;
        unsigned r0 = 0, r1 = 0;
        for (unsigned i = 0; i < count; ++i) {
            const unsigned long long o = c.cand[i];
            r0 += o > m0 ? 1u : 0u;
            r1 += o > m1 ? 1u : 0u;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const unsigned long long mine = h ? m1 : m0;
            const unsigned rank = h ? r1 : r0;
            if ((h == 0 || j1 < count) && rank < k) {
                const unsigned col = 0xFFFFu - (unsigned)(mine & 0xFFFFull);
                const float v = row[col];
                out_idx[rank] = (uint16_t)col;
                out_val[rank] = v;
                if (rank == k - 1) c.kth_bits = __float_as_uint(v) & 0x7fffffffu;
                if (zero_selected) row[col] = 0.0f;
            }
        }
    }
    g.sync();
}

// The same for candidates whose |x| bits are also in c.key[] (finite values, zeros beyond `count` up to a multiple of
// four): ranks come from 32-bit compares, four keys per load, a quarter of the instructions of the 64-bit count above
// (which bounded the error-correction pass: 143 of 14336 per row means ~200 candidates, 200 x 200 compares).  Two
// candidates of equal |x| would get the same rank, which the `seen` bits catch: then everybody ranks on the full
// composite (column ascending breaks the tie).  c.hist[] keeps the ranks; c.seen[] and kFlagTie in c.flags must be
// clear on entry.  Ends with a group sync.
template <int G>
__device__ __forceinline__ void group_rank_emit_keys(const RowGroup<G> &g, GroupCtl &c, float *row, unsigned count, unsigned k,
                                                     uint16_t *out_idx, float *out_val, bool zero_selected) {
    constexpr unsigned L = RowGroup<G>::L;
    const uint4 *key4 = reinterpret_cast<const uint4 *>(c.key);
    const unsigned n4 = (count + 3) >> 2;
    for (unsigned j = g.lane; j < count; j += L) {
        const unsigned m = c.key[j];
        unsigned r = 0;
#pragma unroll 4
        for (unsigned i = 0; i < n4; ++i) {
            const uint4 o = key4[i];
            r += (o.x > m ? 1u : 0u) + (o.y > m ? 1u : 0u) + (o.z > m ? 1u : 0u) + (o.w > m ? 1u : 0u);
        }
        const unsigned bit = 1u << (r & 31);
        if (atomicOr(&c.seen[r >> 5], bit) & bit) atomicOr(&c.flags, kFlagTie);
        c.hist[j] = r;
    }
    g.sync();
    const bool tie = (c.flags & kFlagTie) != 0;
    for (unsigned j = g.lane; j < count; j += L) {
        const unsigned long long mine = c.cand[j];
        unsigned rank = c.hist[j];
        if (tie) {
            rank = 0;
            for (unsigned i = 0; i < count; ++i) rank += c.cand[i] > mine ? 1u : 0u;
        }
        if (rank < k) {
            const unsigned col = 0xFFFFu - (unsigned)(mine & 0xFFFFull);
            const float v = c.val[j];                           // (not row[col]: without zero_selected the row may be gone)
            out_idx[rank] = (uint16_t)col;
            out_val[rank] = v;
            if (rank == k - 1) c.kth_bits = __float_as_uint(v) & 0x7fffffffu;
            if (zero_selected) row[col] = 0.0f;
        }
    }
    g.sync();
}

// Exact selection for rows the quick bound cannot handle (Inf / NaN, heavy ties, rows of zeros):
// 6 passes of 8-bit radix select over the composite, then the same ranking.  `row` may be any
// generic pointer.  Every lane of the group calls it; ends with a group sync.
template <int G>
__device__ __noinline__ void group_topk_exact(const RowGroup<G> &g, GroupCtl &c, float *row, unsigned cols, unsigned k,
                                              uint16_t *out_idx, float *out_val, bool zero_selected) {
    constexpr int L = RowGroup<G>::L;
    unsigned long long prefix = 0;
    unsigned need = k;
    for (int pass = 0; pass < 6; ++pass) {
        const int shift = 40 - 8 * pass;
        for (int i = g.lane; i < 256; i += L) c.hist[i] = 0;
        g.sync();
        for (unsigned col = g.lane; col < cols; col += L) {
            const unsigned long long comp = topk_composite(row[col], col);
            if (pass == 0 || (comp >> (shift + 8)) == (prefix >> (shift + 8)))
                atomicAdd(&c.hist[(unsigned)(comp >> shift) & 0xFFu], 1u);
        }
        g.sync();
        // every lane walks the 256 bins from the top (uniform result, no further exchange needed)
        unsigned acc = 0, bin = 0, rem = need;
        for (int b = 255; b >= 0; --b) {
            const unsigned h = c.hist[b];
            if (acc + h >= need) { bin = (unsigned)b; rem = need - acc; break; }
            acc += h;
        }
        prefix |= (unsigned long long)bin << shift;
        need = rem;
        g.sync();
    }
    if (g.lane == 0) c.count = 0;
    g.sync();
    for (unsigned col = g.lane; col < cols; col += L) {
        const unsigned long long comp = topk_composite(row[col], col);
        if (comp >= prefix) {
            const unsigned pos = atomicAdd(&c.count, 1u);
            if (pos < (unsigned)kCandCap) c.cand[pos] = comp;
        }
    }
    g.sync();
    group_rank_emit<G>(g, c, row, min(c.count, (unsigned)kCandCap), k, out_idx, out_val, zero_selected);
}

// Selection on a shared-memory row (cols % 4 == 0, 16-byte aligned, k <= kCandCap).
//   hint : a guess of a bound slightly below the k-th largest |x| (0 = none), normally from the row
//          the group did before.  Any bound that between k and kCandCap elements reach gives the exact
//          answer, so a bad guess only costs a second sweep.
// Without a usable hint the bound is the k-th largest among the lanes' largest and second-largest
// float4 maxima (2 * L values, each a different float4, so at least k elements reach it).
// Returns the hint for the next row; *special_out says the row holds Inf or NaN.
// Every lane of the group calls it; the caller has synchronised the group since the row was
// written; ends with a group sync.
// row_free(): called (by every lane, after a group sync behind the last read of the row) as soon as nothing will read
// the row any more, if that is before the ranking -- only without zero_selected, and not on the exact path, which
// keeps reading the row to the end; the caller may refill the buffer from then on.
template <int G, class RowFree>
__device__ __forceinline__ float group_topk_row(const RowGroup<G> &g, GroupCtl &c, float *row, unsigned cols, unsigned k,
                                                uint16_t *out_idx, float *out_val, bool zero_selected, float hint,
                                                bool *special_out, RowFree row_free) {
    constexpr int L = RowGroup<G>::L;
    const unsigned f4 = cols >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    if (g.lane == 0) { c.count = 0; c.nhits = 0; c.flags = 0; }
    if (g.lane < 8) c.seen[g.lane] = 0u;
    for (unsigned i = g.lane; i < (unsigned)kCandCap / 4; i += L) reinterpret_cast<uint4 *>(c.key)[i] = make_uint4(0u, 0u, 0u, 0u);
    g.sync();
    float acc = 0.0f, first = 0.0f, second = 0.0f;
    const bool hinted = hint > 0.0f;
    if (hinted) {
#pragma unroll 4
        for (unsigned i = g.lane; i < f4; i += L) {
            const float m = absmax4_nan(row4[i]);
            acc = absmax3_nan(acc, m, 0.0f);
            if (m >= hint) note_hit(i, c);
        }
    } else {
#pragma unroll 4
        for (unsigned i = g.lane; i < f4; i += L) {
            const float m = absmax4_nan(row4[i]);
            acc = absmax3_nan(acc, m, 0.0f);
            second = fmaxf(second, fminf(first, m));
            first = fmaxf(first, m);
        }
    }
    const bool special = g.any(!(acc < __int_as_float(0x7f800000)), c);      // Inf or NaN somewhere
    *special_out = special;
    if (special) {
        group_topk_exact<G>(g, c, row, cols, k, out_idx, out_val, zero_selected);
        return 0.0f;
    }
    g.sync();
    unsigned count = 0;
    if (hinted && c.nhits <= kHitCap) {
        expand_hits<G>(g, c, row, hint);
        g.sync();
        count = c.count;
    }
    float guess = hint;
    for (int retry = 0; retry < 2 && hinted && (c.nhits > kHitCap || count < k || count > (unsigned)kCandCap); ++retry) {
        // The guess was off -- by a little, most of the time (rows of one matrix differ in scale by some per cent, and
        // for a large k the window between k and kCandCap candidates is narrow): another sweep with the guess moved
        // costs a tenth of working the bound out from the lanes' largest values below.  How far to move it: the number
        // that got through (the float4 hits when they overflowed: a lower bound) against a target inside the window
        // (its middle, or 1.6 k where that is less: ranking costs count^2),
        // with the slope of a Gaussian tail near its 1 % quantile, d ln(count) / d ln(bound) = -z^2 ~ -6.6.
        const float passed = (float)max(c.nhits > kHitCap ? c.nhits : count, 1u);
        const float target = fminf(0.5f * (float)(k + (unsigned)kCandCap), 1.6f * (float)k);
        const float factor = exp2f(0.15f * log2f(passed / target));
        guess *= fminf(fmaxf(factor, 0.7f), 1.4f);
        g.sync();                                           // everybody has read nhits / count
        if (g.lane == 0) { c.count = 0; c.nhits = 0; }
        for (unsigned i = g.lane; i < (unsigned)kCandCap / 4; i += L) reinterpret_cast<uint4 *>(c.key)[i] = make_uint4(0u, 0u, 0u, 0u);
        g.sync();
#pragma unroll 4
        for (unsigned i = g.lane; i < f4; i += L)
            if (absmax4_nan(row4[i]) >= guess) note_hit(i, c);
        g.sync();
        count = 0;
        if (c.nhits <= kHitCap) {
            expand_hits<G>(g, c, row, guess);
            g.sync();
            count = c.count;
        }
    }
    if (!hinted || count < k || count > (unsigned)kCandCap) {
        if (k > 2u * L) {                                   // the two-per-lane bound cannot promise k entries
            group_topk_exact<G>(g, c, row, cols, k, out_idx, out_val, zero_selected);
            return 0.0f;
        }
        if (hinted) {                                       // the guess was off: get the lanes' top two
            for (unsigned i = g.lane; i < f4; i += L) {
                const float m = absmax4_nan(row4[i]);
                second = fmaxf(second, fminf(first, m));
                first = fmaxf(first, m);
            }
        }
        // bound = k-th largest of the 2 * L (first, second) values: each stands for a different float4,
        // so at least k elements reach it, and seldom many more
        unsigned *tops = reinterpret_cast<unsigned *>(c.cand);
        const unsigned fb = __float_as_uint(first), sb = __float_as_uint(second);
        tops[g.lane] = fb;
        tops[L + g.lane] = sb;
        g.sync();
        unsigned ge_f = 0, ge_s = 0;
        const uint4 *tops4 = reinterpret_cast<const uint4 *>(tops);
#pragma unroll 4
        for (int i = 0; i < 2 * L / 4; ++i) {
            const uint4 o = tops4[i];
            ge_f += (o.x >= fb ? 1u : 0u) + (o.y >= fb ? 1u : 0u) + (o.z >= fb ? 1u : 0u) + (o.w >= fb ? 1u : 0u);
            ge_s += (o.x >= sb ? 1u : 0u) + (o.y >= sb ? 1u : 0u) + (o.z >= sb ? 1u : 0u) + (o.w >= sb ? 1u : 0u);
        }
        const unsigned mine = ge_f >= k ? fb : (ge_s >= k ? sb : 0u);
        const float bound = __uint_as_float(g.max_bits(mine, c));
        if (g.lane == 0) { c.count = 0; c.nhits = 0; }
        // (keys of the first attempt: tops[] above overlaid only c.cand[]; stale keys beyond the new count must go)
        for (unsigned i = g.lane; i < (unsigned)kCandCap / 4; i += L) reinterpret_cast<uint4 *>(c.key)[i] = make_uint4(0u, 0u, 0u, 0u);
        g.sync();
        if (bound > 0.0f) {
            for (unsigned i = g.lane; i < f4; i += L)
                if (absmax4_nan(row4[i]) >= bound) note_hit(i, c);
            g.sync();
            if (c.nhits <= kHitCap) expand_hits<G>(g, c, row, bound);
        }
        g.sync();
        count = c.count;
        if (bound <= 0.0f || c.nhits > kHitCap || count < k || count > (unsigned)kCandCap) {
            group_topk_exact<G>(g, c, row, cols, k, out_idx, out_val, zero_selected);
            return 0.0f;
        }
    }
    if (!zero_selected) row_free();
    group_rank_emit_keys<G>(g, c, row, count, k, out_idx, out_val, zero_selected);
    // The next row's guess: a little below this row's k-th largest, so that between k and kCandCap of its elements
    // reach it.  The window is narrow for a large k (143 of 256: a Gaussian tail has 225 elements above 0.9375 of the
    // k-th largest, too close to the cap and beyond the 256 float4 the first sweep can note), so the margin shrinks
    // with k; a guess that misses only costs the row a second and third sweep, never the result.
    return __uint_as_float(c.kth_bits) * (k <= 96u ? 0.9375f : 0.9609375f);
}

// Block maxima of the (zeroed) row: blk_out[b] = absmax of block b, 1.0 for a block of zeros
// (quantization_cuda.cu:217-219).  In `special` rows non-finite values count as zero and a block that
// holds one gets its maximum NEGATED, which tells the encoder to take the literal scan there.
// Returns the lane's running maximum of |blk_out|.  cols % 64 == 0.
template <int G>
__device__ __forceinline__ float group_block_absmax(const RowGroup<G> &g, const float *row, unsigned cols, bool special,
                                                    float *blk_out) {
    constexpr int L = RowGroup<G>::L;
    const unsigned f4 = cols >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    const unsigned half_mask = (g.lane & 16) ? 0xffff0000u : 0x0000ffffu;
    float run = 0.0f;
    const unsigned iters = (f4 + L - 1) / L;                // every lane runs every iteration (warp reduces)
#pragma unroll 4
    for (unsigned it = 0; it < iters; ++it) {
        const unsigned i = it * L + g.lane;
        const bool valid = i < f4;
        unsigned m = 0;
        bool nonfinite = false;
        if (valid) {
            const float4 a = row4[i];
            if (!special) {
                m = __float_as_uint(absmax4_nan(a));
            } else {
                const unsigned e[4] = {__float_as_uint(a.x) & 0x7fffffffu, __float_as_uint(a.y) & 0x7fffffffu,
                                       __float_as_uint(a.z) & 0x7fffffffu, __float_as_uint(a.w) & 0x7fffffffu};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    if (e[q] < 0x7f800000u) m = max(m, e[q]);
                    else nonfinite = true;
                }
            }
        }
        m = __reduce_max_sync(half_mask, m);                // the 16 lanes of one 64-element block
        const unsigned nf = special ? __ballot_sync(kFullMask, nonfinite) : 0u;
        if (valid && (g.lane & 15) == 0) {
            const float am = __uint_as_float(m);
            const float v = am > 0.0f ? am : 1.0f;
            const bool marked = ((nf >> (g.lane & 16)) & 0xFFFFu) != 0;
            blk_out[i >> 4] = marked ? -v : v;
            run = fmaxf(run, v);
        }
    }
    return run;
}

// Per block: +-1/scale for the encoder in blk[] (negative = take the literal scan: non-finite
// elements, or a scaled value that can leave the exact range of the table encoder).
//   DQ: blk_in holds the (possibly negated) maxima of pass 1; writes the E4M3 codes.
//  !DQ: blk holds the maxima on entry; writes the FP32 scales.
template <int G, bool DQ>
__device__ __forceinline__ bool group_block_scales(const RowGroup<G> &g, unsigned cols, float dq, const float *blk_in,
                                                   float *blk, float *scales_out, uint8_t *scale_codes_out) {
    constexpr int L = RowGroup<G>::L;
    const unsigned nblk = cols >> 6;
    bool any_slow = false;
    for (unsigned b = g.lane; b < nblk; b += L) {
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
        any_slow |= slow;
        blk[b] = slow ? -inv : inv;
    }
    return any_slow;            // this lane's blocks only; the caller ORs it over the group
}

// Nibbles of the row into codes_smem (cols / 2 bytes); blk[] holds +-1/scale per block.  The main
// loop is branch-free (whole sweeps of the group over the row); blocks marked for the literal scan
// are redone afterwards, which `any_slow` (uniform over the group) says is needed at all.
template <int G>
__device__ __forceinline__ void group_encode(const RowGroup<G> &g, const float *row, unsigned cols, const Nf4Lut &lut,
                                             const float *blk, uint16_t *codes_smem, bool any_slow) {
    constexpr int L = RowGroup<G>::L;
    const unsigned f4 = cols >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    const unsigned full = f4 / L;
#pragma unroll 4
    for (unsigned it = 0; it < full; ++it) {
        const unsigned i = it * L + g.lane;
        const float4 a = row4[i];
        const float inv = fabsf(blk[i >> 4]);
        const unsigned c0 = lut.encode(__fmul_rn(a.x, inv));
        const unsigned c1 = lut.encode(__fmul_rn(a.y, inv));
        const unsigned c2 = lut.encode(__fmul_rn(a.z, inv));
        const unsigned c3 = lut.encode(__fmul_rn(a.w, inv));
        codes_smem[i] = (uint16_t)((c0 << 4) | c1 | (c2 << 12) | (c3 << 8));
    }
    if (full * L < f4) {                                    // ragged last sweep: every lane still shuffles
        const unsigned i = full * L + g.lane;
        const bool valid = i < f4;
        const float4 a = valid ? row4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float inv = valid ? fabsf(blk[i >> 4]) : 1.0f;
        const unsigned c0 = lut.encode(__fmul_rn(a.x, inv));
        const unsigned c1 = lut.encode(__fmul_rn(a.y, inv));
        const unsigned c2 = lut.encode(__fmul_rn(a.z, inv));
        const unsigned c3 = lut.encode(__fmul_rn(a.w, inv));
        if (valid) codes_smem[i] = (uint16_t)((c0 << 4) | c1 | (c2 << 12) | (c3 << 8));
    }
    if (any_slow) {                                         // rare: literal scan on sanitised values
        for (unsigned i = g.lane; i < f4; i += L) {
            const float invs = blk[i >> 4];
            if (invs < 0.0f) {
                const float4 a = row4[i];
                const float inv = -invs;
                const unsigned c0 = nf4_code_scan(__fmul_rn(sanitize(a.x), inv));
                const unsigned c1 = nf4_code_scan(__fmul_rn(sanitize(a.y), inv));
                const unsigned c2 = nf4_code_scan(__fmul_rn(sanitize(a.z), inv));
                const unsigned c3 = nf4_code_scan(__fmul_rn(sanitize(a.w), inv));
                codes_smem[i] = (uint16_t)((c0 << 4) | c1 | (c2 << 12) | (c3 << 8));
            }
        }
    }
}

}  // namespace bsq
