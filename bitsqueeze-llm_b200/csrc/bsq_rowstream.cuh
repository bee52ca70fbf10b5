// Streaming row routines of the fused front end: a group of G warps (bsq_rowgroup.cuh) walks one matrix
// row straight from global memory, 8 float4 per lane in flight, and keeps nothing of it in shared
// memory.  One sweep does the outlier selection AND the NF4 block maxima of the row with the outliers
// taken out:
//
//   * with a bound b slightly below the k-th largest |x| of the row (from the row before, or from a
//     sweep over the lanes' largest values), every float4 whose maximum stays below b contributes its
//     maximum to its 64-element block through one 16-lane reduce instruction; the few float4 that
//     reach b are only noted;
//   * the noted float4 (about 1.2 k per row) are read again (they are in L1): elements >= b become
//     selection candidates, the others are folded into their block's maximum by a shared-memory
//     atomic;
//   * the candidates are ranked by counting; rank < k is an outlier (emitted), the others go back
//     into their block's maximum.
// So the block maxima never need the zeroed row, and nothing is read twice from HBM.  Rows with Inf or
// NaN, rows the bound cannot split (heavy ties, fewer than k non-zero float4) take an exact path:
// 6-pass radix select, then block maxima with the selected columns masked by a bitmap.
//
// The encoder sweep writes the nibbles of a row into a shared-memory staging buffer; selected columns
// are then patched to the code of 0.0 (the reference zeroes them before it quantises,
// src/bitsqz_llm.cu:1036-1056), and the row leaves by one bulk store.
#pragma once

#include "bsq_rowgroup.cuh"


namespace bsq {


// Where a row comes from: global memory (read-only path) or a shared-memory buffer filled by a bulk copy.
struct GlobalRow {
    const float *p;
    __device__ __forceinline__ float4 v4(unsigned i) const { return __ldg(reinterpret_cast<const float4 *>(p) + i); }
    __device__ __forceinline__ float v1(unsigned col) const { return __ldg(p + col); }
};
struct SharedRow {
    const float *p;
    __device__ __forceinline__ float4 v4(unsigned i) const { return reinterpret_cast<const float4 *>(p)[i]; }
    __device__ __forceinline__ float v1(unsigned col) const { return p[col]; }
};

// body(float4 value, unsigned i0, unsigned j, bool valid) for every float4 of the row: the float4 has index
// i0 + lane, i0 = chunk base + j * L is uniform over the group and a multiple of 32, j is a compile-time constant
// after unrolling.  All lanes of the group call body the same number of times (lanes past the end get zeros and
// valid = false), so it may hold warp collectives.
constexpr unsigned kChunk = 8;                              // float4 per lane in flight

// The first chunk of a row, loaded ahead of its use (lanes past the end get zeros).
template <int G, class Row>
__device__ __forceinline__ void load_first_chunk(const RowGroup<G> &g, const Row &row, unsigned f4, float4 (&a)[kChunk]) {
    constexpr unsigned L = 32 * G;
    if (kChunk * L <= f4) {
#pragma unroll
        for (unsigned j = 0; j < kChunk; ++j) a[j] = row.v4(j * L + g.lane);
    } else {
#pragma unroll
        for (unsigned j = 0; j < kChunk; ++j)
            a[j] = j * L + g.lane < f4 ? row.v4(j * L + g.lane) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

template <int G, bool PRELOADED, class Row, class Body>
__device__ __forceinline__ void for_each_float4_impl(const RowGroup<G> &g, const Row &row, unsigned f4,
                                                     const float4 (&first)[kChunk], Body body) {
    constexpr unsigned L = 32 * G, CH = kChunk;
    unsigned base = 0;
    if (PRELOADED) {
#pragma unroll
        for (unsigned j = 0; j < CH; ++j) body(first[j], j * L, j, j * L + g.lane < f4);
        base = CH * L;
    }
#pragma unroll 1
    for (; base + CH * L <= f4; base += CH * L) {          // whole chunks: no per-load checks
        float4 a[CH];
#pragma unroll
        for (unsigned j = 0; j < CH; ++j) a[j] = row.v4(base + j * L + g.lane);
#pragma unroll
        for (unsigned j = 0; j < CH; ++j) body(a[j], base + j * L, j, true);
    }
    if (base < f4) {                                        // ragged end
        float4 a[CH];
#pragma unroll
        for (unsigned j = 0; j < CH; ++j)
            a[j] = base + j * L + g.lane < f4 ? row.v4(base + j * L + g.lane) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (unsigned j = 0; j < CH; ++j) body(a[j], base + j * L, j, base + j * L + g.lane < f4);
    }
}
template <int G, class Row, class Body>
__device__ __forceinline__ void for_each_float4(const RowGroup<G> &g, const Row &row, unsigned f4, Body body) {
    const float4 none[kChunk] = {};
    for_each_float4_impl<G, false>(g, row, f4, none, body);
}

// Clears what one selection attempt accumulates; a group sync must follow before the scan.
template <int G>
__device__ __forceinline__ void stream_reset(const RowGroup<G> &g, GroupCtl &c) {
    if (g.lane == 0) { c.count = 0; c.nhits = 0; }
    if (g.lane < 8) c.seen[g.lane] = 0u;
    for (unsigned i = g.lane; i < (unsigned)kCandCap / 4; i += RowGroup<G>::L)
        reinterpret_cast<uint4 *>(c.key)[i] = make_uint4(0u, 0u, 0u, 0u);
}

// One sweep with a bound: block maxima of everything below the bound into blk[] (bits of |x|), float4 that reach
// it noted in c.hist[] / c.nhits.  The caller has zeroed c.nhits and synchronised.
template <int G, class Row>
__device__ __forceinline__ void stream_scan(const RowGroup<G> &g, GroupCtl &c, unsigned *blk, const Row &row,
                                            unsigned f4, float bound) {
    // one warp sweep covers two 64-element blocks (lanes 0-15, lanes 16-31): two full-warp reduces on masked
    // values (a reduce over half the warp would split the warp's control flow), lane 0 stores both maxima
    const bool upper = (g.lane & 16) != 0, leader = (g.lane & 31) == 0;
    uint2 *blk_pair = reinterpret_cast<uint2 *>(blk + (g.lane >> 5) * 2);
    for_each_float4<G>(g, row, f4, [&](const float4 &a, unsigned i0, unsigned, bool valid) {
        const float m = absmax4_nan(a);
        const bool hit = !(m < bound);                      // reaches the bound, or is NaN
        const unsigned x = hit ? 0u : __float_as_uint(m);
        const unsigned lo = __reduce_max_sync(kFullMask, upper ? 0u : x);
        const unsigned hi = __reduce_max_sync(kFullMask, upper ? x : 0u);
        if (leader && valid) blk_pair[i0 >> 5] = make_uint2(lo, hi);
        if (hit) note_hit(i0 + g.lane, c);
    });
}

// The noted float4: elements >= bound become candidates, finite ones below it join their block's maximum,
// Inf / NaN raise kFlagSpecial.  Ends without a sync.
template <int G, class Row>
__device__ __forceinline__ void stream_expand(const RowGroup<G> &g, GroupCtl &c, unsigned *blk, const Row &row,
                                              float bound) {
    const unsigned n = min(c.nhits, kHitCap);
    for (unsigned e = g.lane; e < n; e += RowGroup<G>::L) {
        const unsigned i = c.hist[e];
        const float4 a = row.v4(i);
        const float v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const unsigned bits = __float_as_uint(v[q]) & 0x7fffffffu;
            if (bits >= 0x7f800000u) {
                atomicOr(&c.flags, kFlagSpecial);
            } else if (__uint_as_float(bits) >= bound) {
                const unsigned pos = atomicAdd(&c.count, 1u);
                if (pos < (unsigned)kCandCap) {
                    c.key[pos] = bits;
                    c.cand[pos] = topk_composite(v[q], i * 4 + q);
                }
            } else {
                atomicMax(&blk[i >> 4], bits);
            }
        }
    }
}

// Rank the candidates by counting; rank < k: emit (index, value) and publish |x| of the k-th; the others join
// their block's maximum.  Ranks come from 32-bit compares of |x| (c.key[], zero beyond `count`); two candidates of
// equal |x| would get the same rank, which the `seen` bits catch: then everybody ranks on the full composite
// (column ascending breaks the tie).  c.hist[] keeps the ranks.  Ends with a group sync.
template <int G, class Row>
__device__ __forceinline__ void stream_rank_emit(const RowGroup<G> &g, GroupCtl &c, unsigned *blk, const Row &row,
                                                 unsigned count, unsigned k, uint16_t *out_idx, float *out_val) {
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
        const unsigned col = 0xFFFFu - (unsigned)(mine & 0xFFFFull);
        const unsigned bits = (unsigned)(mine >> 16) - 1u;                  // candidates are finite: ukey = bits + 1
        if (rank < k) {
            out_idx[rank] = (uint16_t)col;
            out_val[rank] = row.v1(col);
            if (rank == k - 1) c.kth_bits = bits;
        } else {
            atomicMax(&blk[col >> 6], bits);
        }
    }
    g.sync();
}

// A bound that at least k elements reach: the k-th largest of the lanes' largest float4 maxima (k <= L) or of
// their largest and second-largest ones (k <= 2 L); every value stands for a different float4.  Returns 0 when
// there is none (k > 2 L, or fewer than k non-zero values); raises kFlagSpecial when the row holds Inf or NaN.
// Contains group syncs; all lanes call it.
template <int G, class Row>
__device__ __forceinline__ float stream_bound(const RowGroup<G> &g, GroupCtl &c, const Row &row, unsigned f4,
                                              unsigned k) {
    constexpr unsigned L = RowGroup<G>::L;
    float acc = 0.0f, first = 0.0f, second = 0.0f;
    for_each_float4<G>(g, row, f4, [&](const float4 &a, unsigned, unsigned, bool) {
        const float m = absmax4_nan(a);
        acc = absmax3_nan(acc, m, 0.0f);
        second = fmaxf(second, fminf(first, m));
        first = fmaxf(first, m);
    });
    if (!(acc < __int_as_float(0x7f800000))) atomicOr(&c.flags, kFlagSpecial);
    unsigned *tops = reinterpret_cast<unsigned *>(c.cand);   // 2 L <= 512 words
    const unsigned fb = __float_as_uint(first), sb = __float_as_uint(second);
    const bool both = k > L;                                 // uniform
    tops[g.lane] = fb;
    if (both) tops[L + g.lane] = sb;
    g.sync();
    if ((c.flags & kFlagSpecial) || k > 2u * L) return 0.0f;
    unsigned ge_f = 0, ge_s = 0;
    const uint4 *tops4 = reinterpret_cast<const uint4 *>(tops);
    if (!both) {
#pragma unroll 4
        for (unsigned i = 0; i < L / 4; ++i) {
            const uint4 o = tops4[i];
            ge_f += (o.x >= fb ? 1u : 0u) + (o.y >= fb ? 1u : 0u) + (o.z >= fb ? 1u : 0u) + (o.w >= fb ? 1u : 0u);
        }
    } else {
#pragma unroll 4
        for (unsigned i = 0; i < 2 * L / 4; ++i) {
            const uint4 o = tops4[i];
            ge_f += (o.x >= fb ? 1u : 0u) + (o.y >= fb ? 1u : 0u) + (o.z >= fb ? 1u : 0u) + (o.w >= fb ? 1u : 0u);
            ge_s += (o.x >= sb ? 1u : 0u) + (o.y >= sb ? 1u : 0u) + (o.z >= sb ? 1u : 0u) + (o.w >= sb ? 1u : 0u);
        }
    }
    const unsigned mine = ge_f >= k ? fb : ((both && ge_s >= k) ? sb : 0u);
    return __uint_as_float(g.max_bits(mine, c));             // syncs inside: tops[] is free again afterwards
}

// Exact path: 6-pass radix select, then block maxima with the selected columns masked out and Inf / NaN counted as
// zero (blocks that hold one get bit 31 set: the encoder takes the literal scan there).
template <int G, class Row>
__device__ __noinline__ void stream_exact(const RowGroup<G> &g, GroupCtl &c, unsigned *blk, unsigned *bitmap,
                                          const Row &row, unsigned cols, unsigned k, uint16_t *out_idx,
                                          float *out_val) {
    constexpr unsigned L = RowGroup<G>::L;
    const unsigned f4 = cols >> 2;
    for (unsigned w = g.lane; w < (cols + 31) / 32; w += L) bitmap[w] = 0u;
    if (k > 0) group_topk_exact<G>(g, c, const_cast<float *>(row.p), cols, k, out_idx, out_val, false);   // never writes the row
    else g.sync();
    for (unsigned j = g.lane; j < k; j += L) {
        const unsigned col = out_idx[j];
        atomicOr(&bitmap[col >> 5], 1u << (col & 31));
    }
    g.sync();
    const unsigned half_mask = (g.lane & 16) ? 0xffff0000u : 0x0000ffffu;
    for_each_float4<G>(g, row, f4, [&](const float4 &a, unsigned i0, unsigned, bool valid) {
        const unsigned i = i0 + g.lane;
        const unsigned e[4] = {__float_as_uint(a.x) & 0x7fffffffu, __float_as_uint(a.y) & 0x7fffffffu,
                               __float_as_uint(a.z) & 0x7fffffffu, __float_as_uint(a.w) & 0x7fffffffu};
        const unsigned sel = valid ? (bitmap[i >> 3] >> ((i & 7) * 4)) & 0xFu : 0u;
        unsigned m = 0;
        bool nonfinite = false;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            if ((sel >> q) & 1u) continue;
            if (e[q] < 0x7f800000u) m = max(m, e[q]);
            else nonfinite = true;
        }
        m = __reduce_max_sync(half_mask, m);
        const unsigned nf = __ballot_sync(kFullMask, nonfinite);
        if (valid && (g.lane & 15) == 0) {
            const bool marked = ((nf >> (g.lane & 16)) & 0xFFFFu) != 0;
            blk[i >> 4] = m | (marked ? 0x80000000u : 0u);
        }
    });
    g.sync();
}

// Selection and block maxima of one row.
//   blk    : shared, cols / 64 words; on return the block value as a float, absmax or 1.0 for a block of zeros
//            (quantization_cuda.cu:217-219), NEGATED when the block must take the literal scan
//   bitmap : shared, cols / 32 words (exact path only)
//   hint   : bound guess from the row before (0 = none);  returns the guess for the next row
//   run    : running maximum of the block values of this lane
//   fresh  : stream_reset has run (and c.flags is zero) since the last use of the control block, with a sync behind it
//   reset_after : run stream_reset for the next row before the final sync (whose caller then passes fresh = true):
//            one group sync less per row
//   sync_end = false leaves out the final sync (the caller's next sync then orders the blk[] reads)
// The caller has zeroed c.flags and synchronised the group since; ends with a group sync.
template <int G, class Row>
__device__ __forceinline__ float stream_select_absmax(const RowGroup<G> &g, GroupCtl &c, unsigned *blk, unsigned *bitmap,
                                                      const Row &row, unsigned cols, unsigned k,
                                                      uint16_t *out_idx, float *out_val, float hint, float *absmax_out,
                                                      float *run, bool fresh = false, bool sync_end = true,
                                                      bool reset_after = false) {
    constexpr unsigned L = RowGroup<G>::L;
    const unsigned f4 = cols >> 2, nblk = cols >> 6;
    float next_hint = 0.0f;
    bool done = false;
    if (k > 0) {
        float bound = hint;
        for (int attempt = 0; attempt < 2 && !done; ++attempt) {
            if (!(bound > 0.0f)) {
                bound = stream_bound<G>(g, c, row, f4, k);
                if (!(bound > 0.0f)) break;                  // Inf / NaN, or no usable bound: exact path
                attempt = 1;
            }
            if (!(fresh && attempt == 0 && bound == hint)) {   // a fresh control block is already clean
                stream_reset<G>(g, c);
                g.sync();
            }
            stream_scan<G>(g, c, blk, row, f4, bound);
            g.sync();
            if (c.nhits <= kHitCap) {
                stream_expand<G>(g, c, blk, row, bound);
                g.sync();
                const unsigned count = c.count;
                if (!(c.flags & kFlagSpecial) && count >= k && count <= (unsigned)kCandCap) {
                    stream_rank_emit<G>(g, c, blk, row, count, k, out_idx, out_val);
                    next_hint = __uint_as_float(c.kth_bits) * 0.9375f;
                    done = true;
                }
            }
            if (c.flags & kFlagSpecial) break;
            bound = 0.0f;                                    // the guess was off: compute one
        }
    } else {
        // no selection: plain block maxima; Inf / NaN sends the row to the exact path (which masks them)
        if (g.lane == 0) c.nhits = 0;
        g.sync();
        stream_scan<G>(g, c, blk, row, f4, __int_as_float(0x7f800000));
        g.sync();
        done = c.nhits == 0;
    }
    if (!done) stream_exact<G>(g, c, blk, bitmap, row, cols, k, out_idx, out_val);
    for (unsigned b = g.lane; b < nblk; b += L) {
        const unsigned raw = blk[b];
        const float am = __uint_as_float(raw & 0x7fffffffu);
        const float v = am > 0.0f ? am : 1.0f;
        const float fin = (raw >> 31) ? -v : v;
        if (absmax_out) absmax_out[b] = fin;
        reinterpret_cast<float *>(blk)[b] = fin;
        *run = fmaxf(*run, v);
    }
    if (reset_after) stream_reset<G>(g, c);                  // nothing reads the candidate lists after the ranking's last sync
    if (sync_end) g.sync();
    return next_hint;
}

// Nibbles of one row into the staging buffer `codes` (cols / 2 bytes), blk[] = +-1/scale per block (negative:
// literal scan).  any_slow is uniform over the group.  Ends with a group sync.
// `first` holds the row's first chunk (load_first_chunk).
template <int G, class Row>
__device__ __forceinline__ void stream_encode(const RowGroup<G> &g, const Row &row, unsigned cols, const float4 (&first)[kChunk],
                                              const Nf4Lut &lut, const float *blk, uint16_t *codes, bool any_slow) {
    const unsigned f4 = cols >> 2;
    const float *blk_lane = blk + (g.lane >> 4);
    uint16_t *codes_lane = codes + g.lane;
    for_each_float4_impl<G, true>(g, row, f4, first, [&](const float4 &a, unsigned i0, unsigned, bool valid) {
        const float inv = valid ? fabsf(blk_lane[i0 >> 4]) : 1.0f;
        const unsigned c0 = lut.encode(__fmul_rn(a.x, inv));
        const unsigned c1 = lut.encode(__fmul_rn(a.y, inv));
        const unsigned c2 = lut.encode(__fmul_rn(a.z, inv));
        const unsigned c3 = lut.encode(__fmul_rn(a.w, inv));
        if (valid) codes_lane[i0] = (uint16_t)((c0 << 4) | c1 | (c2 << 12) | (c3 << 8));
    });
    if (any_slow) {                                         // rare: literal scan on sanitised values
        for (unsigned i = g.lane; i < f4; i += RowGroup<G>::L) {
            const float invs = blk[i >> 4];
            if (invs < 0.0f) {
                const float4 a = row.v4(i);
                const float inv = -invs;
                const unsigned c0 = nf4_code_scan(__fmul_rn(sanitize(a.x), inv));
                const unsigned c1 = nf4_code_scan(__fmul_rn(sanitize(a.y), inv));
                const unsigned c2 = nf4_code_scan(__fmul_rn(sanitize(a.z), inv));
                const unsigned c3 = nf4_code_scan(__fmul_rn(sanitize(a.w), inv));
                codes[i] = (uint16_t)((c0 << 4) | c1 | (c2 << 12) | (c3 << 8));
            }
        }
    }
    g.sync();
}

// The selected columns of the row get the code of 0.0 (7).  A lane's share of the row's k column indices is
// loaded ahead of its use (load_selected); out-of-range entries are skipped.  No sync inside.
template <int G>
struct SelectedCols {
    static constexpr unsigned N = kCandCap / (32 * G);
    unsigned col[N];
};
template <int G>
__device__ __forceinline__ void load_selected(const RowGroup<G> &g, const uint16_t *idx, unsigned k, SelectedCols<G> &s) {
#pragma unroll
    for (unsigned j = 0; j < SelectedCols<G>::N; ++j)
        s.col[j] = j * RowGroup<G>::L + g.lane < k ? (unsigned)idx[j * RowGroup<G>::L + g.lane] : 0xFFFFFFFFu;
}
template <int G>
__device__ __forceinline__ void stream_patch_selected(const RowGroup<G> &g, uint16_t *codes, const SelectedCols<G> &s,
                                                      unsigned cols) {
    unsigned *words = reinterpret_cast<unsigned *>(codes);
#pragma unroll
    for (unsigned j = 0; j < SelectedCols<G>::N; ++j) {
        const unsigned col = s.col[j];
        if (col < cols) {
            const unsigned shift = ((col >> 1) & 3u) * 8u + ((col & 1u) ? 0u : 4u);   // byte col / 2, even column = high nibble
            atomicAnd(&words[col >> 3], ~(0xFu << shift));
            atomicOr(&words[col >> 3], 7u << shift);
        }
    }
}

}  // namespace bsq
