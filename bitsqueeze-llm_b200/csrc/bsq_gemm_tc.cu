// Tensor-core GEMM of the low-rank stages: tcgen05.mma (kind::tf32) with the accumulator in tensor
// memory, FP32-level accuracy through 3xTF32 operand splitting (sm_100a).
//
// Used for the skinny products of the randomized SVD that stream the big matrix, C[M x N] = opA * opB
// with N = rank (a multiple of 16, at most 256) and K = a matrix dimension; they replace the
// cublasSgemm calls of the reference (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:293-309,
// 319-335,344-360,370-386).  One CTA owns a 128 x N output tile for one slice of K:
//
//   * operands come straight from the caller's row-major arrays in either orientation and are staged
//     through registers into the tensor core's canonical K-major no-swizzle layout (core matrices of
//     8 rows x 16 B); a source that is contiguous along M or N is transposed in registers on the way
//     (TF32 operands that are MN-major in shared memory would need a swizzled layout);
//   * while staging, every FP32 value x is split into hi = x rounded to TF32 and lo = x - hi rounded to
//     TF32; per 8-wide k-step three MMAs accumulate hi*hi into one FP32 accumulator in tensor memory
//     and lo*hi + hi*lo into a second one, added in the epilogue (the dropped lo*lo term and the
//     rounding of lo are ~2^-22 relative; the tensor core truncates when it accumulates, which leaves
//     an error of a few 1e-7 of sum |a||b| for K in the thousands, against a few 1e-8 on the FP32 pipes);
//   * 256 threads stage 16 of K at a time and keep the global loads of three such chunks in flight in
//     registers, so HBM latency hides behind the staging of earlier chunks; two shared-memory stages:
//     the splits of chunk c+1 overlap the MMAs of chunk c; tcgen05.commit on an mbarrier tells when a
//     stage may be overwritten and when the tile is done; two CTAs share an SM when N <= 128;
//   * the 128 x N FP32 tile is read back with tcgen05.ld (two threads per accumulator row, half the
//     columns each) and written to C or to the K-split workspace.
// Every mbarrier wait is bounded; on a timeout the CTA records it in the status word, still frees its
// tensor memory and leaves.
#include "bsq_device.cuh"
#include "bsq_gemm.hpp"
#include "bsq_gemm_tc.cuh"

#include <cstdlib>

namespace bsq {
namespace {

// Shared-memory position (in 16-byte units) of the 4 consecutive k values kc*4 .. kc*4+3 of row/column r (the MN
// index) of an operand chunk: the tensor core's canonical K-major layout without swizzle.  A core matrix is 8
// consecutive r at one kc (8 x 16 B); core matrices follow one another along MN every 144 B (SBO, padded from 128 B)
// and along K every lbo_units(extent) * 16 B (LBO, padded to 2 modulo 8 units): with these paddings both staging
// patterns below store without bank conflicts.
__host__ __device__ constexpr unsigned lbo_units(int extent) {
    return (unsigned)(extent / 8) * 9u + (10u - ((unsigned)(extent / 8) * 9u) % 8u) % 8u;
}
__host__ __device__ constexpr unsigned stage_units(int extent) { return (TK / 4) * lbo_units(extent); }
__device__ __forceinline__ unsigned unit_index(int kc, int r, int extent) {
    return (unsigned)kc * lbo_units(extent) + (unsigned)(r >> 3) * 9u + (unsigned)(r & 7);
}

// A thread's share of one operand chunk (extent x TK): four float4, fixed over the K loop.  Threads 0-127 serve A
// (one slot each, TM = 128 slots), threads 128-255 serve B (N slots, one or two each).
//   K-major source (K contiguous in global memory): slot s holds k quad kc = s % 4 of the four rows
//       s / 4 + j * extent / 4, j = 0..3, so four neighbouring threads read 64 contiguous bytes of a row;
//   MN-major source: slot s holds 4 consecutive MN indices x 4 consecutive k (four 16-byte loads from four k rows,
//       neighbouring threads neighbouring 16-byte pieces), transposed in registers so that each output unit again
//       holds 4 consecutive k of one MN index.
// Either way a slot fills four 16-byte units of the K-major layout above, hi and lo.  Everything address-like is
// worked out once; per chunk a slot costs four loads, the splits and eight stores.
struct Item {
    float4 v[4];
};

template <bool KMAJOR>
struct Slot {
    const float *src;        // chunk 0
    long step;               // elements from one chunk to the next
    long off[4];             // elements from src to each of the four loads
    unsigned unit[4];        // 16-byte unit of each output in the operand stage
    int kq;                  // k quad of the slot (K-major: of all four loads; MN-major: the loads are its four k)
    bool active;

    // Rows / columns past the end of the matrix (last tile of A) are read from valid memory instead (the last row,
    // or the row's leading elements): what they produce lands in accumulator rows that are never written out.
    __device__ __forceinline__ void init(const float *P, long ld, int mn_total, int mn0, int k_begin, int extent, int s) {
        active = s < extent;
        const int ss = active ? s : 0;
        if (KMAJOR) {
            kq = ss % 4;
            const int r0 = ss / 4, rstep = extent / 4;
            src = P + k_begin + kq * 4;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                unit[j] = unit_index(kq, r0 + j * rstep, extent);
                off[j] = (long)min(mn0 + r0 + j * rstep, mn_total - 1) * ld;
            }
            step = TK;
        } else {
            const int e4 = extent / 4;
            const int mn4 = ss % e4;
            kq = ss / e4;
            const int gmn = mn0 + mn4 * 4;
            src = P + (long)(k_begin + kq * 4) * ld + (gmn < mn_total ? gmn : 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                unit[j] = unit_index(kq, mn4 * 4 + j, extent);
                off[j] = (long)j * ld;
            }
            step = (long)TK * ld;
        }
    }
    // whole chunk
    __device__ __forceinline__ void load(Item &it, int c) const {
        const float *p = src + (long)c * step;
#pragma unroll
        for (int j = 0; j < 4; ++j) it.v[j] = *reinterpret_cast<const float4 *>(p + off[j]);
    }
    // last chunk of a K range that is no multiple of TK: only k_left of its TK values exist
    __device__ __forceinline__ void load_checked(Item &it, int c, int k_left) const {
        const float *p = src + (long)c * step;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (KMAJOR) {
                const int left = k_left - kq * 4;
                if (left >= 4) v = *reinterpret_cast<const float4 *>(p + off[j]);
                else if (left > 0) { v.x = p[off[j]]; if (left > 1) v.y = p[off[j] + 1]; if (left > 2) v.z = p[off[j] + 2]; }
            } else if (kq * 4 + j < k_left) {
                v = *reinterpret_cast<const float4 *>(p + off[j]);
            }
            it.v[j] = v;
        }
    }
    // opA(i, kk) *= sc[kk] for the chunk whose first k sc points at (k_left of its TK values exist)
    __device__ __forceinline__ void scale(Item &it, const float *sc, int k_left) const {
        if (KMAJOR) {
            float f[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) f[q] = kq * 4 + q < k_left ? sc[kq * 4 + q] : 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) { it.v[j].x *= f[0]; it.v[j].y *= f[1]; it.v[j].z *= f[2]; it.v[j].w *= f[3]; }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float f = kq * 4 + j < k_left ? sc[kq * 4 + j] : 0.0f;
                it.v[j].x *= f; it.v[j].y *= f; it.v[j].z *= f; it.v[j].w *= f;
            }
        }
    }
    __device__ __forceinline__ void store(const Item &it, float4 *hi, float4 *lo) const {
        if (KMAJOR) {
#pragma unroll
            for (int j = 0; j < 4; ++j) split_store(it.v[j], hi + unit[j], lo + unit[j]);
        } else {
            const float4 v0 = it.v[0], v1 = it.v[1], v2 = it.v[2], v3 = it.v[3];
            split_store(make_float4(v0.x, v1.x, v2.x, v3.x), hi + unit[0], lo + unit[0]);
            split_store(make_float4(v0.y, v1.y, v2.y, v3.y), hi + unit[1], lo + unit[1]);
            split_store(make_float4(v0.z, v1.z, v2.z, v3.z), hi + unit[2], lo + unit[2]);
            split_store(make_float4(v0.w, v1.w, v2.w, v3.w), hi + unit[3], lo + unit[3]);
        }
    }
};

// descriptor of the 8-wide k-step `ks` inside a stage
__device__ __forceinline__ uint64_t kstep_desc(unsigned stage_addr, int ks, int extent) {
    return smem_desc(stage_addr + (unsigned)(ks * 2) * lbo_units(extent) * 16u, lbo_units(extent) * 16u, 144u);
}

// Epilogue of both product kernels, for warps 0-7: accumulator row 32 (warp % 4) + lane; warps 0-3 take the lower half
// of the columns, warps 4-7 the upper half.  Adds the two accumulators and writes C (or minuend - product).
__device__ __forceinline__ void tile_epilogue(const GemmArgs &g, unsigned tmem_d, unsigned acc_cols, int chunks, bool ok, int m0, int n0,
                                              int N, int warp, int tid) {
    float *C = g.C + (long)blockIdx.z * g.split_stride;
    const int row = m0 + (warp & 3) * 32 + (tid & 31);
    const int half = (N / 16 + 1) / 2 * 16;                  // columns of the lower half, a multiple of 16
    const int c_begin = warp < 4 ? 0 : half, c_end = warp < 4 ? half : N;
    bool any = false;
    // 32-byte stores need 32-byte aligned rows of C (tile columns start at multiples of 16)
    const bool wide32 = (reinterpret_cast<uintptr_t>(g.C) | (uintptr_t)(g.ldc * 4) | (uintptr_t)(g.split_stride * 4)) % 32 == 0;
    if (ok) {
        for (int c0 = c_begin; c0 < c_end; c0 += 16) {
            unsigned r[16], q[16];
            if (chunks > 0) {
                const unsigned taddr = tmem_d + ((unsigned)((warp & 3) * 32) << 16) + (unsigned)c0;
                tmem_ld16(taddr, r);
                tmem_ld16(taddr + acc_cols, q);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(q[j])));
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) r[j] = 0u;
            }
            if (row < g.M) {
                float4 *dst = reinterpret_cast<float4 *>(C + (long)row * g.ldc + n0 + c0);
                if (g.minuend) {                             // C = minuend - product, note whether anything is left
                    const float4 *mn = reinterpret_cast<const float4 *>(g.minuend + (long)row * g.ldm + n0 + c0);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 m4 = mn[j];
                        const float4 o = make_float4(__fsub_rn(m4.x, __uint_as_float(r[4 * j])), __fsub_rn(m4.y, __uint_as_float(r[4 * j + 1])),
                                                     __fsub_rn(m4.z, __uint_as_float(r[4 * j + 2])), __fsub_rn(m4.w, __uint_as_float(r[4 * j + 3])));
                        any |= fabsf(o.x) > 1.1920928955078125e-07f || fabsf(o.y) > 1.1920928955078125e-07f ||
                               fabsf(o.z) > 1.1920928955078125e-07f || fabsf(o.w) > 1.1920928955078125e-07f;
                        dst[j] = o;
                    }
                } else if (wide32) {
                    st_global_v8(reinterpret_cast<float *>(dst), make_float4(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]), __uint_as_float(r[3])),
                                 make_float4(__uint_as_float(r[4]), __uint_as_float(r[5]), __uint_as_float(r[6]), __uint_as_float(r[7])));
                    st_global_v8(reinterpret_cast<float *>(dst + 2), make_float4(__uint_as_float(r[8]), __uint_as_float(r[9]), __uint_as_float(r[10]), __uint_as_float(r[11])),
                                 make_float4(__uint_as_float(r[12]), __uint_as_float(r[13]), __uint_as_float(r[14]), __uint_as_float(r[15])));
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                             __uint_as_float(r[4 * j + 3]));
                }
            }
        }
    }
    if (g.flag && __any_sync(0xffffffffu, any) && (tid & 31) == 0) atomicOr(g.flag, 1u);
}

template <bool A_KMAJOR, bool B_KMAJOR, int NMAX>
__global__ void __launch_bounds__(NT) gemm_tc_kernel(GemmArgs g, unsigned *status) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_free[STAGES];
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ unsigned tmem_base_slot;
    constexpr int ITEMS = NMAX / (NT - TM);                   // slots of B per serving thread: 1 (N <= 128) or 2
    const int tid = threadIdx.x, warp = tid >> 5;
    const int n0 = blockIdx.y * g.n_tile;                     // this CTA's columns: n0 .. n0 + N
    const int N = min(g.n_tile, g.N - n0);                    // multiple of 16, <= NMAX
    const int m0 = blockIdx.x * TM;
    const int k_begin = blockIdx.z * g.k_per_split;
    const int k_end = min(g.K, k_begin + g.k_per_split);
    const unsigned a_units = stage_units(TM), b_units = stage_units(N);
    const unsigned stage_bytes = (2 * a_units + 2 * b_units) * 16u;       // stage: [A hi | A lo | B hi | B lo]
    // two accumulators: the hi*hi chain and, half the allocation further on, the two small cross terms
    const unsigned acc_cols = N <= 16 ? 16u : (N <= 32 ? 32u : (N <= 64 ? 64u : (N <= 128 ? 128u : 256u)));
    const unsigned tmem_cols = 2u * acc_cols;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < STAGES; ++i) mbar_init(&bar_free[i], 1);
        mbar_init(&bar_done, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = tmem_base_slot;

    // instruction descriptor: FP32 accumulate, TF32 x TF32, both operands K-major in shared memory, N >> 3, M >> 4
    const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(TM >> 4) << 24);

    // threads 0-127: one slot of A each; threads 128-255: one or two slots of B each
    const bool serves_a = tid < TM;
    Slot<A_KMAJOR> slot_a;
    Slot<B_KMAJOR> slot_b[ITEMS];
    slot_a.init(g.A, g.lda, g.M, m0, k_begin, TM, serves_a ? tid : TM);
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) slot_b[i].init(g.B, g.ldb, g.N, n0, k_begin, N, serves_a ? N : tid - TM + i * (NT - TM));
    Item regs[DEPTH][ITEMS];
    auto load_chunk = [&](Item(&r)[ITEMS], int c, int k_left) {
        if (k_left >= TK) {
            if (serves_a) {
                slot_a.load(r[0], c);
                if (g.kscale) slot_a.scale(r[0], g.kscale + k_begin + c * TK, TK);
            } else {
#pragma unroll
                for (int i = 0; i < ITEMS; ++i)
                    if (slot_b[i].active) slot_b[i].load(r[i], c);
            }
        } else if (serves_a) {
            slot_a.load_checked(r[0], c, k_left);
            if (g.kscale) slot_a.scale(r[0], g.kscale + k_begin + c * TK, k_left);
        } else {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i)
                if (slot_b[i].active) slot_b[i].load_checked(r[i], c, k_left);
        }
    };
    auto store_chunk = [&](const Item(&r)[ITEMS], float4 *a_hi, float4 *a_lo, float4 *b_hi, float4 *b_lo) {
        if (serves_a) {
            slot_a.store(r[0], a_hi, a_lo);
        } else {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i)
                if (slot_b[i].active) slot_b[i].store(r[i], b_hi, b_lo);
        }
    };

    const int chunks = (k_end - k_begin + TK - 1) / TK;
    bool ok = true;
    unsigned free_phase = 0;                                  // bit s: parity of the next wait on bar_free[s]
#pragma unroll
    for (int d = 0; d < DEPTH; ++d)
        if (d < chunks) load_chunk(regs[d], d, k_end - k_begin - d * TK);
    for (int c0 = 0; c0 < chunks && ok; c0 += DEPTH) {
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int c = c0 + d;
            if (c < chunks && ok) {                           // uniform over the CTA
                const int s = c % STAGES;
                bool mine = true;
                if (c >= STAGES) {                            // the MMAs of chunk c - STAGES must be done with stage s
                    mine = mbar_wait_bounded(&bar_free[s], (free_phase >> s) & 1u, status);
                    free_phase ^= 1u << s;
                }
                float4 *a_hi = reinterpret_cast<float4 *>(smem_raw + (size_t)s * stage_bytes), *a_lo = a_hi + a_units,
                       *b_hi = a_lo + a_units, *b_lo = b_hi + b_units;
                store_chunk(regs[d], a_hi, a_lo, b_hi, b_lo);
                if (c + DEPTH < chunks) load_chunk(regs[d], c + DEPTH, k_end - k_begin - (c + DEPTH) * TK);
                fence_proxy_async_smem();                     // generic-proxy stores -> tensor-core (async proxy) reads
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                ok = __syncthreads_and(mine) != 0;            // uniform: after a timeout nobody issues or loops on
                if (tid == 0 && ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_hi_addr = smem_u32(a_hi), a_lo_addr = smem_u32(a_lo);
                    const unsigned b_hi_addr = smem_u32(b_hi), b_lo_addr = smem_u32(b_lo);
#pragma unroll
                    for (int ks = 0; ks < TK / 8; ++ks) {
                        const uint64_t dah = kstep_desc(a_hi_addr, ks, TM), dal = kstep_desc(a_lo_addr, ks, TM);
                        const uint64_t dbh = kstep_desc(b_hi_addr, ks, N), dbl = kstep_desc(b_lo_addr, ks, N);
                        mma_tf32(tmem_d, dah, dbh, idesc, c > 0 || ks > 0);
                        mma_tf32(tmem_d + acc_cols, dal, dbh, idesc, c > 0 || ks > 0);
                        mma_tf32(tmem_d + acc_cols, dah, dbl, idesc, true);
                    }
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                     smem_u32(c + 1 == chunks ? &bar_done : &bar_free[s]))
                                 : "memory");
                }
            }
        }
    }
    if (chunks > 0 && ok) ok = mbar_wait_bounded(&bar_done, 0, status);
    ok = __syncthreads_and(ok) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    tile_epilogue(g, tmem_d, acc_cols, chunks, ok, m0, n0, N, warp, tid);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same product with the B operand split beforehand.  In the kernel above every CTA splits its B chunk again
// although all CTAs of a tile column use the same values, and half (N = 128) or two thirds (N = 256) of the staging
// instructions go into that.  Here one small kernel writes, once per product, the hi / lo images of B exactly as a
// stage of shared memory wants them (per 16 of K and tile column: [B hi | B lo] in the padded K-major layout), and
// the product kernel fetches one image per chunk with a single bulk copy (TMA, 1-D) that counts off on an mbarrier.
// All 256 staging threads then serve A, half a slot each; a ninth warp does nothing but issue the MMAs (one lane:
// wait for the chunk's image, six MMAs from descriptors that differ from precomputed ones by an addition, one
// commit), because that chain of dependent instructions is what bounds the time per chunk.  B images have a ring of
// their own (NB stages): a copy takes longer than one chunk's MMAs.  Staging thread 0 starts a copy as soon as it
// has seen the MMAs of two chunks ago finish, which is also what frees that chunk's image.
constexpr int NT2 = NT + 32;     // 8 staging / epilogue warps + the control warp
constexpr int IMG_DEPTH_2CTA = 3, IMG_DEPTH_1CTA = 3;
constexpr int MAX_RING = 8;      // most stages of A, and most images of B, in shared memory

// Half of a Slot: two 16-byte units of the operand stage per chunk.
//   K-major source: k quad kq of two rows (64 contiguous bytes per four neighbouring threads, as in Slot);
//   MN-major source: 2 consecutive MN indices x 4 consecutive k (four 8-byte loads), transposed in registers.
struct HalfItem {
    float2 v[4];
};

template <bool KMAJOR>
struct HalfSlot {
    const float *src;
    long step;
    long off[KMAJOR ? 2 : 4];
    unsigned unit[2];
    int kq;

    __device__ __forceinline__ void init(const float *P, long ld, int mn_total, int mn0, int k_begin, int extent, int hs) {
        if (KMAJOR) {
            const int s = hs % extent, h = hs / extent;       // slot of the full scheme and which half of its rows
            kq = s % 4;
            const int r0 = s / 4, rstep = extent / 4;
            src = P + k_begin + kq * 4;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                unit[j] = unit_index(kq, r0 + (2 * h + j) * rstep, extent);
                off[j] = (long)min(mn0 + r0 + (2 * h + j) * rstep, mn_total - 1) * ld;
            }
            step = TK;
        } else {
            const int e2 = extent / 2;
            const int mn2 = hs % e2;
            kq = hs / e2;
            const int gmn = mn0 + mn2 * 2;
            src = P + (long)(k_begin + kq * 4) * ld + (gmn < mn_total ? gmn : 0);
#pragma unroll
            for (int j = 0; j < 4; ++j) off[j] = (long)j * ld;
            unit[0] = unit_index(kq, mn2 * 2, extent);
            unit[1] = unit_index(kq, mn2 * 2 + 1, extent);
            step = (long)TK * ld;
        }
    }
    __device__ __forceinline__ void load(HalfItem &it, int c) const {
        const float *p = src + (long)c * step;
        if (KMAJOR) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float4 v = *reinterpret_cast<const float4 *>(p + off[j]);
                it.v[2 * j] = make_float2(v.x, v.y);
                it.v[2 * j + 1] = make_float2(v.z, v.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) it.v[j] = *reinterpret_cast<const float2 *>(p + off[j]);
        }
    }
    __device__ __forceinline__ void load_checked(HalfItem &it, int c, int k_left) const {
        const float *p = src + (long)c * step;
        if (KMAJOR) {
            const int left = k_left - kq * 4;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (left >= 4) v = *reinterpret_cast<const float4 *>(p + off[j]);
                else if (left > 0) { v.x = p[off[j]]; if (left > 1) v.y = p[off[j] + 1]; if (left > 2) v.z = p[off[j] + 2]; }
                it.v[2 * j] = make_float2(v.x, v.y);
                it.v[2 * j + 1] = make_float2(v.z, v.w);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                it.v[j] = kq * 4 + j < k_left ? *reinterpret_cast<const float2 *>(p + off[j]) : make_float2(0.f, 0.f);
        }
    }
    __device__ __forceinline__ void scale(HalfItem &it, const float *sc, int k_left) const {
        float f[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) f[q] = kq * 4 + q < k_left ? sc[kq * 4 + q] : 0.0f;
        if (KMAJOR) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                it.v[2 * j].x *= f[0]; it.v[2 * j].y *= f[1]; it.v[2 * j + 1].x *= f[2]; it.v[2 * j + 1].y *= f[3];
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) { it.v[j].x *= f[j]; it.v[j].y *= f[j]; }
        }
    }
    __device__ __forceinline__ void store(const HalfItem &it, float4 *hi, float4 *lo) const {
        if (KMAJOR) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
                split_store(make_float4(it.v[2 * j].x, it.v[2 * j].y, it.v[2 * j + 1].x, it.v[2 * j + 1].y), hi + unit[j], lo + unit[j]);
        } else {
            split_store(make_float4(it.v[0].x, it.v[1].x, it.v[2].x, it.v[3].x), hi + unit[0], lo + unit[0]);
            split_store(make_float4(it.v[0].y, it.v[1].y, it.v[2].y, it.v[3].y), hi + unit[1], lo + unit[1]);
        }
    }
};

// One thread per (chunk, k quad, column): the four values B(16 c + 4 kc .. + 3, n0 + r) split into the hi and the lo
// unit of the chunk's image.  k past K gives zeros.
template <bool B_KMAJOR>
__global__ void __launch_bounds__(256) presplit_b_kernel(const float *__restrict__ B, long ldb, int N, int K, int n_tile, int chunks,
                                                         float4 *__restrict__ image) {
    const int n0 = blockIdx.y * n_tile;
    const int Nt = min(n_tile, N - n0);
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)chunks * 4 * Nt) return;
    int kc, r;
    long c;
    if (B_KMAJOR) {                                           // four neighbouring threads read 64 contiguous bytes
        kc = (int)(idx % 4);
        r = (int)((idx / 4) % Nt);
    } else {                                                  // neighbouring threads read neighbouring columns
        r = (int)(idx % Nt);
        kc = (int)((idx / Nt) % 4);
    }
    c = idx / (4 * Nt);
    const long k = c * TK + kc * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (B_KMAJOR) {
        const float *p = B + (long)(n0 + r) * ldb + k;
        if (k + 3 < K) {
            const float4 q = *reinterpret_cast<const float4 *>(p);
            v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (k + j < K) v[j] = p[j];
        }
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (k + j < K) v[j] = B[(k + j) * ldb + n0 + r];
    }
    float4 *img = image + ((size_t)blockIdx.y * chunks + c) * image_units(n_tile);
    const unsigned u = image_unit_index(kc, r, Nt);
    split_store(make_float4(v[0], v[1], v[2], v[3]), img + u, img + image_half_units(Nt) + u);
}

// A (contiguous along K, times kscale) split into two row-major rows_pad x K matrices, hi then lo, four k per thread;
// rows past M are zeros.  The values are those the product kernel's transform warps would make of the same A.
__global__ void __launch_bounds__(256) presplit_a_kernel(const float *__restrict__ A, long lda, int M, int K, const float *__restrict__ kscale,
                                                         float *__restrict__ image, int rows_pad) {
    const int k4 = K / 4;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)rows_pad * k4) return;
    const int m = (int)(idx / k4), k = (int)(idx % k4) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < M) {
        v = *reinterpret_cast<const float4 *>(A + (long)m * lda + k);
        if (kscale) { v.x *= kscale[k]; v.y *= kscale[k + 1]; v.z *= kscale[k + 2]; v.w *= kscale[k + 3]; }
    }
    float4 *hi = reinterpret_cast<float4 *>(image + (long)m * K + k);
    split_store(v, hi, hi + (long)rows_pad * k4);
}

// The largest |x| of a rows x cols matrix (leading dimension ld) as float bits, by atomicMax into *out (cleared by the
// caller).  Non-finite values leave bits >= 0x7f800000 there, which split16_scale answers with... a scale that no
// longer matters: the product is NaN or Inf then, as it is for the reference.
__global__ void __launch_bounds__(256) absmax_bits_kernel(const float *__restrict__ x, long ld, int rows, int cols, unsigned *out,
                                                          const float *__restrict__ colscale = nullptr) {
    const int c4 = cols / 4;
    unsigned m = 0;
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < (long)rows * c4; e += (long)gridDim.x * blockDim.x) {
        float4 v = *reinterpret_cast<const float4 *>(x + (e / c4) * ld + (e % c4) * 4);
        if (colscale) {
            const int c = (int)(e % c4) * 4;
            v.x *= colscale[c]; v.y *= colscale[c + 1]; v.z *= colscale[c + 2]; v.w *= colscale[c + 3];
        }
        m = max(max(m, __float_as_uint(v.x) & 0x7fffffffu), max(__float_as_uint(v.y) & 0x7fffffffu, max(__float_as_uint(v.z) & 0x7fffffffu, __float_as_uint(v.w) & 0x7fffffffu)));
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

// The FP16 form of presplit_b_kernel: one thread per (chunk of 32 k, unit of 8 k, column): the eight values
// B(32 c + 8 kc .. + 7, n0 + r), scaled, as the hi and the lo unit of the chunk's image (same unit order and image size
// as the TF32 images, which hold 16 k per chunk).  k past K gives zeros.
template <bool B_KMAJOR>
__global__ void __launch_bounds__(256) presplit_b16_kernel(const float *__restrict__ B, long ldb, int N, int K, int n_tile, int chunks,
                                                           uint4 *__restrict__ image, const unsigned *__restrict__ absmax_bits, float fixed_scale,
                                                           float lo_scale) {
    const int n0 = blockIdx.y * n_tile;
    const int Nt = min(n_tile, N - n0);
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)chunks * 4 * Nt) return;
    int kc, r;
    if (B_KMAJOR) {
        kc = (int)(idx % 4);
        r = (int)((idx / 4) % Nt);
    } else {
        r = (int)(idx % Nt);
        kc = (int)((idx / Nt) % 4);
    }
    const long c = idx / (4 * Nt);
    const long k = c * 32 + kc * 8;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (B_KMAJOR) {
        const float *p = B + (long)(n0 + r) * ldb + k;
        if (k + 7 < K) {
            const float4 q0 = *reinterpret_cast<const float4 *>(p), q1 = *reinterpret_cast<const float4 *>(p + 4);
            v[0] = q0.x; v[1] = q0.y; v[2] = q0.z; v[3] = q0.w; v[4] = q1.x; v[5] = q1.y; v[6] = q1.z; v[7] = q1.w;
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (k + j < K) v[j] = p[j];
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (k + j < K) v[j] = B[(k + j) * ldb + n0 + r];
    }
    uint4 *img = image + ((size_t)blockIdx.y * chunks + c) * image_units(n_tile);
    const unsigned u = image_unit_index(kc, r, Nt);
    split16_store8(make_float4(v[0], v[1], v[2], v[3]), make_float4(v[4], v[5], v[6], v[7]), fixed_scale > 0.0f ? fixed_scale : split16_scale(*absmax_bits), img + u,
                   img + image_half_units(Nt) + u, lo_scale);
}

// The FP16 form of presplit_a_kernel: two row-major rows_pad x K matrices of FP16 values, hi then lo, eight k per thread;
// the scale comes from *absmax_bits, the largest |A(m, k) kscale(k)| (absmax_bits_kernel with the same kscale).
__global__ void __launch_bounds__(256) presplit_a16_kernel(const float *__restrict__ A, long lda, int M, int K, const float *__restrict__ kscale,
                                                           uint4 *__restrict__ image, int rows_pad, const unsigned *__restrict__ absmax_bits,
                                                           float lo_scale) {
    const int k8 = K / 8;
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)rows_pad * k8) return;
    const int m = (int)(idx / k8), k = (int)(idx % k8) * 8;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
    if (m < M) {
        a = *reinterpret_cast<const float4 *>(A + (long)m * lda + k);
        b = *reinterpret_cast<const float4 *>(A + (long)m * lda + k + 4);
        if (kscale) {
            a.x *= kscale[k]; a.y *= kscale[k + 1]; a.z *= kscale[k + 2]; a.w *= kscale[k + 3];
            b.x *= kscale[k + 4]; b.y *= kscale[k + 5]; b.z *= kscale[k + 6]; b.w *= kscale[k + 7];
        }
    }
    uint4 *hi = image + idx;
    split16_store8(a, b, split16_scale(*absmax_bits), hi, hi + (long)rows_pad * k8, lo_scale);
}

template <bool A_KMAJOR, int NMAX>
__global__ void __launch_bounds__(NT2, NMAX <= 128 ? 2 : 1) gemm_tc_image_kernel(GemmArgs g, unsigned *status) {
    // chunks of A in flight in registers per thread: what is in flight per SM is what bounds these products (the
    // pieces of A are small and far apart in HBM), so as many as the registers of 2 CTAs (N <= 128) or 1 CTA hold
    constexpr int DEPTH = NMAX <= 128 ? IMG_DEPTH_2CTA : IMG_DEPTH_1CTA;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_free[MAX_RING];       // A stage may be overwritten (MMAs that read it are done)
    __shared__ __align__(8) uint64_t bar_b_full[MAX_RING];          // B image has landed
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ unsigned tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    const bool control = warp == NT / 32;                     // the ninth warp; its lane 0 does the work
    const int n0 = blockIdx.y * g.n_tile;
    const int N = min(g.n_tile, g.N - n0);
    const int m0 = blockIdx.x * TM;
    const int k_begin = blockIdx.z * g.k_per_split;
    const int k_end = min(g.K, k_begin + g.k_per_split);
    const unsigned a_units = stage_units(TM), b_units = image_half_units(N);
    const unsigned a_stage_bytes = 2 * a_units * 16u, b_stage_bytes = 2 * b_units * 16u;
    const int SA = g.a_stages, NB = g.b_stages;               // ring lengths: A stages, B images (NB > SA: the copies' head start)
    unsigned char *b_stages = smem_raw + (size_t)SA * a_stage_bytes;
    const unsigned acc_cols = N <= 16 ? 16u : (N <= 32 ? 32u : (N <= 64 ? 64u : (N <= 128 ? 128u : 256u)));
    const unsigned tmem_cols = 2u * acc_cols;

    if (tid == 0) {
        for (int i = 0; i < SA; ++i) mbar_init(&bar_free[i], 1);
        for (int i = 0; i < NB; ++i) mbar_init(&bar_b_full[i], 1);
        mbar_init(&bar_done, 1);
        mbar_fence_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = tmem_base_slot;
    const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(TM >> 4) << 24);

    const int chunks = (k_end - k_begin + TK - 1) / TK;
    const int chunks_total = (g.K + TK - 1) / TK;
    const float4 *image = g.b_image + ((size_t)blockIdx.y * chunks_total + k_begin / TK) * image_units(g.n_tile);
    const bool lane0 = control && (tid & 31) == 0;
    int issued = 0;                                           // thread 0: B copies started
    auto fetch_b = [&](int c) {                               // thread 0: image of chunk c into its ring stage
        uint64_t *bar = &bar_b_full[c % NB];
        mbar_expect_tx(bar, b_stage_bytes);
        bulk_g2s(b_stages + (size_t)(c % NB) * b_stage_bytes, image + (size_t)c * image_units(g.n_tile), b_stage_bytes, bar);
        ++issued;
    };
    if (tid == 0)
        for (int c = 0; c < NB && c < chunks; ++c) fetch_b(c);
    // descriptors of stage 0, k-step 0 (hi); the others differ in the address field only, by whole 16-byte units
    const uint64_t desc_a0 = smem_desc(smem_u32(smem_raw), lbo_units(TM) * 16u, 144u);
    const uint64_t desc_b0 = smem_desc(smem_u32(b_stages), (unsigned)N * 16u, 128u);
    const unsigned a_kstep = 2 * lbo_units(TM), b_kstep = 2u * (unsigned)N;          // units from one 8-wide k-step to the next

    HalfSlot<A_KMAJOR> slot;
    slot.init(g.A, g.lda, g.M, m0, k_begin, TM, control ? 0 : tid);
    HalfItem regs[DEPTH];
    auto load_chunk = [&](HalfItem &r, int c, int k_left) {
        if (control) return;
        if (k_left >= TK) {
            slot.load(r, c);
            if (g.kscale) slot.scale(r, g.kscale + k_begin + c * TK, TK);
        } else {
            slot.load_checked(r, c, k_left);
            if (g.kscale) slot.scale(r, g.kscale + k_begin + c * TK, k_left);
        }
    };
    bool ok = true, mine = true;                              // mine: this thread's waits so far succeeded
    unsigned free_phase = 0;
#pragma unroll
    for (int d = 0; d < DEPTH; ++d)
        if (d < chunks) load_chunk(regs[d], d, k_end - k_begin - d * TK);
    for (int c0 = 0; c0 < chunks && ok; c0 += DEPTH) {
#pragma unroll
        for (int d = 0; d < DEPTH; ++d) {
            const int c = c0 + d;
            if (c < chunks && ok) {                           // uniform over the CTA
                const int s = c % SA;
                float4 *a_hi = reinterpret_cast<float4 *>(smem_raw + (size_t)s * a_stage_bytes), *a_lo = a_hi + a_units;
                if (!control) {
                    if (c >= SA) {                            // the MMAs of chunk c - SA must be done with stage s
                        mine = mbar_wait_bounded(&bar_free[s], (free_phase >> s) & 1u, status);
                        free_phase ^= 1u << s;
                        // ... and with that chunk's image of B: the next one for its place in the ring can come
                        if (tid == 0 && mine && c - SA + NB < chunks) fetch_b(c - SA + NB);
                    }
                    slot.store(regs[d], a_hi, a_lo);
                    if (c + DEPTH < chunks) load_chunk(regs[d], c + DEPTH, k_end - k_begin - (c + DEPTH) * TK);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                ok = __syncthreads_and(mine) != 0;            // uniform: after a timeout nobody issues or loops on
                if (lane0 && ok) {
                    // The stores of all staging threads happen before this point (the CTA barrier); the fence that hands
                    // them from the generic proxy to the tensor core's (async) proxy is executed here, by the one thread
                    // that issues the MMAs.  A fence in every staging thread also waits for that thread's global loads
                    // in flight, which costs a memory latency per chunk.
                    fence_proxy_async_smem();
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const int sb = c % NB;
                    mine = mbar_wait_bounded(&bar_b_full[sb], (unsigned)(c / NB) & 1u, status);
                    if (mine) {
                        const uint64_t dah0 = desc_a0 + (uint64_t)((unsigned)s * 2u * a_units), dbh0 = desc_b0 + (uint64_t)((unsigned)sb * 2u * b_units);
#pragma unroll
                        for (int ks = 0; ks < TK / 8; ++ks) {
                            const uint64_t dah = dah0 + (uint64_t)(ks * a_kstep), dal = dah + a_units;
                            const uint64_t dbh = dbh0 + (uint64_t)(ks * b_kstep), dbl = dbh + b_units;
                            mma_tf32(tmem_d, dah, dbh, idesc, c > 0 || ks > 0);
                            mma_tf32(tmem_d + acc_cols, dal, dbh, idesc, c > 0 || ks > 0);
                            mma_tf32(tmem_d + acc_cols, dah, dbl, idesc, true);
                        }
                        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                         smem_u32(c + 1 == chunks ? &bar_done : &bar_free[s]))
                                     : "memory");
                    }
                }
            }
        }
    }
    if (chunks > 0 && ok) ok = mbar_wait_bounded(&bar_done, 0, status);
    ok = __syncthreads_and(ok && mine) != 0;
    if (tid == 0 && !ok) {
        // leaving early: the copies still in flight must have landed before this CTA's shared memory goes away (a
        // wait for an image that was already used returns at once)
        for (int c = max(0, issued - NB); c < issued; ++c) mbar_wait_bounded(&bar_b_full[c % NB], (unsigned)(c / NB) & 1u, status);
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!control) tile_epilogue(g, tmem_d, acc_cols, chunks, ok, m0, n0, N, warp, tid);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
    }
}

// STAGES stages of [A hi | A lo | B hi | B lo]; padded so that no more CTAs share an SM than their tensor-memory
// allocations (2 * N columns of 512) allow: a CTA too many would sit in tcgen05.alloc until another one leaves.
size_t tc_smem_bytes(int N) {
    const size_t need = (size_t)STAGES * (2 * stage_units(TM) + 2 * stage_units(N)) * 16;
    const size_t floor = N > 128 ? 116 * 1024 : (N > 64 ? 78 * 1024 : (N > 32 ? 56 * 1024 : 0));
    return need > floor ? need : floor;
}

template <bool AK, bool BK, int NMAX>
cudaError_t launch(const GemmArgs &g, unsigned *status, cudaStream_t stream) {
    const size_t smem = tc_smem_bytes(g.n_tile);
    cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<AK, BK, NMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    dim3 grid((g.M + TM - 1) / TM, (g.N + g.n_tile - 1) / g.n_tile, g.splits);
    gemm_tc_kernel<AK, BK, NMAX><<<grid, NT, smem, stream>>>(g, status);
    return cudaGetLastError();
}

// Ring lengths of the image kernel for a tile of N columns: two stages of A and four images of B (two chunks of head
// start for the copies).  Longer rings (up to 6 + 8, one CTA per SM) measured the same for N = 256 and slower for
// N = 128, where they cost the second CTA on the SM.  BSQ_TC_SA / BSQ_TC_NB override them for experiments.
void tc_image_rings(int N, int *sa, int *nb) {
    static const int env_sa = [] { const char *e = std::getenv("BSQ_TC_SA"); return e ? atoi(e) : 0; }();
    static const int env_nb = [] { const char *e = std::getenv("BSQ_TC_NB"); return e ? atoi(e) : 0; }();
    *sa = 2;
    *nb = 4;
    if (env_sa >= 2 && env_sa <= MAX_RING && env_nb > env_sa && env_nb <= MAX_RING) {
        *sa = env_sa;
        *nb = env_nb;
    }
    while (((size_t)*sa * 2 * stage_units(TM) + (size_t)*nb * 2 * image_half_units(N)) * 16 > 226 * 1024 && *sa > 2) {
        --*sa;
        --*nb;
    }
}
size_t tc_image_smem_bytes(int N, int sa, int nb) { return ((size_t)sa * 2 * stage_units(TM) + (size_t)nb * 2 * image_half_units(N)) * 16; }

template <bool AK, int NMAX>
cudaError_t launch_image(const GemmArgs &g, bool b_kmajor, unsigned *status, cudaStream_t stream) {
    const int chunks = g.f16 ? (g.K + 31) / 32 : (g.K + TK - 1) / TK, n_tiles = (g.N + g.n_tile - 1) / g.n_tile;
    float4 *image = const_cast<float4 *>(g.b_image);
    dim3 pgrid((unsigned)(((long)chunks * 4 * g.n_tile + 255) / 256), n_tiles, 1);
    cudaError_t err;
    if (g.f16) {
        // the scale of B's split comes from its largest magnitude (B is a panel: a pass over it costs microseconds)
        // (unless the caller knows a bound: FP16 is floating point, so a loose bound costs range, not precision)
        unsigned *bmax = const_cast<unsigned *>(g.b_absmax_bits);
        if (!(g.b_scale_fixed > 0.0f)) {
            if ((err = cudaMemsetAsync(bmax, 0, sizeof(unsigned), stream)) != cudaSuccess) return err;
            const int b_rows = b_kmajor ? g.N : g.K, b_cols = b_kmajor ? g.K : g.N;
            absmax_bits_kernel<<<296, 256, 0, stream>>>(g.B, g.ldb, b_rows, b_cols, bmax);
        }
        uint4 *image16 = reinterpret_cast<uint4 *>(image);
        const float lo_scale = g.lo_unscaled ? 1.0f : kSplit16LoScale;
        if (b_kmajor) presplit_b16_kernel<true><<<pgrid, 256, 0, stream>>>(g.B, g.ldb, g.N, g.K, g.n_tile, chunks, image16, bmax, g.b_scale_fixed, lo_scale);
        else presplit_b16_kernel<false><<<pgrid, 256, 0, stream>>>(g.B, g.ldb, g.N, g.K, g.n_tile, chunks, image16, bmax, g.b_scale_fixed, lo_scale);
    } else if (b_kmajor) presplit_b_kernel<true><<<pgrid, 256, 0, stream>>>(g.B, g.ldb, g.N, g.K, g.n_tile, chunks, image);
    else presplit_b_kernel<false><<<pgrid, 256, 0, stream>>>(g.B, g.ldb, g.N, g.K, g.n_tile, chunks, image);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
    if (g.use_tma && g.a_image && g.f16) {
        // the largest |A kscale| for the scale, then the two FP16 matrices
        unsigned *amax = const_cast<unsigned *>(g.a_absmax_bits);
        if ((err = cudaMemsetAsync(amax, 0, sizeof(unsigned), stream)) != cudaSuccess) return err;
        absmax_bits_kernel<<<296, 256, 0, stream>>>(g.A, g.lda, g.M, g.K, amax, g.kscale);
        const long units = (long)g.a_image_rows * (g.K / 8);
        presplit_a16_kernel<<<(unsigned)((units + 255) / 256), 256, 0, stream>>>(g.A, g.lda, g.M, g.K, g.kscale, reinterpret_cast<uint4 *>(g.a_image),
                                                                                  g.a_image_rows, amax, g.lo_unscaled ? 1.0f : kSplit16LoScale);
        if ((err = cudaGetLastError()) != cudaSuccess) return err;
    } else if (g.use_tma && g.a_image) {
        const long quads = (long)g.a_image_rows * (g.K / 4);
        presplit_a_kernel<<<(unsigned)((quads + 255) / 256), 256, 0, stream>>>(g.A, g.lda, g.M, g.K, g.kscale, g.a_image, g.a_image_rows);
        if ((err = cudaGetLastError()) != cudaSuccess) return err;
    }
    if (g.use_tma) return gemm_tc_tma_launch(g, AK, status, stream);
    const size_t smem = tc_image_smem_bytes(g.n_tile, g.a_stages, g.b_stages);
    err = cudaFuncSetAttribute(gemm_tc_image_kernel<AK, NMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    dim3 grid((g.M + TM - 1) / TM, n_tiles, g.splits);
    gemm_tc_image_kernel<AK, NMAX><<<grid, NT2, smem, stream>>>(g, status);
    return cudaGetLastError();
}

}  // namespace

// CTAs of the image kernel that share an SM (tensor memory: 2 x 256 columns up to N = 128; shared memory: the rings)
int gemm_tc_image_ctas_per_sm(int n_tile) {
    int sa, nb;
    tc_image_rings(n_tile, &sa, &nb);
    const size_t smem = tc_image_smem_bytes(n_tile, sa, nb) + 1024;
    const int by_smem = (int)((size_t)228 * 1024 / smem), by_tmem = n_tile <= 128 ? 2 : 1;
    return by_smem < by_tmem ? (by_smem < 1 ? 1 : by_smem) : by_tmem;
}
void gemm_tc_image_rings(int n_tile, int *sa, int *nb) { tc_image_rings(n_tile, sa, nb); }

cudaError_t gemm_absmax_bits(const float *x, long ld, int rows, int cols, unsigned *d_out, cudaStream_t stream) {
    if (cols % 4 != 0 || ld % 4 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0) return cudaErrorInvalidValue;
    cudaError_t err = cudaMemsetAsync(d_out, 0, sizeof(unsigned), stream);
    if (err != cudaSuccess) return err;
    absmax_bits_kernel<<<592, 256, 0, stream>>>(x, ld, rows, cols, d_out);
    return cudaGetLastError();
}

size_t gemm_tc_a_image_bytes(int M, int K) { return (size_t)2 * ((M + TM - 1) / TM * TM) * K * sizeof(float); }

size_t gemm_tc_image_bytes(int N, int n_tile, int K) {
    return (size_t)((N + n_tile - 1) / n_tile) * ((K + TK - 1) / TK) * image_units(n_tile) * 16;
}

bool gemm_tc_eligible(const GemmArgs &g, bool a_kmajor, bool b_kmajor) {
    (void)a_kmajor;
    (void)b_kmajor;
    if (g.N < 16 || g.N % 16 != 0 || g.n_tile < 16 || g.n_tile > 256 || g.n_tile % 16 != 0) return false;
    if ((g.kscale || g.minuend) && g.splits != 1) return false;
    if (g.lda % 4 != 0 || g.ldb % 4 != 0 || g.ldc % 4 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) | reinterpret_cast<uintptr_t>(g.C)) % 16 != 0)
        return false;
    if (g.minuend && (g.ldm % 4 != 0 || reinterpret_cast<uintptr_t>(g.minuend) % 16 != 0)) return false;
    if (g.k_per_split % TK != 0) return false;
    return g.M >= TM && g.K >= 4 * TK;
}

cudaError_t gemm_tc_launch(const GemmArgs &g, bool a_kmajor, bool b_kmajor, unsigned *status, cudaStream_t stream) {
    if (g.b_image) {                                          // B split beforehand, fetched by bulk copies
        if (a_kmajor) return g.n_tile <= 128 ? launch_image<true, 128>(g, b_kmajor, status, stream) : launch_image<true, 256>(g, b_kmajor, status, stream);
        return g.n_tile <= 128 ? launch_image<false, 128>(g, b_kmajor, status, stream) : launch_image<false, 256>(g, b_kmajor, status, stream);
    }
#define BSQ_TC(AK, BK)                                                                  \
    (g.n_tile <= 128 ? launch<AK, BK, 128>(g, status, stream) : launch<AK, BK, 256>(g, status, stream))
    if (a_kmajor && b_kmajor) return BSQ_TC(true, true);
    if (a_kmajor) return BSQ_TC(true, false);
    if (b_kmajor) return BSQ_TC(false, true);
    return BSQ_TC(false, false);
#undef BSQ_TC
}

}  // namespace bsq
