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

namespace bsq {
namespace {

constexpr int TM = 128;          // output rows per CTA (UMMA M)
constexpr int TK = 16;           // K per shared-memory stage (two k-steps of 8)
constexpr int NT = 256;          // threads: all stage operands, one issues the MMAs, two per accumulator row in the epilogue
constexpr int DEPTH = 3;         // chunks of K in flight in registers per thread
constexpr int STAGES = 2;        // operand stages in shared memory (three measured slower: less L1 left for the loads)

__device__ __forceinline__ uint64_t smem_desc(unsigned addr_bytes, unsigned lbo_bytes, unsigned sbo_bytes) {
    // start address, leading / stride byte offsets in 16-byte units; version 1 (bits 46-47); no swizzle
    return (uint64_t)((addr_bytes >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

__device__ __forceinline__ void mma_tf32(unsigned tmem_d, uint64_t desc_a, uint64_t desc_b, unsigned idesc, bool accumulate) {
    const unsigned acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// 16 consecutive accumulator columns of this thread's row (lane) of tensor memory
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// Round to TF32 (10 mantissa bits), ties away from zero, by integer arithmetic on the bit pattern: two full-rate
// instructions (add half of the last kept place, clear the 13 low bits; a carry out of the mantissa bumps the exponent
// as it should).  Same result as cvt.rna.tf32.f32 for every finite value.
__device__ __forceinline__ float tf32_rna(float x) {
    return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
}

// x = hi + lo + e with hi, lo exactly representable in TF32 and |e| <= 2^-22 |x|
__device__ __forceinline__ void split_store(float4 v, float4 *hi, float4 *lo) {
    const float4 h = make_float4(tf32_rna(v.x), tf32_rna(v.y), tf32_rna(v.z), tf32_rna(v.w));
    *hi = h;
    *lo = make_float4(tf32_rna(__fsub_rn(v.x, h.x)), tf32_rna(__fsub_rn(v.y, h.y)), tf32_rna(__fsub_rn(v.z, h.z)),
                      tf32_rna(__fsub_rn(v.w, h.w)));
}

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
    // epilogue: accumulator row 32 (w % 4) + lane; warps 0-3 take the lower half of the columns, warps 4-7 the upper
    if (chunks > 0 && ok) ok = mbar_wait_bounded(&bar_done, 0, status);
    ok = __syncthreads_and(ok) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float *C = g.C + (long)blockIdx.z * g.split_stride;
    const int row = m0 + (warp & 3) * 32 + (tid & 31);
    const int half = (N / 16 + 1) / 2 * 16;                  // columns of the lower half, a multiple of 16
    const int c_begin = warp < 4 ? 0 : half, c_end = warp < 4 ? half : N;
    bool any = false;
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

}  // namespace

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
#define BSQ_TC(AK, BK)                                                                  \
    (g.n_tile <= 128 ? launch<AK, BK, 128>(g, status, stream) : launch<AK, BK, 256>(g, status, stream))
    if (a_kmajor && b_kmajor) return BSQ_TC(true, true);
    if (a_kmajor) return BSQ_TC(true, false);
    if (b_kmajor) return BSQ_TC(false, true);
    return BSQ_TC(false, false);
#undef BSQ_TC
}

}  // namespace bsq
