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
//   * two shared-memory stages: the loads and splits of chunk c+1 overlap the MMAs of chunk c;
//     tcgen05.commit on an mbarrier tells when a stage may be overwritten and when the tile is done;
//   * the 128 x N FP32 tile is read back with tcgen05.ld (one accumulator row per thread) and written
//     to C or to the K-split workspace.
// Every mbarrier wait is bounded; on a timeout the CTA records it in the status word, still frees its
// tensor memory and leaves.
#include "bsq_device.cuh"
#include "bsq_gemm.hpp"

namespace bsq {
namespace {

constexpr int TM = 128;          // output rows per CTA (UMMA M)
constexpr int TK = 32;           // K per shared-memory stage (four k-steps of 8)
constexpr int NT = 128;          // threads: one accumulator row each in the epilogue

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

__device__ __forceinline__ float tf32_rna(float x) {
    unsigned r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
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
// and along K every lbo_units(extent) * 16 B (LBO, padded to an odd number of units): with these paddings both
// staging patterns below store without bank conflicts.
__host__ __device__ constexpr unsigned lbo_units(int extent) { return (unsigned)(extent / 8) * 9u + 1u; }
__host__ __device__ constexpr unsigned stage_units(int extent) { return (TK / 4) * lbo_units(extent); }
__device__ __forceinline__ unsigned unit_index(int kc, int r, int extent) {
    return (unsigned)kc * lbo_units(extent) + (unsigned)(r >> 3) * 9u + (unsigned)(r & 7);
}

// One operand chunk: `extent` (MN) x TK (K) starting at (mn0, k0), read from a row-major array in which either K
// (KMAJOR) or MN is the contiguous dimension; consecutive threads read consecutive 16-byte pieces of global
// memory.  A K-contiguous float4 is one unit of the layout; MN-contiguous sources are transposed in registers,
// four float4 of consecutive k giving four units.
template <bool KMAJOR, int MAXU>
struct Stager {
    float4 regs[MAXU];
    __device__ __forceinline__ void load(const float *__restrict__ P, long ld, int mn_total, int k_end, int mn0, int k0,
                                         int extent) {
        const int units = extent * (TK / 4);
        if (KMAJOR) {
#pragma unroll
            for (int i = 0; i < MAXU; ++i) {
                const int f = threadIdx.x + i * NT;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                const int kc = f % (TK / 4), r = f / (TK / 4);
                const int gk = k0 + kc * 4, gr = mn0 + r;
                if (f < units && gr < mn_total && gk < k_end) {
                    const float *src = P + (long)gr * ld + gk;
                    if (gk + 3 < k_end) v = *reinterpret_cast<const float4 *>(src);
                    else { v.x = src[0]; if (gk + 1 < k_end) v.y = src[1]; if (gk + 2 < k_end) v.z = src[2]; }
                }
                regs[i] = v;
            }
        } else {
            const int e4 = extent / 4;
#pragma unroll
            for (int i = 0; i < MAXU / 4; ++i) {
                const int f = threadIdx.x + i * NT;          // item: 4 MN values x 4 k values
                const int mn4 = f % e4, kq = f / e4;
                const int gmn = mn0 + mn4 * 4;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const int gk = k0 + kq * 4 + t;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (f * 4 < units && gk < k_end && gmn < mn_total) {
                        const float *src = P + (long)gk * ld + gmn;
                        if (gmn + 3 < mn_total) v = *reinterpret_cast<const float4 *>(src);
                        else { v.x = src[0]; if (gmn + 1 < mn_total) v.y = src[1]; if (gmn + 2 < mn_total) v.z = src[2]; }
                    }
                    regs[i * 4 + t] = v;
                }
            }
        }
    }
    __device__ __forceinline__ void store(float4 *hi, float4 *lo, int extent) const {
        const int units = extent * (TK / 4);
        if (KMAJOR) {
#pragma unroll
            for (int i = 0; i < MAXU; ++i) {
                const int f = threadIdx.x + i * NT;
                if (f < units) {
                    const unsigned u = unit_index(f % (TK / 4), f / (TK / 4), extent);
                    split_store(regs[i], hi + u, lo + u);
                }
            }
        } else {
            const int e4 = extent / 4;
#pragma unroll
            for (int i = 0; i < MAXU / 4; ++i) {
                const int f = threadIdx.x + i * NT;
                if (f * 4 < units) {
                    const int mn4 = f % e4, kq = f / e4;
                    const float4 v0 = regs[i * 4], v1 = regs[i * 4 + 1], v2 = regs[i * 4 + 2], v3 = regs[i * 4 + 3];
                    const unsigned u = unit_index(kq, mn4 * 4, extent);          // mn4 * 4 .. + 3 stay inside one core matrix
                    split_store(make_float4(v0.x, v1.x, v2.x, v3.x), hi + u, lo + u);
                    split_store(make_float4(v0.y, v1.y, v2.y, v3.y), hi + u + 1, lo + u + 1);
                    split_store(make_float4(v0.z, v1.z, v2.z, v3.z), hi + u + 2, lo + u + 2);
                    split_store(make_float4(v0.w, v1.w, v2.w, v3.w), hi + u + 3, lo + u + 3);
                }
            }
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
    __shared__ __align__(8) uint64_t bar_free[2];
    __shared__ __align__(8) uint64_t bar_done;
    __shared__ unsigned tmem_base_slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int N = g.N;                                        // multiple of 16, <= NMAX
    const int m0 = blockIdx.x * TM;
    const int k_begin = blockIdx.z * g.k_per_split;
    const int k_end = min(g.K, k_begin + g.k_per_split);
    const unsigned a_units = stage_units(TM), b_units = stage_units(N);
    // stage s: [A hi | A lo | B hi | B lo]
    const unsigned stage_bytes = (2 * a_units + 2 * b_units) * 16u;
    // two accumulators: the hi*hi chain and, half the allocation further on, the two small cross terms
    const unsigned acc_cols = N <= 16 ? 16u : (N <= 32 ? 32u : (N <= 64 ? 64u : (N <= 128 ? 128u : 256u)));
    const unsigned tmem_cols = 2u * acc_cols;

    if (tid == 0) {
        mbar_init(&bar_free[0], 1);
        mbar_init(&bar_free[1], 1);
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

    // instruction descriptor: FP32 accumulate, TF32 x TF32, majors, N >> 3, M >> 4
    // (both operands are K-major in shared memory whatever their orientation in global memory)
    const unsigned idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(TM >> 4) << 24);

    Stager<A_KMAJOR, TM * (TK / 4) / NT> sa;
    Stager<B_KMAJOR, NMAX * (TK / 4) / NT> sb;
    const int chunks = (k_end - k_begin + TK - 1) / TK;
    bool ok = true;
    unsigned free_phase = 0;                                  // bit s: parity of the next wait on bar_free[s]
    if (chunks > 0) {
        sa.load(g.A, g.lda, g.M, k_end, m0, k_begin, TM);
        sb.load(g.B, g.ldb, N, k_end, 0, k_begin, N);
    }
    for (int c = 0; c < chunks && ok; ++c) {
        const int s = c & 1;
        bool mine = true;
        if (c >= 2) {                                         // the MMAs of chunk c-2 must be done with stage s
            mine = mbar_wait_bounded(&bar_free[s], (free_phase >> s) & 1u, status);
            free_phase ^= 1u << s;
        }
        float4 *a_hi = reinterpret_cast<float4 *>(smem_raw + (size_t)s * stage_bytes), *a_lo = a_hi + a_units, *b_hi = a_lo + a_units, *b_lo = b_hi + b_units;
        sa.store(a_hi, a_lo, TM);
        sb.store(b_hi, b_lo, N);
        fence_proxy_async_smem();                             // generic-proxy stores -> tensor-core (async proxy) reads
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        ok = __syncthreads_and(mine) != 0;                    // uniform: after a timeout nobody issues or loops on
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
        if (c + 1 < chunks) {                                 // next chunk's loads overlap the MMAs
            sa.load(g.A, g.lda, g.M, k_end, m0, k_begin + (c + 1) * TK, TM);
            sb.load(g.B, g.ldb, N, k_end, 0, k_begin + (c + 1) * TK, N);
        }
    }
    // epilogue: thread t of warp w owns accumulator row 32 w + t
    if (chunks > 0 && ok) ok = mbar_wait_bounded(&bar_done, 0, status);
    ok = __syncthreads_and(ok) != 0;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float *C = g.C + (long)blockIdx.z * g.split_stride;
    const int row = m0 + tid;
    if (ok) {
        for (int c0 = 0; c0 < N; c0 += 16) {
            unsigned r[16], q[16];
            if (chunks > 0) {
                const unsigned taddr = tmem_d + ((unsigned)(warp * 32) << 16) + (unsigned)c0;
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
                float4 *dst = reinterpret_cast<float4 *>(C + (long)row * g.ldc + c0);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                         __uint_as_float(r[4 * j + 3]));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
    }
}

template <int NMAX>
size_t tc_smem_bytes(bool a_kmajor, bool b_kmajor, int N) {
    (void)a_kmajor;
    (void)b_kmajor;
    return (size_t)2 * (2 * stage_units(TM) + 2 * stage_units(N)) * 16;
}

template <bool AK, bool BK, int NMAX>
cudaError_t launch(const GemmArgs &g, unsigned *status, cudaStream_t stream) {
    const size_t smem = tc_smem_bytes<NMAX>(AK, BK, g.N);
    cudaError_t err = cudaFuncSetAttribute(gemm_tc_kernel<AK, BK, NMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    dim3 grid((g.M + TM - 1) / TM, 1, g.splits);
    gemm_tc_kernel<AK, BK, NMAX><<<grid, NT, smem, stream>>>(g, status);
    return cudaGetLastError();
}

}  // namespace

bool gemm_tc_eligible(const GemmArgs &g, bool a_kmajor, bool b_kmajor) {
    (void)a_kmajor;
    (void)b_kmajor;
    if (g.N < 16 || g.N > 256 || g.N % 16 != 0) return false;
    if (g.kscale || g.minuend) return false;
    if (g.lda % 4 != 0 || g.ldb % 4 != 0 || g.ldc % 4 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) | reinterpret_cast<uintptr_t>(g.C)) % 16 != 0)
        return false;
    if (g.k_per_split % TK != 0) return false;
    return g.M >= TM && g.K >= 4 * TK;
}

cudaError_t gemm_tc_launch(const GemmArgs &g, bool a_kmajor, bool b_kmajor, unsigned *status, cudaStream_t stream) {
#define BSQ_TC(AK, BK)                                                                  \
    (g.N <= 128 ? launch<AK, BK, 128>(g, status, stream) : launch<AK, BK, 256>(g, status, stream))
    if (a_kmajor && b_kmajor) return BSQ_TC(true, true);
    if (a_kmajor) return BSQ_TC(true, false);
    if (b_kmajor) return BSQ_TC(false, true);
    return BSQ_TC(false, false);
#undef BSQ_TC
}

}  // namespace bsq
