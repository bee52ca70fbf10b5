// Tensor-core product with the streamed operand fed by TMA (sm_100a): C[M x N] = A * opB for a row-major A that is
// contiguous along K (the orientation of the caller's matrix in half of the range finder's products, of U in the
// reconstruction and of the tall panels in the orthonormalisation), N <= 256 columns per tile, 3xTF32 like the other
// tensor-core kernels (bsq_gemm_tc.cu), which this one replaces for that orientation wherever the second operand has
// been split into images beforehand.  It replaces the same cublasSgemm calls of the reference
// (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:293-386, modules/reconstruct_lowrank_cuda/src/
// reconstruct_lowrank_cuda.cu:46-61).
//
// What is different from the register-staged kernels: nothing of A passes through registers on its way in.
//   * A producer thread brings A in 128-row x 32-float boxes with tiled TMA copies (cp.async.bulk.tensor.2d, one
//     tensor map per launch over the caller's matrix, 128-byte swizzle, rows and columns past the matrix zero-filled
//     by the copy engine) into a ring of slots, several boxes ahead of the tensor core: HBM latency is hidden by the
//     ring's depth instead of by loads held in registers.
//   * The box arrives in exactly the layout the tensor core reads (K-major, 128-byte swizzle), so the TF32 split is an
//     element-wise pass over shared memory that knows nothing about layouts: four warps read a slot 16 bytes at a
//     time, write hi = tf32(x) back in place and lo = tf32(x - hi) at the same offset of the slot's second half.
//     About a tenth of the instructions the register-staged kernels spend per element, no transposes, no bank
//     conflicts, no CTA-wide barrier.
//   * A second producer thread fetches the images of B (hi | lo per 16 of K, made once per product by
//     presplit_b_kernel) with plain bulk copies into a ring of their own; one thread issues the MMAs (per 8 of K:
//     hi*hi into one accumulator in tensor memory, lo*hi and hi*lo into a second), tcgen05.commit hands slots and
//     images back to the producers; four epilogue warps read the accumulators back and write C.
//   * A wide product (the reconstruction: hundreds of tiles, each with a short K) runs as a persistent grid, one CTA
//     per SM walking over its tiles with two accumulator sets in tensor memory: the MMAs of the next tile overlap the
//     write-out of the last one, and rings, barriers and tensor memory are set up once per SM instead of once per tile.
// Roles meet only through mbarriers; every wait is bounded (status word, tensor memory freed, copies in flight
// waited for before the CTA leaves).  No multicast, no cluster: the tensor map covers this GPU's own memory only.
#include "bsq_device.cuh"
#include "bsq_gemm.hpp"
#include "bsq_gemm_tc.cuh"

#include <cuda.h>

#include <cstdlib>
#include <mutex>

namespace bsq {
namespace {

constexpr int KS = 32;                          // K per slot of A: one 128-byte swizzle row
constexpr unsigned A_HALF = TM * KS * 4;        // bytes of one image of a slot (hi, in place over the box; lo behind it)
constexpr unsigned A_SLOT = 2 * A_HALF;
constexpr int NTH = 11 * 32;                    // warp 0: A producer, 1: MMA issuer, 2: B producer, 3-6: transform, 7-10: epilogue
constexpr int XF = 128;                         // transform threads; as many epilogue threads
constexpr int MAXR = 8;                         // most slots of A / images of B in their rings

// K-major operand in 128-byte-swizzled shared memory: rows of 128 B, groups of 8 rows 1024 B apart (stride byte
// offset), leading byte offset unused, descriptor version 1, layout type 2 (128-byte swizzle).  Steps of 8 along K
// inside the 128-byte row are steps of 32 B of the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(unsigned addr_bytes) {
    return (uint64_t)((addr_bytes >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Position in a ring of `n` stages and the parity of its current round.  Every role walks its rings with one of these:
// a division and a remainder by the (run-time) ring length per stage were most of what the single threads that issue
// the copies and the MMAs executed per stage.
struct Ring {
    int pos = 0, n;
    unsigned par = 0;            // parity of the round `pos` is in
    bool wrapped = false;        // the ring has been around at least once: the stage at `pos` has a previous use
    __device__ __forceinline__ explicit Ring(int stages) : n(stages) {}
    __device__ __forceinline__ void next() {
        if (++pos == n) { pos = 0; par ^= 1u; wrapped = true; }
    }
};
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

constexpr unsigned RAW_BOX = 32 * 32 * 4;       // A contiguous along M: one box of 32 k x 32 rows, four per slot
constexpr unsigned RAW_SLOT = 4 * RAW_BOX;

struct TmaBars {
    uint64_t full_a[MAXR], ready_a[MAXR], empty_a[MAXR], full_b[MAXR], empty_b[MAXR];
    uint64_t raw_full[MAXR], raw_empty[MAXR];   // A contiguous along M: boxes as they come from memory, before the transposing split
    uint64_t acc_full[2], acc_empty[2];         // accumulator set of a tile: written completely / read out completely
    unsigned tmem_base, failed;
};

// The tiles of one CTA.  Skinny products: one tile, given by the block index (grid = row tiles x column tiles x K
// slices).  Wide products (g.persistent: the reconstruction, hundreds of tiles with a short K): tile numbers
// blockIdx.x, + gridDim.x, ..., row tile fastest; the rings and the roles just keep going from one tile to the next,
// and with two accumulator sets in tensor memory (tiles of at most 128 columns) the tensor core works on the next
// tile while the epilogue warps still write the last one out.
struct TileWalk {
    int first, step, count, m_tiles;
    bool persistent;
    __device__ __forceinline__ TileWalk(const GemmArgs &g) {
        persistent = g.persistent;
        m_tiles = (g.M + TM - 1) / TM;
        if (persistent) {
            const int n_tiles = (g.N + g.n_tile - 1) / g.n_tile;
            first = blockIdx.x;
            step = gridDim.x;
            count = (m_tiles * n_tiles - first + step - 1) / step;
        } else {
            first = 0; step = 1; count = 1;
        }
    }
    __device__ __forceinline__ void at(int i, int *m_tile, int *n_tile, int *z) const {
        if (persistent) {
            const int t = first + i * step;
            *m_tile = t % m_tiles;
            *n_tile = t / m_tiles;
            *z = 0;
        } else {
            *m_tile = blockIdx.x; *n_tile = blockIdx.y; *z = blockIdx.z;
        }
    }
};

// A_KMAJOR = false: the caller's matrix is contiguous along M (the product W^T X read from W's storage).  Its boxes (32 k
// x 32 rows, 128-byte swizzle, four per slot) land in a ring of their own; the transform warps transpose while they split:
// thread m gathers the four k of a unit from four rows of the box (a warp reads 32 neighbouring floats of one k: no
// bank conflict, the swizzle only permutes 16-byte pieces) and writes hi and lo into row m of an operand stage in the
// same K-major swizzled layout as above.  The raw box is handed back to the producer as soon as it has been read.
// F16 = true: the operands are split into two FP16 halves instead of two TF32 halves (see split16 in bsq_gemm_tc.cuh):
// all layouts keep their BYTES (a 128-byte operand row now holds 64 of K, an image of B 32 of K), so descriptors, rings
// and the MMA issue loop are the same; the caller's FP32 boxes go through the raw ring in both orientations, because
// the 16-bit images cannot be made in place.
template <bool A_KMAJOR, int NMAX, bool F16 = false>
__global__ void __launch_bounds__(NTH, 1) gemm_tc_tma_kernel(const __grid_constant__ CUtensorMap tmap_a, GemmArgs g, unsigned *status) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char *base = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);      // the swizzle wants 1024-byte aligned slots
    constexpr int KS = F16 ? 64 : bsq::KS;                 // K per slot of A
    constexpr int TK = F16 ? 32 : bsq::TK;                 // K per image of B
    constexpr bool USES_RAW = !A_KMAJOR || F16;
    constexpr unsigned RAW_SLOT = F16 ? 2u * bsq::RAW_SLOT : bsq::RAW_SLOT;
    const int NR = g.a_stages, NB = g.b_stages, NRAW = (USES_RAW && g.a_image == nullptr) ? g.raw_stages : 0;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool a_img = A_KMAJOR && g.a_image != nullptr;           // A split beforehand: both halves of a slot come in by TMA
    const unsigned b_stride = 2u * image_half_units(g.n_tile) * 16u;
    unsigned char *raw_slots = base;
    unsigned char *a_slots = raw_slots + (size_t)NRAW * RAW_SLOT;
    unsigned char *b_slots = a_slots + (size_t)NR * A_SLOT;
    TmaBars &bars = *reinterpret_cast<TmaBars *>(b_slots + (size_t)NB * b_stride);
    // accumulator columns of one set (hi*hi chain and, acc_cols further on, the cross terms), and how many sets
    const unsigned acc_cols = g.n_tile <= 16 ? 16u : (g.n_tile <= 32 ? 32u : (g.n_tile <= 64 ? 64u : (g.n_tile <= 128 ? 128u : 256u)));
    const bool one_acc = a_img && g.wide_tiles;                    // the cross terms go into the hi * hi accumulator
    const unsigned acc_stride = one_acc ? acc_cols : 2u * acc_cols;  // tensor-memory columns of one set
    const int acc_sets = (g.persistent && acc_stride <= 256u) ? 2 : 1;
    const unsigned tmem_cols = acc_stride * (unsigned)acc_sets;
    const int epi_groups = one_acc ? 2 : 1;                        // wide tiles: the transform warps take the tile's second 128 columns
    const TileWalk walk(g);
    const int chunks_total = (g.K + TK - 1) / TK;

    if (tid == 0) {
        for (int i = 0; i < NR; ++i) {
            mbar_init(&bars.full_a[i], 1);
            mbar_init(&bars.ready_a[i], XF);
            mbar_init(&bars.empty_a[i], 1);
        }
        for (int i = 0; i < NB; ++i) {
            mbar_init(&bars.full_b[i], 1);
            mbar_init(&bars.empty_b[i], 1);
        }
        for (int i = 0; i < NRAW; ++i) {
            mbar_init(&bars.raw_full[i], 1);
            mbar_init(&bars.raw_empty[i], XF);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars.acc_full[i], 1);
            mbar_init(&bars.acc_empty[i], XF * epi_groups);
        }
        bars.failed = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars.tmem_base)), "r"(tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = bars.tmem_base;
    bool ok = true;

    if (warp == 0) {
        // ---- A producer: one box per slot, as far ahead as the ring allows ----
        if (lane == 0) {
            int ca = 0;                                                  // slots filled so far, over all tiles
            Ring ra((USES_RAW && !a_img) ? NRAW : NR);
            for (int i = 0; i < walk.count && ok; ++i) {
                int mt, nt, z;
                walk.at(i, &mt, &nt, &z);
                const int k_begin = z * g.k_per_split, k_end = min(g.K, k_begin + g.k_per_split);
                const int chunks_a = (k_end - k_begin + KS - 1) / KS;
                for (int c = 0; c < chunks_a; ++c, ++ca, ra.next()) {
                    const int s = ra.pos;
                    if (A_KMAJOR && F16 && !a_img) {
                        // two boxes of 32 k x 128 rows, as they are in the caller's matrix; the transform warps make the
                        // slot's two FP16 images from them
                        if (ra.wrapped) ok = mbar_wait_bounded(&bars.raw_empty[s], ra.par ^ 1u, status);
                        if (!ok) break;
                        mbar_expect_tx(&bars.raw_full[s], RAW_SLOT);
                        tma_load_2d(raw_slots + (size_t)s * RAW_SLOT, &tmap_a, k_begin + c * KS, mt * TM, &bars.raw_full[s]);
                        tma_load_2d(raw_slots + (size_t)s * RAW_SLOT + RAW_SLOT / 2, &tmap_a, k_begin + c * KS + 32, mt * TM, &bars.raw_full[s]);
                    } else if (A_KMAJOR) {
                        if (ra.wrapped) ok = mbar_wait_bounded(&bars.empty_a[s], ra.par ^ 1u, status);
                        if (!ok) break;
                        if (a_img) {                                     // hi and lo of the slot, split beforehand
                            mbar_expect_tx(&bars.full_a[s], A_SLOT);
                            tma_load_2d(a_slots + (size_t)s * A_SLOT, &tmap_a, k_begin + c * KS, mt * TM, &bars.full_a[s]);
                            tma_load_2d(a_slots + (size_t)s * A_SLOT + A_HALF, &tmap_a, k_begin + c * KS, g.a_image_rows + mt * TM, &bars.full_a[s]);
                        } else {
                            mbar_expect_tx(&bars.full_a[s], A_HALF);
                            tma_load_2d(a_slots + (size_t)s * A_SLOT, &tmap_a, k_begin + c * KS, mt * TM, &bars.full_a[s]);
                        }
                    } else {
                        if (ra.wrapped) ok = mbar_wait_bounded(&bars.raw_empty[s], ra.par ^ 1u, status);
                        if (!ok) break;
                        mbar_expect_tx(&bars.raw_full[s], RAW_SLOT);
#pragma unroll
                        for (int kg = 0; kg < (F16 ? 2 : 1); ++kg)       // (F16: a slot is 64 of k, two boxes deep)
#pragma unroll
                            for (int b = 0; b < 4; ++b)       // inner coordinate: the row (contiguous), outer: k
                                tma_load_2d(raw_slots + (size_t)s * RAW_SLOT + (kg * 4 + b) * RAW_BOX, &tmap_a, mt * TM + 32 * b,
                                            k_begin + c * KS + 32 * kg, &bars.raw_full[s]);
                    }
                }
            }
            if (!ok) {
                // leaving early: boxes still in flight must have landed before this CTA's shared memory goes away
                atomicOr(&bars.failed, 1u);
                if (!USES_RAW || a_img)
                    for (int c = max(0, ca - NR); c < ca; ++c) mbar_wait_bounded(&bars.full_a[c % NR], (unsigned)(c / NR) & 1u, status);
                else
                    for (int c = max(0, ca - NRAW); c < ca; ++c) mbar_wait_bounded(&bars.raw_full[c % NRAW], (unsigned)(c / NRAW) & 1u, status);
            }
        }
    } else if (warp == 2) {
        // ---- B producer: the images of the tile's columns, one bulk copy each ----
        if (lane == 0) {
            int jb = 0;
            Ring rb(NB);
            for (int i = 0; i < walk.count && ok; ++i) {
                int mt, nt, z;
                walk.at(i, &mt, &nt, &z);
                const int k_begin = z * g.k_per_split, k_end = min(g.K, k_begin + g.k_per_split);
                const int chunks_b = (k_end - k_begin + TK - 1) / TK;
                const int N = min(g.n_tile, g.N - nt * g.n_tile);
                const unsigned b_bytes = 2u * image_half_units(N) * 16u;
                const float4 *image = g.b_image + ((size_t)nt * chunks_total + k_begin / TK) * image_units(g.n_tile);
                for (int j = 0; j < chunks_b; ++j, ++jb, rb.next()) {
                    const int sb = rb.pos;
                    if (rb.wrapped) ok = mbar_wait_bounded(&bars.empty_b[sb], rb.par ^ 1u, status);
                    if (!ok) break;
                    mbar_expect_tx(&bars.full_b[sb], b_bytes);
                    bulk_g2s(b_slots + (size_t)sb * b_stride, image + (size_t)j * image_units(g.n_tile), b_bytes, &bars.full_b[sb]);
                }
            }
            if (!ok) {
                atomicOr(&bars.failed, 1u);
                for (int j = max(0, jb - NB); j < jb; ++j) mbar_wait_bounded(&bars.full_b[j % NB], (unsigned)(j / NB) & 1u, status);
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer ----
        if (lane == 0) {
            Ring ra(NR), rb(NB), rs(acc_sets);
            for (int i = 0; i < walk.count && ok; ++i, rs.next()) {
                int mt, nt, z;
                walk.at(i, &mt, &nt, &z);
                const int k_begin = z * g.k_per_split, k_end = min(g.K, k_begin + g.k_per_split);
                const int chunks_a = (k_end - k_begin + KS - 1) / KS, chunks_b = (k_end - k_begin + TK - 1) / TK;
                const int N = min(g.n_tile, g.N - nt * g.n_tile);
                const unsigned b_units = image_half_units(N);
                // FP32 accumulate, TF32 x TF32, both operands K-major, N >> 3, M >> 4
                // (F16: A and B formats 0 = FP16 instead of 2 = TF32, and the instruction is kind::f16, 16 of K each)
                const unsigned idesc = (1u << 4) | ((F16 ? 0u : 2u) << 7) | ((F16 ? 0u : 2u) << 10) | ((unsigned)(N >> 3) << 17) | ((unsigned)(TM >> 4) << 24);
                const unsigned b_kstep = 2u * (unsigned)N;              // units from one 8-wide k-step of an image to the next
                const int set = rs.pos;
                const unsigned acc = tmem_d + (unsigned)set * acc_stride, acc_x = one_acc ? acc : acc + acc_cols;
                // the epilogue must have read this accumulator set's previous tile out
                if (rs.wrapped) ok = mbar_wait_bounded(&bars.acc_empty[set], rs.par ^ 1u, status);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int c = 0; c < chunks_a && ok; ++c, ra.next()) {
                    const int s = ra.pos;
                    ok = mbar_wait_bounded(a_img ? &bars.full_a[s] : &bars.ready_a[s], ra.par, status);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_addr = smem_u32(a_slots + (size_t)s * A_SLOT);
                    const uint64_t da_hi = smem_desc_sw128(a_addr), da_lo = smem_desc_sw128(a_addr + A_HALF);
                    for (int h = 0; h < 2 && ok; ++h) {
                        if (2 * c + h >= chunks_b) break;                // K ends inside this slot: its second half is zeros
                        const int sb = rb.pos;
                        ok = mbar_wait_bounded(&bars.full_b[sb], rb.par, status);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint64_t db0 = smem_desc(smem_u32(b_slots + (size_t)sb * b_stride), (unsigned)N * 16u, 128u);
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) {                 // two k-steps of 32 bytes of K per image
                            const int kk = 2 * h + ks;                   // k-step of 8 inside the slot's 32
                            const uint64_t dah = da_hi + (uint64_t)(kk * 2), dal = da_lo + (uint64_t)(kk * 2);
                            const uint64_t dbh = db0 + (uint64_t)(ks * b_kstep), dbl = dbh + b_units;
                            if (F16) {
                                mma_f16(acc, dah, dbh, idesc, c > 0 || kk > 0);
                                mma_f16(acc_x, dal, dbh, idesc, one_acc || c > 0 || kk > 0);
                                mma_f16(acc_x, dah, dbl, idesc, true);
                            } else {
                                mma_tf32(acc, dah, dbh, idesc, c > 0 || kk > 0);
                                mma_tf32(acc_x, dal, dbh, idesc, one_acc || c > 0 || kk > 0);
                                mma_tf32(acc_x, dah, dbl, idesc, true);
                            }
                        }
                        tc_commit(&bars.empty_b[sb]);
                        rb.next();
                    }
                    if (ok) tc_commit(&bars.empty_a[s]);
                }
                if (ok) tc_commit(&bars.acc_full[set]);
            }
            if (!ok) atomicOr(&bars.failed, 1u);
        }
    } else if (warp < 7 && !one_acc) {
        // ---- transform: hi in place, lo behind it (nothing to do when A was split beforehand) ----
        const int t = tid - 3 * 32;
        Ring ra(NR), rr(USES_RAW ? NRAW : 1);
        const float sa16 = F16 ? split16_scale(*g.a_absmax_bits) : 1.0f;
        for (int i = 0; i < (a_img ? 0 : walk.count) && ok; ++i) {
            int mt, nt, z;
            walk.at(i, &mt, &nt, &z);
            const int k_begin = z * g.k_per_split, k_end = min(g.K, k_begin + g.k_per_split);
            const int chunks_a = (k_end - k_begin + KS - 1) / KS;
            for (int c = 0; c < chunks_a; ++c, ra.next(), rr.next()) {
                const int s = ra.pos;
                float4 *hi = reinterpret_cast<float4 *>(a_slots + (size_t)s * A_SLOT);
                float4 *lo = hi + A_HALF / 16;
                if (A_KMAJOR && F16) {
                    const int sr = rr.pos;
                    ok = mbar_wait_bounded(&bars.raw_full[sr], rr.par, status);
                    if (ok && ra.wrapped) ok = mbar_wait_bounded(&bars.empty_a[s], ra.par ^ 1u, status);
                    if (!ok) break;
                    // thread t owns row t: its 64 k are 8 units of 4 k in each of the slot's two boxes (unit u of row t
                    // sits at position u ^ (t & 7)); they become 8 units of 8 FP16 k in the hi and in the lo image
                    const float4 *box0 = reinterpret_cast<const float4 *>(raw_slots + (size_t)sr * RAW_SLOT), *box1 = box0 + RAW_SLOT / 32;
                    float4 w[16];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        w[u] = box0[t * 8 + (u ^ (t & 7))];
                        w[8 + u] = box1[t * 8 + (u ^ (t & 7))];
                    }
                    mbar_arrive(&bars.raw_empty[sr]);
                    uint4 *hi16 = reinterpret_cast<uint4 *>(hi), *lo16 = reinterpret_cast<uint4 *>(lo);
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        const int at = t * 8 + (c8 ^ (t & 7));
                        split16_store8(w[2 * c8], w[2 * c8 + 1], sa16, hi16 + at, lo16 + at);
                    }
                    fence_proxy_async_smem();
                    mbar_arrive(&bars.ready_a[s]);
                    continue;
                }
                if (!A_KMAJOR) {
                    const int sr = rr.pos;
                    ok = mbar_wait_bounded(&bars.raw_full[sr], rr.par, status);
                    // the MMAs that read this operand stage NR slots ago must be done with it
                    if (ok && ra.wrapped) ok = mbar_wait_bounded(&bars.empty_a[s], ra.par ^ 1u, status);
                    if (!ok) break;
                    if (F16) {
                        // thread t owns row t of the slot: float t % 32 of every k in boxes t / 32 (k 0..31) and 4 + t / 32
                        float4 w[16];
#pragma unroll
                        for (int kg = 0; kg < 2; ++kg) {
                            const float *bx = reinterpret_cast<const float *>(raw_slots + (size_t)sr * RAW_SLOT + (kg * 4 + (t >> 5)) * RAW_BOX);
                            const int mm = t & 31;
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                float e[4];
#pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    const int kk = 4 * q + u;
                                    e[u] = bx[kk * 32 + ((((mm >> 2) ^ (kk & 7)) << 2) | (mm & 3))];
                                }
                                w[kg * 8 + q] = make_float4(e[0], e[1], e[2], e[3]);
                            }
                        }
                        mbar_arrive(&bars.raw_empty[sr]);
                        uint4 *hi16 = reinterpret_cast<uint4 *>(hi), *lo16 = reinterpret_cast<uint4 *>(lo);
#pragma unroll
                        for (int c8 = 0; c8 < 8; ++c8) {
                            const int at = t * 8 + (c8 ^ (t & 7));
                            split16_store8(w[2 * c8], w[2 * c8 + 1], sa16, hi16 + at, lo16 + at);
                        }
                        fence_proxy_async_smem();
                        mbar_arrive(&bars.ready_a[s]);
                        continue;
                    }
                    // thread t owns row t of the slot: box t / 32, float t % 32 of every k
                    const float *box = reinterpret_cast<const float *>(raw_slots + (size_t)sr * RAW_SLOT + (t >> 5) * RAW_BOX);
                    const int mm = t & 31, k0 = k_begin + c * KS;
                    float4 w[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float e[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int kk = 4 * q + u;
                            e[u] = box[kk * 32 + ((((mm >> 2) ^ (kk & 7)) << 2) | (mm & 3))];
                            if (g.kscale) e[u] *= (k0 + kk < k_end ? g.kscale[k0 + kk] : 0.f);
                        }
                        w[q] = make_float4(e[0], e[1], e[2], e[3]);
                    }
                    mbar_arrive(&bars.raw_empty[sr]);                    // (shared-memory reads above are complete: their values are in registers)
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        const int at = t * 8 + (q ^ (t & 7));            // unit q of row t sits at position q ^ (t & 7)
                        split_store(w[q], hi + at, lo + at);
                    }
                    fence_proxy_async_smem();
                    mbar_arrive(&bars.ready_a[s]);
                    continue;
                }
                ok = mbar_wait_bounded(&bars.full_a[s], ra.par, status);
                if (!ok) break;
                float4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = hi[t + XF * j];
                if (g.kscale) {
                    // opA(i, kk) *= kscale[kk]: unit u of row r holds the 4 k of logical unit u ^ (r & 7).  A thread's
                    // eight units (e = t + 128 j: row (t >> 3) + 16 j, position t & 7) are the same logical unit of
                    // eight rows, so the four factors are fetched once per slot.
                    const int kk = k_begin + c * KS + (((t & 7) ^ ((t >> 3) & 7)) << 2);
                    const float f0 = kk < k_end ? g.kscale[kk] : 0.f, f1 = kk + 1 < k_end ? g.kscale[kk + 1] : 0.f;
                    const float f2 = kk + 2 < k_end ? g.kscale[kk + 2] : 0.f, f3 = kk + 3 < k_end ? g.kscale[kk + 3] : 0.f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) { v[j].x *= f0; v[j].y *= f1; v[j].z *= f2; v[j].w *= f3; }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) split_store(v[j], hi + t + XF * j, lo + t + XF * j);
                fence_proxy_async_smem();                                // generic-proxy stores -> tensor-core (async proxy) reads
                mbar_arrive(&bars.ready_a[s]);
            }
        }
        if (!ok) atomicOr(&bars.failed, 1u);
    } else {
        // ---- epilogue: this thread's accumulator row of every tile, 16 columns at a time ----
        const int quarter = warp & 3;                                    // the tensor-memory lanes this warp may read
        const int cb = (one_acc && warp < 7) ? 128 : 0;                  // wide tiles: first column of this warp's half of the tile
        const float inv16 = F16 ? 1.0f / (split16_scale(*g.a_absmax_bits) * (g.b_scale_fixed > 0.0f ? g.b_scale_fixed : split16_scale(*g.b_absmax_bits))) : 1.0f;
        // 32-byte accesses need 32-byte aligned rows of C and of the minuend (tile columns start at multiples of 16)
        const bool wide32 = ((reinterpret_cast<uintptr_t>(g.C) | (uintptr_t)(g.ldc * 4) | (uintptr_t)(g.split_stride * 4)) % 32 == 0) &&
                            (!g.minuend || (reinterpret_cast<uintptr_t>(g.minuend) | (uintptr_t)(g.ldm * 4)) % 32 == 0);
        bool any = false;
        Ring rs(acc_sets);
        for (int i = 0; i < walk.count && ok; ++i, rs.next()) {
            int mt, nt, z;
            walk.at(i, &mt, &nt, &z);
            const int n0 = nt * g.n_tile, N = min(g.n_tile, g.N - n0);
            const int row = mt * TM + quarter * 32 + lane;
            const int set = rs.pos;
            float *C = g.C + (long)z * g.split_stride;
            // A full 128-column tile with a minuend: the thread's whole row segment of the minuend is asked for before
            // the wait for the accumulators, so that its HBM latency passes while the tensor core still works on the
            // tile (fetched 16 columns at a time inside the loop below, every step would wait for memory on its own).
            const int ce = one_acc ? min(N, cb + 128) : N;                // this thread's columns of the tile: cb .. ce - 1
            const bool pre = g.minuend != nullptr && ce - cb == 128 && row < g.M;
            float4 mn_pre[32];
            if (pre) {
                const float *mn = g.minuend + (long)row * g.ldm + n0 + cb;
                if (wide32) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) ld_global_v8(mn + 8 * j, mn_pre[2 * j], mn_pre[2 * j + 1]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) mn_pre[j] = reinterpret_cast<const float4 *>(mn)[j];
                }
            }
            ok = mbar_wait_bounded(&bars.acc_full[set], rs.par, status);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (pre) {
                float4 *dst = reinterpret_cast<float4 *>(C + (long)row * g.ldc + n0 + cb);
#pragma unroll
                for (int s16 = 0; s16 < 8; ++s16) {
                    unsigned r[16], q[16];
                    const unsigned taddr = tmem_d + (unsigned)set * acc_stride + ((unsigned)(quarter * 32) << 16) + (unsigned)(cb + s16 * 16);
                    tmem_ld16(taddr, r);
                    if (!one_acc) tmem_ld16(taddr + acc_cols, q);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (one_acc) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) q[j] = 0x80000000u;    // (-0.0f: the sum below leaves r as it is, bit for bit)
                    }
                    float4 o4[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 m4 = mn_pre[s16 * 4 + j];
                        float p0 = __fadd_rn(__uint_as_float(r[4 * j]), __uint_as_float(q[4 * j]));
                        float p1 = __fadd_rn(__uint_as_float(r[4 * j + 1]), __uint_as_float(q[4 * j + 1]));
                        float p2 = __fadd_rn(__uint_as_float(r[4 * j + 2]), __uint_as_float(q[4 * j + 2]));
                        float p3 = __fadd_rn(__uint_as_float(r[4 * j + 3]), __uint_as_float(q[4 * j + 3]));
                        if (F16) { p0 = __fmul_rn(p0, inv16); p1 = __fmul_rn(p1, inv16); p2 = __fmul_rn(p2, inv16); p3 = __fmul_rn(p3, inv16); }
                        const float4 o = make_float4(__fsub_rn(m4.x, p0), __fsub_rn(m4.y, p1), __fsub_rn(m4.z, p2), __fsub_rn(m4.w, p3));
                        any |= fabsf(o.x) > 1.1920928955078125e-07f || fabsf(o.y) > 1.1920928955078125e-07f ||
                               fabsf(o.z) > 1.1920928955078125e-07f || fabsf(o.w) > 1.1920928955078125e-07f;
                        o4[j] = o;
                    }
                    if (wide32) {
                        st_global_v8(reinterpret_cast<float *>(dst + s16 * 4), o4[0], o4[1]);
                        st_global_v8(reinterpret_cast<float *>(dst + s16 * 4 + 2), o4[2], o4[3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) dst[s16 * 4 + j] = o4[j];
                    }
                }
            } else
            for (int c0 = cb; c0 < ce; c0 += 16) {
                unsigned r[16], q[16];
                const unsigned taddr = tmem_d + (unsigned)set * acc_stride + ((unsigned)(quarter * 32) << 16) + (unsigned)c0;
                tmem_ld16(taddr, r);
                if (!one_acc) tmem_ld16(taddr + acc_cols, q);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (F16 && one_acc) {                                // one accumulator (low halves without their factor): the scales taken out
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__fmul_rn(__uint_as_float(r[j]), inv16));
                } else if (F16) {                                    // hi * hi + (cross terms) / 2^11, and the operands' scales taken out
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        r[j] = __float_as_uint(__fmul_rn(__fmaf_rn(__uint_as_float(q[j]), 1.0f / kSplit16LoScale, __uint_as_float(r[j])), inv16));
                } else if (!one_acc) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__fadd_rn(__uint_as_float(r[j]), __uint_as_float(q[j])));
                }
                if (row < g.M) {
                    float4 *dst = reinterpret_cast<float4 *>(C + (long)row * g.ldc + n0 + c0);
                    if (g.minuend) {
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
            // this set may be overwritten by the tile after next
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&bars.acc_empty[set]);
        }
        if (!ok) atomicOr(&bars.failed, 1u);
        if (g.flag && __any_sync(0xffffffffu, any) && lane == 0) atomicOr(g.flag, 1u);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols) : "memory");
    }
}

// cuTensorMapEncodeTiled from the driver, looked up once (the library links the runtime only).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    });
    return fn;
}

bool tma_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("BSQ_GEMM_TMA");                 // 0: keep the register-staged kernels (A/B comparisons)
        return !(e && e[0] == '0');
    }();
    return on;
}

size_t tma_smem_bytes(int n_tile, int nraw, int nr, int nb, bool f16 = false) {
    return 1024 + (size_t)nraw * (f16 ? 2 : 1) * RAW_SLOT + (size_t)nr * A_SLOT + (size_t)nb * 2 * image_half_units(n_tile) * 16 + sizeof(TmaBars) + 64;
}

template <bool AK, int NMAX, bool F16 = false>
cudaError_t launch_tma(const CUtensorMap &map, const GemmArgs &g, dim3 grid, size_t smem, unsigned *status, cudaStream_t stream) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tc_tma_kernel<AK, NMAX, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    gemm_tc_tma_kernel<AK, NMAX, F16><<<grid, NTH, smem, stream>>>(map, g, status);
    return cudaGetLastError();
}

}  // namespace

// Ring lengths.  A contiguous along K: as many slots of A (split in place) as fit beside three images of B (four up to
// 128 columns).  A contiguous along M: two operand stages, and as many raw slots as fit for the copies' head start.
void gemm_tc_tma_rings(int n_tile, bool a_kmajor, int *nraw, int *nr, int *nb, bool f16) {
    *nb = n_tile > 128 ? 3 : 4;
    if (f16) {                                             // raw boxes of 64 k (32 KB), operand stages, images of B
        *nr = 2;
        int r = 4;
        while (r > 2 && tma_smem_bytes(n_tile, r, *nr, *nb, true) > (size_t)227 * 1024) --r;
        *nraw = r;
        return;
    }
    if (a_kmajor) {
        int r = MAXR;
        while (r > 2 && tma_smem_bytes(n_tile, 0, r, *nb) > (size_t)227 * 1024) --r;
        *nr = r;
        *nraw = 0;
    } else {
        *nr = 2;
        int r = MAXR;
        while (r > 2 && tma_smem_bytes(n_tile, r, *nr, *nb) > (size_t)227 * 1024) --r;
        *nraw = r;
    }
}

bool gemm_tc_tma_enabled() { return tma_enabled() && encode_tiled() != nullptr; }

bool gemm_tc_tma_usable(const GemmArgs &g, bool a_kmajor) {
    (void)a_kmajor;
    if (!gemm_tc_tma_enabled() || !g.b_image) return false;
    if (g.M < TM || g.K < 2 * KS || g.n_tile > 256) return false;
    if (g.lda % 4 != 0 || reinterpret_cast<uintptr_t>(g.A) % 16 != 0) return false;
    return g.k_per_split % KS == 0;
}

cudaError_t gemm_tc_tma_launch(const GemmArgs &g, bool a_kmajor, unsigned *status, cudaStream_t stream) {
    CUtensorMap map;
    // innermost dimension first: K (then M) for an A contiguous along K, M (then K) otherwise
    const bool a_img = a_kmajor && g.a_image != nullptr;         // the map then covers the hi and lo matrices, one above the other
    const cuuint64_t dims[2] = {(cuuint64_t)(a_kmajor ? g.K : g.M), (cuuint64_t)(a_img ? 2 * g.a_image_rows : (a_kmajor ? g.M : g.K))};
    const bool img16 = a_img && g.f16;                           // ... of FP16 values: 64 k per 128-byte row of a box
    const cuuint64_t strides[1] = {img16 ? (cuuint64_t)g.K * 2 : (cuuint64_t)(a_img ? g.K : g.lda) * sizeof(float)};
    const cuuint32_t box[2] = {img16 ? 64u : 32u, (cuuint32_t)(a_kmajor ? TM : KS)};
    const cuuint32_t estr[2] = {1, 1};
    static const int l2 = [] { const char *e = std::getenv("BSQ_TMA_L2"); return e ? atoi(e) : 128; }();
    if (encode_tiled()(&map, img16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, a_img ? g.a_image : const_cast<float *>(g.A), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       l2 == 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : (l2 == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE : CU_TENSOR_MAP_L2_PROMOTION_L2_128B),
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    const size_t smem = tma_smem_bytes(g.n_tile, ((a_kmajor && !g.f16) || a_img) ? 0 : g.raw_stages, g.a_stages, g.b_stages, g.f16);
    dim3 grid((g.M + TM - 1) / TM, (g.N + g.n_tile - 1) / g.n_tile, g.splits);
    if (g.persistent) {
        const int tiles = (int)(grid.x * grid.y);
        grid = dim3((unsigned)(tiles < g.sm_count ? tiles : g.sm_count), 1, 1);
    }
    if (g.f16 && g.n_tile > 128) return a_kmajor ? launch_tma<true, 256, true>(map, g, grid, smem, status, stream) : launch_tma<false, 256, true>(map, g, grid, smem, status, stream);
    if (a_kmajor) return g.n_tile <= 128 ? launch_tma<true, 128>(map, g, grid, smem, status, stream) : launch_tma<true, 256>(map, g, grid, smem, status, stream);
    return g.n_tile <= 128 ? launch_tma<false, 128>(map, g, grid, smem, status, stream) : launch_tma<false, 256>(map, g, grid, smem, status, stream);
}

}  // namespace bsq
