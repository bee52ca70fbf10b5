// FP32 GEMM building block of the low-rank stages (sm_100a).
//
// Replaces the cublasSgemm / cublasSdgmm call sites of the reference
// (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:293-309,319-335,344-360,370-386,409-425 and
// modules/reconstruct_lowrank_cuda/src/reconstruct_lowrank_cuda.cu:31-61) with one kernel that reads
// the caller's row-major matrices in whichever orientation a product needs, so the reference's
// explicit transposes of the input and of U, V (svd_lowrank_cuda_utils.cuh:91-109) disappear:
//
//   C[M x N] = opA[M x K] * opB[K x N]
//   A_KMAJOR  : opA(i, kk) = A[i * lda + kk]   (A used as stored)      else opA(i, kk) = A[kk * lda + i]  (A^T)
//   B_KMAJOR  : opB(kk, j) = B[j * ldb + kk]   (B^T of a row-major B)  else opB(kk, j) = B[kk * ldb + j]
//
// All the products of the randomized SVD are "skinny": one of M, N is the rank k (<= 256), the other
// one matrix dimension, and K is the other matrix dimension, so there are few output tiles; the grid's
// third dimension splits K and a second kernel adds the partial tiles in a fixed order (deterministic).
// Optional fusions: a per-k scale on opA (U * diag(S) of reconstruct), and in the epilogue
// "minuend - C" with an any(|.| > FLT_EPSILON) flag (the reference's subtract_kernel + has_nonzero_kernel,
// src/bitsqz_llm.cu:164-184).
//
// This version computes on the FP32 pipes (128 x 128 x 16 tiles, 8 x 8 per thread, double-buffered
// shared memory).
#include "bsq_gemm.hpp"
#include "bsq_internal.hpp"

#include <cstdlib>

namespace bsq {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, GT = 256;
constexpr int PAD = 4;

template <bool KMAJOR>
__device__ __forceinline__ void load_tile(const float *__restrict__ P, long ld, int rows_total, int k_total, int row0, int k0,
                                          int k_end, float (*S)[BM + PAD], bool vec_ok, const float *kscale) {
    // fills S[kk][r] = op(row0 + r, k0 + kk) for r < 128, kk < 16 (zero outside the matrix / split)
    const int t = threadIdx.x;
    if (KMAJOR) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (t >> 2) + h * 64, kk = (t & 3) * 4;
            const int gr = row0 + r, gk = k0 + kk;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (gr < rows_total) {
                const float *src = P + (long)gr * ld + gk;
                if (vec_ok && gk + 3 < k_end) {
                    const float4 q = *reinterpret_cast<const float4 *>(src);
                    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (gk + j < k_end) v[j] = src[j];
                }
                if (kscale) {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (gk + j < k_end) v[j] = __fmul_rn(v[j], kscale[gk + j]);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) S[kk + j][r] = v[j];
        }
    } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kk = (t >> 5) + h * 8, r = (t & 31) * 4;
            const int gk = k0 + kk, gr = row0 + r;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (gk < k_end) {
                const float *src = P + (long)gk * ld + gr;
                if (vec_ok && gr + 3 < rows_total) {
                    const float4 q = *reinterpret_cast<const float4 *>(src);
                    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (gr + j < rows_total) v[j] = src[j];
                }
                if (kscale) {
                    const float s = kscale[gk];
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = __fmul_rn(v[j], s);
                }
            }
            *reinterpret_cast<float4 *>(&S[kk][r]) = make_float4(v[0], v[1], v[2], v[3]);
        }
    }
    (void)k_total;
}

template <bool A_KMAJOR, bool B_KMAJOR>
__global__ void __launch_bounds__(GT) gemm_kernel(GemmArgs g) {
    __shared__ __align__(16) float As[2][BK][BM + PAD];
    __shared__ __align__(16) float Bs[2][BK][BN + PAD];
    const int t = threadIdx.x, tx = t & 15, ty = t >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int k_begin = blockIdx.z * g.k_per_split;
    const int k_end = min(g.K, k_begin + g.k_per_split);
    const bool a_vec = (reinterpret_cast<uintptr_t>(g.A) % 16 == 0) && (g.lda % 4 == 0);
    const bool b_vec = (reinterpret_cast<uintptr_t>(g.B) % 16 == 0) && (g.ldb % 4 == 0);
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    int buf = 0;
    if (k_begin < k_end) {
        load_tile<A_KMAJOR>(g.A, g.lda, g.M, g.K, m0, k_begin, k_end, As[0], a_vec, g.kscale);
        load_tile<B_KMAJOR>(g.B, g.ldb, g.N, g.K, n0, k_begin, k_end, Bs[0], b_vec, nullptr);
    }
    __syncthreads();
    for (int k0 = k_begin; k0 < k_end; k0 += BK) {
        if (k0 + BK < k_end) {
            load_tile<A_KMAJOR>(g.A, g.lda, g.M, g.K, m0, k0 + BK, k_end, As[buf ^ 1], a_vec, g.kscale);
            load_tile<B_KMAJOR>(g.B, g.ldb, g.N, g.K, n0, k0 + BK, k_end, Bs[buf ^ 1], b_vec, nullptr);
        }
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4 *>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4 *>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
        buf ^= 1;
    }

    float *C = g.C + (long)blockIdx.z * g.split_stride;
    bool any = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gm >= g.M) continue;
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const int gn = n0 + jh * 64 + tx * 4;
            float v[4] = {acc[i][jh * 4 + 0], acc[i][jh * 4 + 1], acc[i][jh * 4 + 2], acc[i][jh * 4 + 3]};
            if (g.minuend) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (gn + j < g.N) {
                        v[j] = __fsub_rn(g.minuend[(long)gm * g.ldm + gn + j], v[j]);
                        any |= fabsf(v[j]) > 1.1920928955078125e-07f;
                    }
            }
            float *dst = C + (long)gm * g.ldc + gn;
            if (gn + 3 < g.N && (reinterpret_cast<uintptr_t>(dst) % 16 == 0)) {
                *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (gn + j < g.N) dst[j] = v[j];
            }
        }
    }
    if (g.flag && __any_sync(0xffffffffu, any) && (t & 31) == 0) atomicOr(g.flag, 1u);
}

// C = sum over splits of the partial results, in split order.
__global__ void reduce_splits_kernel(const float *__restrict__ part, float *__restrict__ C, int M, int N, long ldc,
                                     int splits, long split_stride) {
    const long total = (long)M * N;
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
        const int i = (int)(e / N), j = (int)(e % N);
        // eight loads in flight, added in split order (the order fixes the result bit for bit)
        float s = 0.0f;
        int z = 0;
        for (; z + 8 <= splits; z += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = part[(z + u) * split_stride + (long)i * N + j];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += v[u];
        }
        for (; z < splits; ++z) s += part[z * split_stride + (long)i * N + j];
        C[(long)i * ldc + j] = s;
    }
}

cudaError_t launch_reduce(const float *workspace, float *C, int M, int N, long ldc, int splits, int sm_count,
                          cudaStream_t stream) {
    const long total = (long)M * N;
    long rg = (total + 255) / 256;
    if (rg > (long)sm_count * 8) rg = (long)sm_count * 8;
    reduce_splits_kernel<<<(int)rg, 256, 0, stream>>>(workspace, C, M, N, ldc, splits, (long)M * N);
    return cudaGetLastError();
}

// BSQ_GEMM_IMAGE=0 keeps the tensor-core kernel that splits B inside every CTA, =2 uses the kernel with B split
// beforehand wherever it can run (for A/B comparisons and tests); default 1: where it is faster.
int b_image_mode() {
    static const int mode = [] {
        const char *e = std::getenv("BSQ_GEMM_IMAGE");
        return e && e[0] >= '0' && e[0] <= '2' ? e[0] - '0' : 1;
    }();
    return mode;
}

// BSQ_GEMM_AIMAGE=0: the persistent product splits A in the kernel (transform warps) instead of beforehand.
bool a_image_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("BSQ_GEMM_AIMAGE");
        return !(e && e[0] == '0');
    }();
    return on;
}

// BSQ_GEMM_WIDE=0: the persistent product keeps 128-column tiles (two accumulators per tile) when A is split beforehand.
bool wide_tiles_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("BSQ_GEMM_WIDE");
        return !(e && e[0] == '0');
    }();
    return on;
}

// BSQ_GEMM_F16: 0 TF32 halves everywhere; 1 (default): FP16 halves where the caller gives a bound on |A|; 2: also where it
// does not (a pass over A per product).
int f16_mode() {
    static const int mode = [] {
        const char *e = std::getenv("BSQ_GEMM_F16");
        return e && e[0] >= '0' && e[0] <= '2' ? e[0] - '0' : 1;
    }();
    return mode;
}

// BSQ_GEMM_TC=0 keeps every product on the FP32 pipes (for A/B comparisons of the two kernels).
bool tensor_cores_enabled() {
    static const bool on = [] {
        const char *e = std::getenv("BSQ_GEMM_TC");
        return !(e && e[0] == '0');
    }();
    return on;
}

}  // namespace

size_t gemm_workspace_bytes(int M, int N, int max_splits) { return (size_t)M * N * max_splits * sizeof(float); }

// Picks the K split so that about two CTAs per SM are busy; partials go to `workspace` (may be null: no split).
cudaError_t gemm(bool a_kmajor, bool b_kmajor, const float *A, long lda, const float *B, long ldb, float *C, long ldc, int M,
                 int N, int K, const float *kscale, const float *minuend, long ldm, unsigned *flag, unsigned *status,
                 float *workspace, size_t workspace_bytes, int sm_count, cudaStream_t stream, const unsigned *a_absmax_bits, float b_bound) {
    return gemm_select(tensor_cores_enabled(), a_kmajor, b_kmajor, A, lda, B, ldb, C, ldc, M, N, K, kscale, minuend, ldm, flag,
                       status, workspace, workspace_bytes, sm_count, stream, a_absmax_bits, b_bound);
}

cudaError_t gemm_select(bool allow_tensor_cores, bool a_kmajor, bool b_kmajor, const float *A, long lda, const float *B, long ldb,
                        float *C, long ldc, int M, int N, int K, const float *kscale, const float *minuend, long ldm,
                        unsigned *flag, unsigned *status, float *workspace, size_t workspace_bytes, int sm_count,
                        cudaStream_t stream, const unsigned *a_absmax_bits, float b_bound) {
    if (M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
    if (allow_tensor_cores) {
        // tensor-core path: one 128-row tile per CTA, two CTAs per SM up to N = 128; K is split so that the tiles fill
        // the SMs once
        GemmArgs t{};
        t.A = A; t.B = B; t.M = M; t.N = N; t.K = K; t.lda = lda; t.ldb = ldb;
        t.kscale = kscale; t.minuend = minuend; t.ldm = ldm;
        // N up to 256 is one tile; wider products (the reconstruction) are cut into 128-column tiles
        t.n_tile = N <= 256 ? N : 128;
        t.flag = minuend ? flag : nullptr;
        // B split beforehand when several row tiles share it and the workspace has room for its images (at its end)
        const size_t image_bytes = gemm_tc_image_bytes(N, t.n_tile, K);
        // (measured: the products are then bound by what the CTAs draw from L2, A once and B's images once per row
        // tile; that pays for tiles wider than 128 columns, where splitting B in every CTA is two thirds of the
        // staging work, and for long K)
        // (up to 128 columns the register-staged kernel with two CTAs per SM measured faster than either image kernel:
        // 67 against 80-88 us for 8192 x 128 x 4096)
        bool with_image = workspace && image_bytes + 128 <= workspace_bytes &&
                          (b_image_mode() == 2 ? M >= 256 : (b_image_mode() == 1 && M >= 512 && t.n_tile > 128 && K >= 1024));
        // a wide product (the reconstruction: N = a matrix dimension, K = the rank) in 256-column tiles, B's images
        // made once and shared by all row tiles, when the workspace has room for them; otherwise every CTA of a
        // 128-column tile splits its piece of B itself
        if (!with_image && N > 256 && workspace && b_image_mode() >= 1 && M >= 512 && K >= 64 &&
            gemm_tc_image_bytes(N, 256, K) + 128 <= workspace_bytes) {
            t.n_tile = 256;
            with_image = true;
        }
        const size_t image_room = with_image ? gemm_tc_image_bytes(N, t.n_tile, K) : 0;
        if (with_image) workspace_bytes = (workspace_bytes - image_room) & ~(size_t)127;
        const int tiles_tc = ((M + 127) / 128) * ((N + t.n_tile - 1) / t.n_tile);
        int splits_tc = 1;
        if (with_image) {
            // A contiguous along K comes in by TMA (one CTA per SM); the other orientation is staged through registers
            t.b_image = reinterpret_cast<const float4 *>(workspace);      // placeholder for the check; set for good below
            t.k_per_split = 32;
            t.use_tma = gemm_tc_tma_usable(t, a_kmajor);
            t.b_image = nullptr;
            t.sm_count = sm_count;
            if (t.use_tma && N > 256 && (minuend || kscale || tiles_tc >= sm_count)) {       // (no K split then)
                // a wide product on the TMA-fed kernel: 128-column tiles (two accumulator sets fit tensor memory), walked
                // by a persistent grid
                t.n_tile = 128;
                t.persistent = true;
                // a small A read again by every column tile: split once beforehand too, when the workspace has the room
                // (in front of B's images; a persistent product has no K split and so no partial results there)
                const size_t a_room = (gemm_tc_a_image_bytes(M, K) + 127) & ~(size_t)127;
                if (a_kmajor && K % 4 == 0 && a_image_enabled() && workspace_bytes >= a_room && reinterpret_cast<uintptr_t>(workspace) % 128 == 0) {
                    t.a_image = workspace;
                    t.a_image_rows = (M + 127) / 128 * 128;
                    if (wide_tiles_enabled()) {
                        t.n_tile = 256;                                 // (B's images were given room for 256-column tiles above)
                        t.wide_tiles = true;
                        // ... and both operands as FP16 halves (low halves without their factor: the tile's products share
                        // one accumulator); the scales come from the largest |A kscale| and |B|, found by a pass over each
                        // (they are small); the FP16 images take half the room, its last words hold the two maxima
                        if (f16_mode() >= 1 && K % 8 == 0) {
                            unsigned *words = reinterpret_cast<unsigned *>(reinterpret_cast<unsigned char *>(workspace) + a_room - 256);
                            t.f16 = true;
                            t.lo_unscaled = true;
                            t.a_absmax_bits = words;
                            t.b_absmax_bits = words + 1;
                        }
                    }
                }
            }
        }
        const int slots = (t.use_tma ? 1 : with_image ? gemm_tc_image_ctas_per_sm(t.n_tile) : (t.n_tile <= 128 ? 2 : 1)) * sm_count;
        // the FP16 form of the split (BSQ_GEMM_F16=1; =2 also without a given bound on |A|: it is then worked out here,
        // a pass over A): 256-column products with A contiguous along K on the TMA-fed kernel
        if (t.use_tma && !t.persistent && t.n_tile == 256 && !kscale && !minuend && workspace_bytes >= 4096 &&
            (f16_mode() == 2 || (f16_mode() == 1 && a_absmax_bits))) {
            unsigned *words = reinterpret_cast<unsigned *>(workspace);      // [0]: |B| max, [1]: |A| max when not given
            workspace += 64;
            workspace_bytes -= 256;
            t.f16 = true;
            t.b_absmax_bits = words;
            if (b_bound > 0.0f && b_bound < 1.0e30f) t.b_scale_fixed = std::exp2((float)(14 - std::ilogb(b_bound)));
            t.a_absmax_bits = a_absmax_bits;
            if (!a_absmax_bits) {
                const cudaError_t e = gemm_absmax_bits(A, lda, a_kmajor ? M : K, a_kmajor ? K : M, words + 1, stream);
                if (e != cudaSuccess) return e;
                t.a_absmax_bits = words + 1;
            }
        }
        if (t.use_tma) gemm_tc_tma_rings(t.n_tile, a_kmajor, &t.raw_stages, &t.a_stages, &t.b_stages, t.f16 && !t.a_image);
        else if (with_image) gemm_tc_image_rings(t.n_tile, &t.a_stages, &t.b_stages);
        if (workspace && !minuend && !kscale && tiles_tc < slots) {
            const int max_by_k = max(1, K / 256);             // a split below 256 of K costs more in the reduction than it gains
            const int max_by_ws = (int)(workspace_bytes / ((size_t)M * N * sizeof(float)));
            splits_tc = max(1, min(slots / tiles_tc, min(max_by_k, max_by_ws)));
        }
        if (with_image) t.b_image = reinterpret_cast<const float4 *>(reinterpret_cast<unsigned char *>(workspace) + workspace_bytes);
        t.splits = splits_tc;
        t.k_per_split = t.f16 ? ((K + splits_tc - 1) / splits_tc + 63) / 64 * 64 : ((K + splits_tc - 1) / splits_tc + 31) / 32 * 32;
        t.splits = (K + t.k_per_split - 1) / t.k_per_split;                    // no empty split
        if (t.splits > 1) {
            t.C = workspace; t.ldc = N; t.split_stride = (long)M * N;
        } else {
            t.C = C; t.ldc = ldc; t.split_stride = 0;
        }
        if (gemm_tc_eligible(t, a_kmajor, b_kmajor)) {
            cudaError_t err = gemm_tc_launch(t, a_kmajor, b_kmajor, status, stream);
            if (err != cudaSuccess || t.splits == 1) return err;
            return launch_reduce(workspace, C, M, N, ldc, t.splits, sm_count, stream);
        }
    }
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    int splits = 1;
    if (workspace && !minuend && tiles < 2 * sm_count) {
        splits = (2 * sm_count + tiles - 1) / tiles;
        const int max_by_k = (K + 4 * BK - 1) / (4 * BK);                      // at least 64 of K per split
        const int max_by_ws = (int)(workspace_bytes / ((size_t)M * N * sizeof(float)));
        splits = max(1, min(splits, min(max_by_k, max_by_ws)));
    }
    GemmArgs g{};
    g.A = A; g.B = B; g.M = M; g.N = N; g.K = K; g.lda = lda; g.ldb = ldb;
    g.kscale = kscale;
    g.splits = splits;
    g.k_per_split = ((K + splits - 1) / splits + BK - 1) / BK * BK;
    g.minuend = minuend; g.ldm = ldm; g.flag = minuend ? flag : nullptr;
    if (splits > 1) {
        g.C = workspace; g.ldc = N; g.split_stride = (long)M * N;
    } else {
        g.C = C; g.ldc = ldc; g.split_stride = 0;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, splits);
    if (a_kmajor && b_kmajor) gemm_kernel<true, true><<<grid, GT, 0, stream>>>(g);
    else if (a_kmajor) gemm_kernel<true, false><<<grid, GT, 0, stream>>>(g);
    else if (b_kmajor) gemm_kernel<false, true><<<grid, GT, 0, stream>>>(g);
    else gemm_kernel<false, false><<<grid, GT, 0, stream>>>(g);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess || splits == 1) return err;
    return launch_reduce(workspace, C, M, N, ldc, splits, sm_count, stream);
}

}  // namespace bsq
