// Randomized low-rank SVD and low-rank reconstruction (sm_100a host driver + glue kernels).
//
// Replaces svd_lowrank_cuda_initialize / svd_lowrank_cuda / svd_lowrank_cuda_release
// (modules/svd_lowrank_cuda/src/svd_lowrank_cuda.cu:284-581) and reconstruct_lowrank_cuda
// (modules/reconstruct_lowrank_cuda/src/reconstruct_lowrank_cuda.cu:21-62).
//
// Same algorithm family as the reference (Halko-style range finder: Y = W Omega, niter power
// iterations with re-orthonormalisation, projection B = Q^T W, small SVD, U = Q U_hat; the working
// matrix W is A, or A^T when A has fewer rows than columns), different linear algebra:
//   * every product with the big matrix reads the caller's row-major A directly, in either
//     orientation (bsq_gemm.cu) -- no transposed copy of A, no transposes of U and V on the way out;
//   * tall panels are orthonormalised through their k x k Gram matrix instead of Householder QR
//     (Cholesky QR): G = Y^T Y = R^T R, Y <- Y R^-1 -- once inside the power iteration, twice for
//     the bases that the result is built from.  G is shifted by 1e-5 max(diag G) before factoring,
//     so rank-deficient panels (exactly low-rank inputs, all-zero inputs) only leave some columns
//     shorter than unit length instead of dividing by zero;
//   * the small SVD works on a k x k core: B^T = Q2 C with C = R2 R1 the product of the two
//     triangular factors, C = Uc S Vc^T, V_hat = Q2 Uc, U = Q Vc.
// The SVD of the k x k core is a one-sided Jacobi kernel of this library up to 256 columns (one CTA up to 64, a
// thread-block cluster above); larger cores, and devices that cannot place the cluster, go to cuSOLVER's gesvdj on
// the k x k core.  Everything that touches an M- or N-sized array is a kernel of this library.
// Omega comes from cuRAND's XORWOW generator like the reference's (svd_lowrank_cuda.cu:143,289-291),
// seeded per call, column-major N x k.
#include "bsq_device.cuh"
#include "bsq_gemm.hpp"
#include "bsq_internal.hpp"

#include <cooperative_groups.h>
#include <curand.h>
#include <cusolverDn.h>

#include <algorithm>
#include <cstdlib>
#include <new>

namespace bsq {

struct SvdWorkspace {
    int m = 0, n = 0, k = 0, niter = 0, sm_count = 148;
    bool transposed = false;            // working matrix is A^T
    int M = 0, N = 0;                   // working dimensions, M >= N
    float *omega = nullptr;             // N x k, column-major
    float *y = nullptr, *y2 = nullptr;  // M x k
    float *z = nullptr, *z2 = nullptr;  // N x k
    float *g = nullptr;                 // k x k Gram / eigenvectors
    float *w = nullptr;                 // k eigenvalues
    float *t = nullptr, *tinv1 = nullptr, *tinv2 = nullptr, *core = nullptr;   // k x k
    float *uc = nullptr, *vc = nullptr; // k x k outputs of the core SVD
    float *gemm_ws = nullptr;
    size_t gemm_ws_bytes = 0;
    float *solver_work = nullptr;
    int lwork = 0;
    int *dev_info = nullptr;
    curandGenerator_t rng = nullptr;
    cusolverDnHandle_t solver = nullptr;
    gesvdjInfo_t svdj = nullptr;
    // row-sharded mode: sum a device buffer over all ranks, in stream order (null: single GPU)
    SvdAllReduce allreduce = nullptr;
    void *allreduce_ctx = nullptr;
    unsigned *status = nullptr;         // device status word of the current call
    unsigned *own_status = nullptr;     // used when the caller passes none
    unsigned *a_absmax = nullptr;       // bits of the largest |A| of the current call (scale of the FP16 split of the big products)
    bool a_absmax_valid = false;
    const unsigned *a_absmax_use = nullptr;
    int jc_lanes = 4;                   // lanes per column pair of the cluster Jacobi kernel for this k
    bool jc_with_v = false;             // ... and whether it accumulates the right factor (else that comes from the panel)
    bool own_core_svd = false;          // k small enough for jacobi_svd_kernel (else cuSOLVER's gesvdj on the core)
    bool seeded = false;                // omega holds the draw for `seed`
    unsigned long long seed = 0, offset = 0;
    // optional timing of the spans that matter for a roofline: the products with the big matrix (kind 0) and the
    // all-reduces of the row-sharded mode (kind 1), bracketed by events on the call's stream
    static constexpr int kMaxSpans = 32;
    bool profile = false;
    int spans = 0;
    int span_kind[kMaxSpans] = {};
    cudaEvent_t span_ev[2 * kMaxSpans] = {};
};

namespace {

// One CTA factorises the shifted k x k Gram matrix G + s I = R^T R (Cholesky, R upper triangular, in
// place over the upper triangle of A; s = 1e-5 max(diag G)) and inverts R.  The shift, and a floor of
// s / 2 under every pivot, keep a rank-deficient panel from dividing by zero or taking the root of a
// negative number: deficient directions just come out shorter than unit length (an all-zero panel
// gives R = T = 0).  Any invertible R^-1 leaves the span of the panel unchanged; a second pass brings
// every direction above ~3e-5 of the largest singular value to unit length.
//   A    in: G (symmetric, row-major); out: R in the upper triangle, zeros below
//   T    out: R^-1 (upper triangular, row-major), so that Y T has orthonormal columns
//   Rcpy out (nullable): a copy of R, the inverse transform (Y = (Y T) R)
__global__ void __launch_bounds__(1024) cholesky_inverse_kernel(float *A, int k, float *T, float *Rcpy) {
    __shared__ float s_red[32];
    __shared__ float s_floor, s_r;
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
    float md = 0.0f;
    for (int i = tid; i < k; i += nt) md = fmaxf(md, A[(size_t)i * k + i]);
    for (int d = 16; d > 0; d >>= 1) md = fmaxf(md, __shfl_xor_sync(0xffffffffu, md, d));
    if (lane == 0) s_red[warp] = md;
    __syncthreads();
    if (tid == 0) {
        float m = 0.0f;
        for (int w = 0; w < nwarps; ++w) m = fmaxf(m, s_red[w]);
        s_floor = m > 0.0f ? m * 1.0e-5f : 0.0f;
    }
    __syncthreads();
    // shift: G + s I with s = 1e-5 max(diag G), far above the rounding noise of G, so that the Schur
    // complements of a rank-deficient G stay diagonally dominant and R^-1 cannot blow up
    for (int i = tid; i < k; i += nt) A[(size_t)i * k + i] += s_floor;
    __syncthreads();
    for (int j = 0; j < k; ++j) {
        if (tid == 0) {
            float d = A[(size_t)j * k + j];
            if (!(d > 0.5f * s_floor)) d = 0.5f * s_floor;
            s_r = d > 0.0f ? sqrtf(d) : 0.0f;
            A[(size_t)j * k + j] = s_r;
        }
        __syncthreads();
        const float inv = s_r > 0.0f ? 1.0f / s_r : 0.0f;
        for (int c = j + 1 + tid; c < k; c += nt) A[(size_t)j * k + c] *= inv;        // row j of R
        __syncthreads();
        for (int i = j + 1 + warp; i < k; i += nwarps) {                               // trailing update
            const float rji = A[(size_t)j * k + i];
            for (int c = i + lane; c < k; c += 32) A[(size_t)i * k + c] -= rji * A[(size_t)j * k + c];
        }
        __syncthreads();
    }
    for (int e = tid; e < k * k; e += nt) {                // clear below the diagonal, copy R, clear T
        const int i = e / k, c = e % k;
        if (c < i) A[e] = 0.0f;
        if (Rcpy) Rcpy[e] = c < i ? 0.0f : A[e];
        T[e] = 0.0f;
    }
    __syncthreads();
    // T = R^-1, row by row from the bottom: T(i,c) = (delta_ic - sum_{l=i+1..c} R(i,l) T(l,c)) / R(i,i)
    for (int i = k - 1; i >= 0; --i) {
        const float rii = A[(size_t)i * k + i];
        const float inv = rii > 0.0f ? 1.0f / rii : 0.0f;
        for (int c = i + tid; c < k; c += nt) {
            float acc = (c == i) ? 1.0f : 0.0f;
            for (int l = i + 1; l <= c; ++l) acc -= A[(size_t)i * k + l] * T[(size_t)l * k + c];
            T[(size_t)i * k + c] = acc * inv;
        }
        __syncthreads();
    }
}

// The same factorisation and inverse for k up to kCholeskySmemMaxK, entirely in shared memory: the upper
// triangle is held packed (row i at row_off(i) + c, c >= i), k (k + 1) / 2 floats, so k = 256 takes 129 KB.
// G is only read; R goes to Rcpy, R^-1 to T (both full row-major k x k with zeros below the diagonal).
// Two CTA barriers per column in the factorisation, two per row in the inversion.
constexpr int kCholeskySmemMaxK = 320;
__host__ __device__ constexpr size_t cholesky_smem_bytes(int k) { return ((size_t)k * (k + 1) / 2 + 2 * (size_t)k + 2 * 1024 + 64) * sizeof(float); }

__global__ void __launch_bounds__(1024) cholesky_inverse_smem_kernel(const float *__restrict__ G, int k, float *__restrict__ T,
                                                                     float *__restrict__ Rcpy) {
    extern __shared__ float sm[];
    float *P = sm;                                         // packed upper triangle
    float *vec = sm + (size_t)k * (k + 1) / 2;             // 2 x k: the scaled pivot row / the row of R being inverted
    float *part = vec + 2 * k;                             // 2 x 1024: partial sums of the split dot products
    float *red = part + 2 * 1024;                          // 32 + 1
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
    auto row_off = [k](int i) { return i * k - (i * (i - 1)) / 2 - i; };
    float md = 0.0f;
    for (int e = tid; e < k * k; e += nt) {
        const int i = e / k, c = e % k;
        if (c >= i) {
            const float v = G[e];
            P[row_off(i) + c] = v;
            if (c == i) md = fmaxf(md, v);
        }
    }
    for (int d = 16; d > 0; d >>= 1) md = fmaxf(md, __shfl_xor_sync(0xffffffffu, md, d));
    if (lane == 0) red[warp] = md;
    __syncthreads();
    if (tid == 0) {
        float m = 0.0f;
        for (int w = 0; w < nwarps; ++w) m = fmaxf(m, red[w]);
        red[32] = m > 0.0f ? m * 1.0e-5f : 0.0f;
    }
    __syncthreads();
    const float shift = red[32];
    for (int i = tid; i < k; i += nt) P[row_off(i) + i] += shift;
    __syncthreads();
    for (int j = 0; j < k; ++j) {
        // pivot and scaled row j (every thread derives the pivot itself; it is stored in the next phase)
        const int oj = row_off(j);
        float d = P[oj + j];
        if (!(d > 0.5f * shift)) d = 0.5f * shift;
        const float r = d > 0.0f ? sqrtf(d) : 0.0f;
        const float inv = r > 0.0f ? 1.0f / r : 0.0f;
        for (int c = j + 1 + tid; c < k; c += nt) vec[c] = P[oj + c] * inv;
        __syncthreads();
        if (tid == 0) P[oj + j] = r;
        for (int c = j + 1 + tid; c < k; c += nt) P[oj + c] = vec[c];
        for (int i = j + 1 + warp; i < k; i += nwarps) {    // trailing update, one warp per row
            const float rji = vec[i];
            const int oi = row_off(i);
            for (int c = i + lane; c < k; c += 32) P[oi + c] -= rji * vec[c];
        }
        __syncthreads();
    }
    for (int e = tid; e < k * k; e += nt) {                // R out; T's zeros below the diagonal
        const int i = e / k, c = e % k;
        if (Rcpy) Rcpy[e] = c < i ? 0.0f : P[row_off(i) + c];
        if (c < i) T[e] = 0.0f;
    }
    __syncthreads();
    // T = R^-1 in place, row by row from the bottom: T(i,c) = (delta_ic - sum_{l=i+1..c} R(i,l) T(l,c)) / R(i,i).
    // Column c is served by `ways` threads (one per residue of l); their partial sums are added in a fixed order,
    // so the result is the same on every run.  vec and part alternate between two copies: the stores of row i - 1
    // may overtake the last reads of row i.
    const int ways = max(1, min(32, nt / k));              // 1024 / 256 = 4, 1024 / 128 = 8
    const int c_of = tid % k, way = tid / k;
    for (int i = k - 1; i >= 0; --i) {
        const int oi = row_off(i);
        float *v = vec + (i & 1) * k, *ps = part + (i & 1) * 1024;
        for (int c = i + tid; c < k; c += nt) v[c] = P[oi + c];
        __syncthreads();
        if (way < ways) {
            float acc = 0.0f;
            for (int l = i + 1 + way; l <= c_of; l += ways) acc += v[l] * P[row_off(l) + c_of];
            ps[way * k + c_of] = acc;
        }
        __syncthreads();
        const float rii = v[i];
        const float inv = rii > 0.0f ? 1.0f / rii : 0.0f;
        for (int c = i + tid; c < k; c += nt) {
            float sum = 0.0f;
            for (int w = 0; w < ways; ++w) sum += ps[w * k + c];
            P[oi + c] = ((c == i ? 1.0f : 0.0f) - sum) * inv;
        }
    }
    __syncthreads();
    for (int e = tid; e < k * k; e += nt) {
        const int i = e / k, c = e % k;
        if (c >= i) T[e] = P[row_off(i) + c];
    }
}

// The same again for k <= kCholeskyBlockedMaxK, by 32 x 32 blocks, which takes the number of CTA-wide barriers from
// four per column to a handful per block column.  The block-upper-triangular matrix lives in shared memory
// (block (I, J), I <= J, at blk_id(I, J)); k is padded to a multiple of 32 with an identity.
//   factorisation, per block column J: warp 0 factors the diagonal block in registers (one column per lane, the
//       pivot row travels by shuffles); every thread then solves one column of the block row against it
//       (R_JJ^T Y = G_JC, forward substitution), and all threads apply the rank-32 update to the trailing blocks;
//       every sum runs in the order of the unblocked algorithm (the pivots use a reciprocal square root, so R agrees
//       with it to rounding, not bit for bit);
//   inverse: the diagonal blocks are inverted by one warp each, all at once; block column J of T = R^-1 is then
//       T_IJ = -(sum_{L=I..J-1} T_IL R_LJ) T_JJ, two rounds of 32 x 32 block products per column.
constexpr int kCholeskyBlockedMaxK = 256;
constexpr int kCB = 32;
__host__ __device__ constexpr int chol_blocks(int k) { return (k + kCB - 1) / kCB; }
__host__ __device__ constexpr size_t cholesky_blocked_smem_bytes(int k) {
    // packed blocks + inverted diagonal blocks + one temporary block column + 1 / diagonal + scalars
    return ((size_t)(chol_blocks(k) * (chol_blocks(k) + 1) / 2 + 2 * chol_blocks(k)) * kCB * kCB + (size_t)chol_blocks(k) * kCB + 64) *
           sizeof(float);
}
__device__ __forceinline__ int blk_id(int I, int J, int nb) { return I * nb - (I * (I - 1)) / 2 + (J - I); }

// Sixteen 32 x 32 block products at a time: 64 threads per product, 4 x 4 outputs per thread (rows 4 ti .. + 3,
// columns 4 tc .. + 3), operands read as float4: 2 shared-memory loads per 16 multiply-adds (with 2 x 2 outputs
// per thread the loads, not the arithmetic, filled the issue slots of the one SM this kernel runs on).
//   out -= A^T B  (AT = true:  A, B hold the contraction index in rows)
//   out += A B    (AT = false: A holds it in columns)
template <bool AT>
__device__ __forceinline__ void block_mac(float (&acc)[4][4], const float *__restrict__ A, const float *__restrict__ B, int ti, int tc) {
    if (AT) {
#pragma unroll 4
        for (int l = 0; l < kCB; ++l) {
            const float4 a = *reinterpret_cast<const float4 *>(A + l * kCB + 4 * ti);
            const float4 b = *reinterpret_cast<const float4 *>(B + l * kCB + 4 * tc);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[r][q] = fmaf(-av[r], bv[q], acc[r][q]);
        }
    } else {
#pragma unroll 2
        for (int l0 = 0; l0 < kCB; l0 += 4) {
            float4 a[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const float4 *>(A + (4 * ti + r) * kCB + l0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 b = *reinterpret_cast<const float4 *>(B + (l0 + u) * kCB + 4 * tc);
                const float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float ar = u == 0 ? a[r].x : (u == 1 ? a[r].y : (u == 2 ? a[r].z : a[r].w));
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[r][q] += ar * bv[q];
                }
            }
        }
    }
}
// a thread's 4 x 4 tile of a block, as four float4
__device__ __forceinline__ void tile_load(float (&acc)[4][4], const float *O, int ti, int tc) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float4 v = *reinterpret_cast<const float4 *>(O + (4 * ti + r) * kCB + 4 * tc);
        acc[r][0] = v.x; acc[r][1] = v.y; acc[r][2] = v.z; acc[r][3] = v.w;
    }
}
__device__ __forceinline__ void tile_store(const float (&acc)[4][4], float *O, int ti, int tc, float sign) {
#pragma unroll
    for (int r = 0; r < 4; ++r)
        *reinterpret_cast<float4 *>(O + (4 * ti + r) * kCB + 4 * tc) =
            make_float4(sign * acc[r][0], sign * acc[r][1], sign * acc[r][2], sign * acc[r][3]);
}

__global__ void __launch_bounds__(1024) cholesky_inverse_blocked_kernel(const float *__restrict__ G, int k, float *__restrict__ T,
                                                                        float *__restrict__ Rcpy) {
    extern __shared__ __align__(16) float sm[];
    const int nb = chol_blocks(k), nbt = nb * (nb + 1) / 2;
    float *blocks = sm;                                    // nbt blocks of 32 x 32, row-major
    float *tinv = blocks + (size_t)nbt * kCB * kCB;        // nb inverted diagonal blocks
    float *tmp = tinv + (size_t)nb * kCB * kCB;            // nb blocks: one block column of partial products
    float *dinv = tmp + (size_t)nb * kCB * kCB;            // 1 / R(i, i)
    float *red = dinv + nb * kCB;                          // 32 + 1
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarps = nt >> 5;
    const int bi = tid >> 5, bc = tid & 31;               // this thread's element of a block when the CTA walks blocks
    const int part = tid >> 6, ti = (tid & 63) >> 3, tc = tid & 7;         // ... and its 4 x 4 tile of its sixteenth's block
    // load block by block (row bi, column bc of each), padded with an identity; what lies below the diagonal of a
    // diagonal block is never read.  Four blocks per trip, so that four global loads are in flight per thread.
    float md = 0.0f;
    for (int b0 = 0; b0 < nbt; b0 += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int b = b0 + u;
            v[u] = 0.0f;
            if (b < nbt) {
                int I = 0, rem = b;
                while (rem >= nb - I) { rem -= nb - I; ++I; }      // block (I, I + rem)
                const int i = I * kCB + bi, c = (I + rem) * kCB + bc;
                v[u] = (i == c) ? 1.0f : 0.0f;
                if (i < k && c < k) v[u] = G[(size_t)i * k + c];
                if (i == c && i < k) md = fmaxf(md, v[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (b0 + u < nbt) blocks[(size_t)(b0 + u) * kCB * kCB + tid] = v[u];
    }
    for (int d = 16; d > 0; d >>= 1) md = fmaxf(md, __shfl_xor_sync(0xffffffffu, md, d));
    if (lane == 0) red[warp] = md;
    __syncthreads();
    if (tid == 0) {
        float m = 0.0f;
        for (int w = 0; w < nwarps; ++w) m = fmaxf(m, red[w]);
        red[32] = m > 0.0f ? m * 1.0e-5f : 0.0f;
    }
    __syncthreads();
    const float shift = red[32];
    for (int i = tid; i < k; i += nt) blocks[(size_t)blk_id(i / kCB, i / kCB, nb) * kCB * kCB + (i % kCB) * (kCB + 1)] += shift;
    __syncthreads();

    for (int J = 0; J < nb; ++J) {
        float *D = blocks + (size_t)blk_id(J, J, nb) * kCB * kCB;
        if (warp == 0) {                                    // diagonal block: lane c keeps column c
            float a[kCB];
#pragma unroll
            for (int i = 0; i < kCB; ++i) a[i] = D[i * kCB + lane];
            float my_inv = 0.0f;
#pragma unroll
            for (int j = 0; j < kCB; ++j) {
                float d = __shfl_sync(0xffffffffu, a[j], j);
                if (!(d > 0.5f * shift)) d = 0.5f * shift;
                // the 32 pivots of a block are one dependent chain: reciprocal square root from the special-function
                // unit plus one Newton step (a relative error of ~1e-7 in R(j, j) and 1 / R(j, j) alike) instead of
                // an IEEE square root followed by an IEEE division
                float inv = 0.0f;
                if (d > 0.0f) {
                    inv = rsqrtf(d);
                    inv = inv * (1.5f - 0.5f * d * inv * inv);
                }
                const float r = d * inv;
                a[j] = (lane == j) ? r : a[j] * inv;
                if (lane == j) my_inv = inv;
#pragma unroll
                for (int i = j + 1; i < kCB; ++i) {
                    const float rji = __shfl_sync(0xffffffffu, a[j], i);
                    a[i] -= rji * a[j];
                }
            }
#pragma unroll
            for (int i = 0; i < kCB; ++i) D[i * kCB + lane] = (i <= lane) ? a[i] : 0.0f;
            dinv[J * kCB + lane] = my_inv;
        }
        __syncthreads();
        // block row J: one thread per column, forward substitution with R_JJ^T
        for (int col = tid; col < (nb - J - 1) * kCB; col += nt) {
            float *X = blocks + (size_t)blk_id(J, J + 1 + col / kCB, nb) * kCB * kCB + col % kCB;
            float y[kCB];
#pragma unroll
            for (int i = 0; i < kCB; ++i) {
                float acc = X[i * kCB];
#pragma unroll
                for (int l = 0; l < i; ++l) acc -= D[l * kCB + i] * y[l];
                y[i] = acc * dinv[J * kCB + i];
            }
#pragma unroll
            for (int i = 0; i < kCB; ++i) X[i * kCB] = y[i];
        }
        __syncthreads();
        // trailing blocks (A, B), J < A <= B: G_AB -= R_JA^T R_JB, sixteen blocks per trip
        {
            const int rest = nb - J - 1, pairs = rest * (rest + 1) / 2;
            for (int pr0 = 0; pr0 < pairs; pr0 += 16) {
                const int pr = pr0 + part;
                if (pr < pairs) {
                    int A = 0, rem = pr;
                    while (rem >= rest - A) { rem -= rest - A; ++A; }
                    const int B = A + rem;
                    const float *RA = blocks + (size_t)blk_id(J, J + 1 + A, nb) * kCB * kCB;
                    const float *RB = blocks + (size_t)blk_id(J, J + 1 + B, nb) * kCB * kCB;
                    float *O = blocks + (size_t)blk_id(J + 1 + A, J + 1 + B, nb) * kCB * kCB;
                    float acc[4][4];
                    tile_load(acc, O, ti, tc);
                    block_mac<true>(acc, RA, RB, ti, tc);
                    tile_store(acc, O, ti, tc, 1.0f);
                }
            }
        }
        __syncthreads();
    }
    // R out and the zeros below the diagonal of R and T, block by block; the diagonal blocks' inverses, one warp each
    for (int I = 0; I < nb; ++I) {
        for (int Jb = 0; Jb < nb; ++Jb) {
            const int i = I * kCB + bi, c = Jb * kCB + bc;
            if (i < k && c < k) {
                const size_t e = (size_t)i * k + c;
                if (c < i) {
                    if (T) T[e] = 0.0f;
                    if (Rcpy) Rcpy[e] = 0.0f;
                } else if (Rcpy) {
                    Rcpy[e] = blocks[(size_t)blk_id(I, Jb, nb) * kCB * kCB + tid];
                }
            }
        }
    }
    if (!T) return;                                         // only the factor was wanted (uniform over the CTA)
    if (warp < nb) {
        const float *D = blocks + (size_t)blk_id(warp, warp, nb) * kCB * kCB;
        float a[kCB], t[kCB];
#pragma unroll
        for (int i = 0; i < kCB; ++i) { a[i] = D[i * kCB + lane]; t[i] = 0.0f; }
        const float my_inv = dinv[warp * kCB + lane];
#pragma unroll
        for (int i = kCB - 1; i >= 0; --i) {
            float acc = (lane == i) ? 1.0f : 0.0f;
#pragma unroll
            for (int l = i + 1; l < kCB; ++l) acc -= __shfl_sync(0xffffffffu, a[i], l) * t[l];
            const float inv = __shfl_sync(0xffffffffu, my_inv, i);
            t[i] = (lane >= i) ? acc * inv : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < kCB; ++i) tinv[(size_t)warp * kCB * kCB + i * kCB + lane] = t[i];
    }
    __syncthreads();
    // block column J of T, from the left: needs T_IL for L < J (already in place) and R_LJ (still in place)
    for (int J = 1; J < nb; ++J) {
        for (int I0 = 0; I0 < J; I0 += 16) {
            const int I = I0 + part;
            if (I < J) {
                float acc[4][4] = {};
                for (int L = I; L < J; ++L) {
                    const float *TL = (L == I) ? tinv + (size_t)I * kCB * kCB : blocks + (size_t)blk_id(I, L, nb) * kCB * kCB;
                    block_mac<false>(acc, TL, blocks + (size_t)blk_id(L, J, nb) * kCB * kCB, ti, tc);
                }
                tile_store(acc, tmp + (size_t)I * kCB * kCB, ti, tc, 1.0f);
            }
        }
        __syncthreads();
        const float *TJ = tinv + (size_t)J * kCB * kCB;
        for (int I0 = 0; I0 < J; I0 += 16) {
            const int I = I0 + part;
            if (I < J) {
                float acc[4][4] = {};
                block_mac<false>(acc, tmp + (size_t)I * kCB * kCB, TJ, ti, tc);
                tile_store(acc, blocks + (size_t)blk_id(I, J, nb) * kCB * kCB, ti, tc, -1.0f);
            }
        }
        __syncthreads();
    }
    for (int I = 0; I < nb; ++I) {
        for (int Jb = I; Jb < nb; ++Jb) {
            const int i = I * kCB + bi, c = Jb * kCB + bc;
            if (i < k && c < k && c >= i) {
                const float *src = (I == Jb) ? tinv + (size_t)I * kCB * kCB : blocks + (size_t)blk_id(I, Jb, nb) * kCB * kCB;
                T[(size_t)i * k + c] = src[tid];
            }
        }
    }
}

// SVD of the k x k core for k <= kJacobiMaxK: one-sided (Hestenes) Jacobi in one CTA, everything in shared memory.
// The reference runs cusolverDnSgesvd on the k x n matrix B (svd_lowrank_cuda.cu:399-440); here only the k x k
// triangular factor is left to decompose.
//   in : C, row-major k x k; read as the column-major matrix M = C^T (column j = row j of C)
//   out: M = U diag(S) V^T with S descending; U and V column-major k x k
// Column pairs (p, q) are rotated until all columns of M V are orthogonal to tol (LAPACK's sgesvj criterion,
// |m_p . m_q| <= tol |m_p| |m_q|, tol = sqrt(len) eps); the k / 2 pairs of a round are disjoint (round-robin
// schedule), 8 lanes serve a pair, a CTA barrier separates the rounds.  Squared column norms are carried along
// through the rotations and recomputed exactly at the start of every sweep.  At the end S(j) = |column j|,
// U(:, j) = column j / S(j) (zero for S(j) = 0), and a rank by counting puts S in descending order.
constexpr int kJacobiMaxK = 128;              // what the one-CTA kernel can hold
constexpr int kJacobiSingleMaxK = 64;         // what it is used for: above, the cluster kernel is faster
constexpr int kJacobiMaxSweeps = 30;
// A sweep in which no visited pair had |cos(m_p, m_q)| above this is the last one: Jacobi converges quadratically,
// so what such a sweep's rotations leave between the columns is of the order of the square of what it met
// (<= 1e-8, below tol), and the sweep that would only confirm it (a full sweep's time for no rotation) is not run.
// Pairs between tol and this bound are still rotated when they are met.
constexpr float kJacobiLastSweepCos = 1.0e-4f;
__host__ __device__ constexpr int jacobi_len(int k) { return k <= 64 ? 64 : 128; }
__host__ __device__ constexpr size_t jacobi_smem_bytes(int k) {
    return ((size_t)2 * ((k + 1) & ~1) * jacobi_len(k) + 2 * (size_t)((k + 1) & ~1) + 64) * sizeof(float);
}

__global__ void __launch_bounds__(512) jacobi_svd_kernel(const float *__restrict__ C, int k, float *__restrict__ S,
                                                         float *__restrict__ Ucol, float *__restrict__ Vcol) {
    extern __shared__ __align__(16) float sm[];
    const int LEN = jacobi_len(k), kp = (k + 1) & ~1, npairs = kp / 2;
    float *M = sm, *V = M + (size_t)kp * LEN, *nrm = V + (size_t)kp * LEN;
    int *rank_of = reinterpret_cast<int *>(nrm + kp);
    const int tid = threadIdx.x, nt = blockDim.x;
    const int slot = tid >> 3, l = tid & 7;                   // 8 lanes per pair, 64 pair slots
    const int F4 = LEN / 32;                                  // float4 per lane and column: 2 or 4
    for (int e0 = tid; e0 < kp * LEN; e0 += 4 * nt) {        // four global loads in flight per thread
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt, j = e / LEN, i = e % LEN;
            v[u] = (e < kp * LEN && j < k && i < k) ? C[(size_t)j * k + i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt, j = e / LEN, i = e % LEN;
            if (e < kp * LEN) {
                M[e] = v[u];
                V[e] = (i == j && j < k) ? 1.0f : 0.0f;
            }
        }
    }
    __syncthreads();
    const float tol = sqrtf((float)LEN) * 5.9604645e-08f, tol2 = tol * tol;
    auto sum8 = [&](float x) {                                // sum over the 8 lanes of a pair slot
        x += __shfl_xor_sync(0xffffffffu, x, 4, 8);
        x += __shfl_xor_sync(0xffffffffu, x, 2, 8);
        x += __shfl_xor_sync(0xffffffffu, x, 1, 8);
        return x;
    };
    // squared norm of column j; every lane of a warp calls it together (columns past the end count as zero)
    auto norm2 = [&](int j) {
        float acc = 0.0f;
        if (j < kp) {
            for (int f = 0; f < F4; ++f) {
                const float4 a = reinterpret_cast<const float4 *>(M + (size_t)j * LEN)[f * 8 + l];
                acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
            }
        }
        return sum8(acc);
    };
    for (int sweep = 0; sweep < kJacobiMaxSweeps; ++sweep) {
        for (int j0 = 0; j0 < kp; j0 += nt / 8) {             // exact squared norms (uniform trip count: shuffles inside)
            const float a = norm2(j0 + slot);
            if (l == 0 && j0 + slot < kp) nrm[j0 + slot] = a;
        }
        __syncthreads();
        bool rotated = false;
        for (int r = 0; r < kp - 1; ++r) {
            const bool active = slot < npairs;
            int p = 0, q = 0;
            if (active) {
                if (slot == 0) { p = kp - 1; q = r; }
                else { p = (r + slot) % (kp - 1); q = (r + kp - 1 - slot) % (kp - 1); }
            }
            float4 *mp = reinterpret_cast<float4 *>(M + (size_t)p * LEN), *mq = reinterpret_cast<float4 *>(M + (size_t)q * LEN);
            float4 ap[4], aq[4];
            float g = 0.0f;
#pragma unroll
            for (int f = 0; f < 4; ++f) {
                if (f < F4) {
                    ap[f] = mp[f * 8 + l];
                    aq[f] = mq[f * 8 + l];
                    g += ap[f].x * aq[f].x + ap[f].y * aq[f].y + ap[f].z * aq[f].z + ap[f].w * aq[f].w;
                }
            }
            g = sum8(g);
            const float alpha = nrm[p], beta = nrm[q];
            // |m_p . m_q| > tol |m_p| |m_q|, compared in squares
            if (active && alpha > 0.0f && beta > 0.0f && g * g > tol2 * alpha * beta) {
                const float zeta = (beta - alpha) / (2.0f * g);
                // 1 / (2 zeta) once zeta^2 would overflow: the rotation is then too small to change anything
                const float t = fabsf(zeta) > 1.0e8f ? 0.5f / zeta : copysignf(1.0f, zeta) / (fabsf(zeta) + sqrtf(1.0f + zeta * zeta));
                const float c = rsqrtf(1.0f + t * t), sn = c * t;
                float4 *vp = reinterpret_cast<float4 *>(V + (size_t)p * LEN), *vq = reinterpret_cast<float4 *>(V + (size_t)q * LEN);
#pragma unroll
                for (int f = 0; f < 4; ++f) {
                    if (f < F4) {
                        const float4 x = ap[f], y = aq[f];
                        mp[f * 8 + l] = make_float4(c * x.x - sn * y.x, c * x.y - sn * y.y, c * x.z - sn * y.z, c * x.w - sn * y.w);
                        mq[f * 8 + l] = make_float4(sn * x.x + c * y.x, sn * x.y + c * y.y, sn * x.z + c * y.z, sn * x.w + c * y.w);
                        const float4 u = vp[f * 8 + l], w = vq[f * 8 + l];
                        vp[f * 8 + l] = make_float4(c * u.x - sn * w.x, c * u.y - sn * w.y, c * u.z - sn * w.z, c * u.w - sn * w.w);
                        vq[f * 8 + l] = make_float4(sn * u.x + c * w.x, sn * u.y + c * w.y, sn * u.z + c * w.z, sn * u.w + c * w.w);
                    }
                }
                if (l == 0) {
                    nrm[p] = fmaxf(alpha - t * g, 0.0f);
                    nrm[q] = beta + t * g;
                }
                rotated = rotated || g * g > kJacobiLastSweepCos * kJacobiLastSweepCos * alpha * beta;
            }
            __syncthreads();
        }
        if (!__syncthreads_or(rotated)) break;
    }
    // singular values, order, output
    for (int j0 = 0; j0 < kp; j0 += nt / 8) {
        const float a = norm2(j0 + slot);
        if (l == 0 && j0 + slot < kp) nrm[j0 + slot] = sqrtf(a);
    }
    __syncthreads();
    for (int j = tid; j < k; j += nt) {
        const float sj = nrm[j];
        int rk = 0;
        for (int i = 0; i < k; ++i) {
            const float si = nrm[i];
            rk += (si > sj || (si == sj && i < j)) ? 1 : 0;
        }
        rank_of[j] = rk;
        S[rk] = sj;
    }
    __syncthreads();
    for (int e = tid; e < k * k; e += nt) {
        const int j = e / k, i = e % k;
        const float sj = nrm[j];
        const size_t o = (size_t)rank_of[j] * k + i;
        Ucol[o] = sj > 0.0f ? M[(size_t)j * LEN + i] / sj : 0.0f;
        Vcol[o] = V[(size_t)j * LEN + i];
    }
}

// The same Jacobi iteration for larger cores, up to kJacobiClusterMaxK (two 256 x 256 matrices do not fit one SM's
// shared memory, and already at 128 x 128 one SM's shared-memory bandwidth is the limit): a thread-block cluster of
// 8 CTAs, each holding a slice of LEN / 8 rows of every column of M and V.  A column
// pair's dot product is the sum of the eight slices' partial products: every CTA stores its partials into the
// shared memory of all eight (distributed shared memory), one cluster barrier later every CTA adds them in the
// same order, so all of them see bit-identical values, take identical decisions and rotate their own slices with
// identical angles.  Control flow is the same in all CTAs by construction (same data, same arithmetic), which is
// what the hardware cluster barrier needs; the sweep count is bounded.
constexpr int kJacobiClusterMaxK = 256;
constexpr int kJcCtas = 8;                                   // 16 measured slower: the partial products take longer to arrive
__host__ __device__ constexpr int jacobi_cluster_len(int k) { return k <= 128 ? 128 : 256; }     // padded column length
__host__ __device__ constexpr size_t jacobi_cluster_smem_bytes(int k) {
    // M and V slices, norms, two rounds of CTAs x LEN / 2 partial products, CTAs x LEN partial norms, ranks, votes, mbarriers
    return ((size_t)2 * ((k + 1) & ~1) * (jacobi_cluster_len(k) / kJcCtas) + ((k + 1) & ~1) + kJcCtas * jacobi_cluster_len(k) +
            kJcCtas * jacobi_cluster_len(k) + jacobi_cluster_len(k) + 64) *
           sizeof(float);
}

// The shared::cluster address of `smem_addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ unsigned cluster_addr(unsigned smem_addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// 16-byte store into another CTA's shared memory that counts itself off on that CTA's mbarrier when it has landed:
// the receiver waits for the bytes, no fence and no cluster-wide barrier on the sender's side.
__device__ __forceinline__ void st_async_f4(unsigned dst, const float4 &v, unsigned mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(dst), "f"(v.x),
                 "f"(v.y), "f"(v.z), "f"(v.w), "r"(mbar)
                 : "memory");
}

// kWithV = false leaves the right factor out: nothing accumulates the rotations (half the shared-memory traffic of a
// round), and Vcol receives column j of M divided by S(j)^2 instead -- the k x k matrix that turns the panel the core
// came from into its singular vectors (B^T v_j / S(j) with v_j = M(:, j) / S(j)).
template <int kJcLen, int kLpp, bool kWithV>
__global__ void __launch_bounds__(kJcLen / 2 * kLpp, 1) jacobi_svd_cluster_kernel(const float *__restrict__ C, int k, float *__restrict__ S,
                                                                        float *__restrict__ Ucol, float *__restrict__ Vcol,
                                                                        unsigned *__restrict__ status) {
    constexpr int kJcRows = kJcLen / kJcCtas, kJcF4 = kJcRows / (4 * kLpp);      // rows per CTA; float4 per lane and column
    static_assert(kLpp == 2 || kLpp == 4, "lanes per column pair");
    static_assert(kJcF4 == 1 || kJcF4 == 2 || kJcF4 == 4, "float4 per lane and column");
    constexpr int kSlots = kJcLen / 2;                                   // pair slots = partial products per CTA and round
    constexpr unsigned kRoundBytes = kJcCtas * kSlots * sizeof(float);   // what one CTA receives per round
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned cr = cluster.block_rank();                 // this CTA holds rows cr * kJcRows .. + kJcRows - 1
    extern __shared__ __align__(16) float sm[];
    const int kp = (k + 1) & ~1, npairs = kp / 2;
    float *M = sm, *V = M + (size_t)kp * kJcRows, *nrm = V + (size_t)kp * kJcRows;
    float *part = nrm + ((kp + 3) & ~3);                      // [2][kJcCtas][kSlots], 16-byte aligned
    float *npart = part + 2 * kJcCtas * kSlots;               // [kJcCtas][kJcLen]
    int *rank_of = reinterpret_cast<int *>(npart + kJcCtas * kJcLen);
    int *votes = rank_of + kJcLen;                            // [kJcCtas]
    uint64_t *mbar = reinterpret_cast<uint64_t *>(votes + kJcCtas);      // [2], one per parity of the round counter
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31;
    const int slot = tid / kLpp, l = tid % kLpp;              // kLpp lanes per pair, kSlots pair slots, kJcF4 float4 per lane and column
    // A warp holds 32 / kLpp pair slots, that many partial products per round, in groups of four: the warp is cut
    // into as many parts as it has groups, and in each part lane d (d < 8) sends the part's group as one 16-byte
    // store to CTA d.
    static_assert(kJcCtas == 8, "one sending lane per destination CTA and group");
    constexpr int kPartLanes = 4 * kLpp;                      // lanes that own one group of four slots
    const int part_lane0 = lane / kPartLanes * kPartLanes;
    const bool sender = lane - part_lane0 < kJcCtas;
    const unsigned part_to = cluster_addr(smem_u32(part + cr * kSlots + (tid >> 5) * (32 / kLpp) + part_lane0 / kLpp), lane & 7);
    const unsigned mbar_to = cluster_addr(smem_u32(mbar), lane & 7);
    // A column slice of more than one float4 per lane starts at a multiple of 128 bytes, the same banks for every
    // slot: slot s takes its float4 in the order f ^ (s mod kJcF4), so neighbouring slots spread over all banks.
    const int fsw = slot & (kJcF4 - 1);
    const int row0 = cr * kJcRows;
    if (tid == 0) {
        mbar_init(&mbar[0], 1);
        mbar_init(&mbar[1], 1);
        mbar_fence_init();
    }
    for (int e0 = tid; e0 < kp * kJcRows; e0 += 4 * nt) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt, j = e / kJcRows, i = row0 + e % kJcRows;
            v[u] = (e < kp * kJcRows && j < k && i < k) ? C[(size_t)j * k + i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int e = e0 + u * nt, j = e / kJcRows, i = row0 + e % kJcRows;
            if (e < kp * kJcRows) {
                M[e] = v[u];
                if (kWithV) V[e] = (i == j && j < k) ? 1.0f : 0.0f;
            }
        }
    }
    __syncthreads();
    const float tol = sqrtf((float)kJcLen) * 5.9604645e-08f, tol2 = tol * tol;
    auto sum4 = [&](float x) {                                // over the lanes of a pair
        if (kLpp == 4) x += __shfl_xor_sync(0xffffffffu, x, 2, 4);
        x += __shfl_xor_sync(0xffffffffu, x, 1, kLpp);
        return x;
    };
    // Exact squared norms of all columns (partial over this CTA's rows, exchanged, added in CTA order) and, on the
    // same cluster barrier, the CTAs' votes: bit 0 = "met a pair above kJacobiLastSweepCos in the last sweep", bit 1 = "a wait ran out".
    // Every CTA reads the same eight votes, so all of them leave the sweep loop in the same sweep whatever happened.
    // (The first of these barriers also makes the mbarriers' initialisation known to the whole cluster.)
    auto norms_and_votes = [&](int my_vote) {
        for (int j0 = 0; j0 < kp; j0 += nt / kLpp) {          // uniform trip count: shuffles inside
            const int j = j0 + slot;
            float acc = 0.0f;
            if (j < kp) {
#pragma unroll
                for (int f = 0; f < kJcF4; ++f) {
                    const float4 a = reinterpret_cast<const float4 *>(M + (size_t)j * kJcRows)[f * kLpp + l];
                    acc += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
                }
            }
            acc = sum4(acc);
            if (l == 0 && j < kp) {
#pragma unroll
                for (int d = 0; d < kJcCtas; ++d) cluster.map_shared_rank(npart, d)[cr * kJcLen + j] = acc;
            }
        }
        if (tid < kJcCtas) cluster.map_shared_rank(votes, tid)[cr] = my_vote;
        cluster.sync();
        for (int j = tid; j < kp; j += nt) {
            float a = 0.0f;
#pragma unroll
            for (int d = 0; d < kJcCtas; ++d) a += npart[d * kJcLen + j];
            nrm[j] = a;
        }
        int all = 0;
#pragma unroll
        for (int d = 0; d < kJcCtas; ++d) all |= votes[d];
        __syncthreads();
        return all;
    };
    // The rotation of V's columns is not needed before the next round's end (nothing reads V to take a decision),
    // so it is kept back and done while the next round's partial products are in flight.
    // Columns p, q of one round belong to one pair slot; the barrier at the end of every round orders this slot's
    // late rotation before the rotation that the columns' next owners keep back in their turn.
    int dv_p = 0, dv_q = 0;
    float dv_c = 1.0f, dv_sn = 0.0f;
    bool dv_pending = false;
    auto apply_to_v = [&]() {
        if (!kWithV || !dv_pending) return;
        float4 *vp = reinterpret_cast<float4 *>(V + (size_t)dv_p * kJcRows), *vq = reinterpret_cast<float4 *>(V + (size_t)dv_q * kJcRows);
        const float c = dv_c, sn = dv_sn;
#pragma unroll
        for (int f = 0; f < kJcF4; ++f) {
            const int i4 = (f ^ fsw) * kLpp + l;
            const float4 u = vp[i4], w = vq[i4];
            vp[i4] = make_float4(c * u.x - sn * w.x, c * u.y - sn * w.y, c * u.z - sn * w.z, c * u.w - sn * w.w);
            vq[i4] = make_float4(sn * u.x + c * w.x, sn * u.y + c * w.y, sn * u.z + c * w.z, sn * u.w + c * w.w);
        }
        dv_pending = false;
    };
    // One round's exchange: every CTA sends its kSlots partial products to all eight (itself included) with stores
    // that count off on the receiver's mbarrier of the round's parity; a receiver's phase ends when all
    // kRoundBytes are there.  Two buffers and two mbarriers are enough: a CTA sends round i + 2 only after it has
    // round i + 1 from everybody, and everybody sent round i + 1 after the CTA barrier that ends its round i, so
    // nobody still reads or waits for round i then.
    int vote = 1;
    bool failed = false;                                      // a wait ran out: stop sending and waiting, finish quickly
    unsigned it = 0;                                          // rounds so far
    for (int sweep = 0;; ++sweep) {
        const int all = norms_and_votes(vote);
        if (!(all & 1) || (all & 2) || sweep == kJacobiMaxSweeps) break;
        bool rotated = false;
        for (int r = 0; r < kp - 1; ++r, ++it) {
            const unsigned par = it & 1, phase = (it >> 1) & 1;
            if (tid == 0) mbar_expect_tx(&mbar[par], kRoundBytes);
            const bool active = slot < npairs;
            int p = 0, q = 0;
            if (active) {
                if (slot == 0) { p = kp - 1; q = r; }
                else {                                        // (r + slot) mod (kp - 1) and (r - slot) mod (kp - 1)
                    p = r + slot;
                    q = r + kp - 1 - slot;
                    p -= p >= kp - 1 ? kp - 1 : 0;
                    q -= q >= kp - 1 ? kp - 1 : 0;
                }
            }
            float4 *mp = reinterpret_cast<float4 *>(M + (size_t)p * kJcRows), *mq = reinterpret_cast<float4 *>(M + (size_t)q * kJcRows);
            float4 ap[kJcF4], aq[kJcF4];
            float g = 0.0f;
#pragma unroll
            for (int f = 0; f < kJcF4; ++f) {
                ap[f] = mp[(f ^ fsw) * kLpp + l];
                aq[f] = mq[(f ^ fsw) * kLpp + l];
                g += ap[f].x * aq[f].x + ap[f].y * aq[f].y + ap[f].z * aq[f].z + ap[f].w * aq[f].w;
            }
            const float alpha = nrm[p], beta = nrm[q];
            g = sum4(g);
            {
                float4 g4;
                g4.x = __shfl_sync(0xffffffffu, g, part_lane0);
                g4.y = __shfl_sync(0xffffffffu, g, part_lane0 + kLpp);
                g4.z = __shfl_sync(0xffffffffu, g, part_lane0 + 2 * kLpp);
                g4.w = __shfl_sync(0xffffffffu, g, part_lane0 + 3 * kLpp);
                if (sender && !failed)
                    st_async_f4(part_to + par * (unsigned)(kJcCtas * kSlots * sizeof(float)), g4, mbar_to + par * (unsigned)sizeof(uint64_t));
            }
            apply_to_v();                                     // the previous round's rotation of V, while the stores travel
            // one lane per warp polls the barrier (256 polling threads get in the way of the stores that are arriving in
            // this CTA's shared memory); the warp's other lanes take its word
            {
                int got = 1;
                if (lane == 0 && !failed) got = mbar_wait_bounded(&mbar[par], phase, status) ? 1 : 0;
                got = __shfl_sync(0xffffffffu, got, 0);
                if (!got) failed = true;
            }
            const float *pp = part + par * kJcCtas * kSlots + slot;
            g = ((pp[0] + pp[kSlots]) + (pp[2 * kSlots] + pp[3 * kSlots])) + ((pp[4 * kSlots] + pp[5 * kSlots]) + (pp[6 * kSlots] + pp[7 * kSlots]));
            if (active && alpha > 0.0f && beta > 0.0f && g * g > tol2 * alpha * beta) {
                // tangent, cosine and sine to a few units in the last place: what they leave of the pair's
                // product is far below the tolerance, and every CTA gets the same bits from the same inputs
                const float zeta = __fdividef(beta - alpha, 2.0f * g);
                const float w = fmaf(zeta, zeta, 1.0f);
                const float t = fabsf(zeta) > 1.0e8f ? __fdividef(0.5f, zeta) : __fdividef(copysignf(1.0f, zeta), fabsf(zeta) + w * rsqrtf(w));
                const float c = rsqrtf(fmaf(t, t, 1.0f)), sn = c * t;
#pragma unroll
                for (int f = 0; f < kJcF4; ++f) {
                    const float4 x = ap[f], y = aq[f];
                    mp[(f ^ fsw) * kLpp + l] = make_float4(c * x.x - sn * y.x, c * x.y - sn * y.y, c * x.z - sn * y.z, c * x.w - sn * y.w);
                    mq[(f ^ fsw) * kLpp + l] = make_float4(sn * x.x + c * y.x, sn * x.y + c * y.y, sn * x.z + c * y.z, sn * x.w + c * y.w);
                }
                dv_p = p; dv_q = q; dv_c = c; dv_sn = sn; dv_pending = true;
                if (l == 0) {
                    nrm[p] = fmaxf(alpha - t * g, 0.0f);
                    nrm[q] = beta + t * g;
                }
                rotated = rotated || g * g > kJacobiLastSweepCos * kJacobiLastSweepCos * alpha * beta;
            }
            __syncthreads();                                  // this CTA's slices are rotated before the next round reads them
        }
        vote = (__syncthreads_or(rotated) ? 1 : 0) | (__syncthreads_or(failed) ? 2 : 0);
    }
    apply_to_v();                                             // the last rotation kept back
    for (int j = tid; j < kp; j += nt) nrm[j] = sqrtf(nrm[j]);           // singular values: the norms are fresh, nothing rotated since
    __syncthreads();
    for (int j = tid; j < k; j += nt) {
        const float sj = nrm[j];
        int rk = 0;
        for (int i = 0; i < k; ++i) {
            const float si = nrm[i];
            rk += (si > sj || (si == sj && i < j)) ? 1 : 0;
        }
        rank_of[j] = rk;
        if (cr == 0) S[rk] = sj;
    }
    __syncthreads();
    for (int e = tid; e < k * kJcRows; e += nt) {
        const int j = e / kJcRows, i = row0 + e % kJcRows;
        if (i < k) {
            const float sj = nrm[j];
            const size_t o = (size_t)rank_of[j] * k + i;
            Ucol[o] = sj > 0.0f ? M[e] / sj : 0.0f;
            Vcol[o] = kWithV ? V[e] : (sj > 0.0f ? M[e] / (sj * sj) : 0.0f);
        }
    }
    cluster.sync();                                           // nobody leaves while a neighbour could still store into it
}

// The instance of the cluster kernel for a core of k columns: `lanes` threads per pair slot, with or without the
// accumulated right factor.
typedef void (*JacobiClusterFn)(const float *, int, float *, float *, float *, unsigned *);
JacobiClusterFn jacobi_cluster_fn(int k, int lanes, bool with_v) {
    if (k <= 128) return with_v ? jacobi_svd_cluster_kernel<128, 4, true> : jacobi_svd_cluster_kernel<128, 4, false>;
    if (lanes == 4) return with_v ? jacobi_svd_cluster_kernel<256, 4, true> : jacobi_svd_cluster_kernel<256, 4, false>;
    return with_v ? jacobi_svd_cluster_kernel<256, 2, true> : jacobi_svd_cluster_kernel<256, 2, false>;
}

// Launch configuration of the cluster kernel: one cluster of kJcCtas CTAs, `lanes` threads per pair slot.
void jacobi_cluster_config(cudaLaunchConfig_t *cfg, cudaLaunchAttribute *attr, int k, int lanes, cudaStream_t st) {
    cfg->gridDim = dim3(kJcCtas, 1, 1);
    cfg->blockDim = dim3(jacobi_cluster_len(k) / 2 * lanes, 1, 1);
    cfg->dynamicSmemBytes = jacobi_cluster_smem_bytes(k);
    cfg->stream = st;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kJcCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg->attrs = attr;
    cfg->numAttrs = 1;
}

// A timed span of the current call (no-ops unless the workspace's profiling is on).
int span_begin(SvdWorkspace *ws, int kind, cudaStream_t st) {
    if (!ws->profile || ws->spans >= SvdWorkspace::kMaxSpans) return -1;
    const int i = ws->spans++;
    ws->span_kind[i] = kind;
    cudaEventRecord(ws->span_ev[2 * i], st);
    return i;
}
void span_end(SvdWorkspace *ws, int i, cudaStream_t st) {
    if (i >= 0) cudaEventRecord(ws->span_ev[2 * i + 1], st);
}
cudaError_t timed_allreduce(SvdWorkspace *ws, float *buf, size_t count, cudaStream_t st) {
    const int sp = span_begin(ws, 1, st);
    const cudaError_t err = ws->allreduce(ws->allreduce_ctx, buf, count, st);
    span_end(ws, sp, st);
    return err;
}

bool alloc_f(float **p, size_t count) {
    if (cudaMalloc(reinterpret_cast<void **>(p), std::max<size_t>(count, 1) * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        *p = nullptr;
        return false;
    }
    return true;
}

// Y (rows x k, row-major) <- Y with orthonormalised columns, `passes` (1 or 2) Gram/Cholesky passes:
// one is enough to keep a power iteration stable, two give orthonormality to rounding.  `tmp` is a
// second rows x k buffer; the result ends in Y for 2 passes and in tmp for 1 (returned through *out).
// r_a / r_b (nullable) receive the triangular factors of the passes (Y_in = Y_out * r_b * r_a).
// last_factor_only: the last pass stops after its Cholesky factor (no inverse, no panel product): the caller wants the
// triangular factors only, and Y itself is left as it was (k <= kCholeskyBlockedMaxK).
cudaError_t orthonormalise(SvdWorkspace *ws, float *Y, float *tmp, int rows, int passes, float *r_a, float *r_b,
                           float **out, bool sharded_rows, cudaStream_t st, bool last_factor_only = false) {
    const int k = ws->k;
    float *src = Y, *dst = tmp;
    for (int pass = 0; pass < passes; ++pass) {
        const bool factor_only = last_factor_only && pass + 1 == passes;
        // G = src^T src
        cudaError_t err = gemm(false, false, src, k, src, k, ws->g, k, k, k, rows, nullptr, nullptr, 0, nullptr, ws->status, ws->gemm_ws,
                               ws->gemm_ws_bytes, ws->sm_count, st);
        if (err != cudaSuccess) return err;
        // a row-sharded panel: its Gram matrix is the sum of the shards' (the one exchange per QR pass);
        // every rank then factors the same k x k matrix and gets bit-identical R
        if (sharded_rows && ws->allreduce && (err = timed_allreduce(ws, ws->g, (size_t)k * k, st)) != cudaSuccess) return err;
        if (k <= kCholeskyBlockedMaxK) {
            cholesky_inverse_blocked_kernel<<<1, 1024, cholesky_blocked_smem_bytes(k), st>>>(ws->g, k, factor_only ? nullptr : ws->t,
                                                                                                pass == 0 ? r_a : r_b);
        } else if (k <= kCholeskySmemMaxK) {
            cholesky_inverse_smem_kernel<<<1, 1024, cholesky_smem_bytes(k), st>>>(ws->g, k, ws->t, pass == 0 ? r_a : r_b);
        } else {
            cholesky_inverse_kernel<<<1, 1024, 0, st>>>(ws->g, k, ws->t, pass == 0 ? r_a : r_b);
        }
        err = cudaGetLastError();
        if (err != cudaSuccess) return err;
        if (factor_only) break;
        // dst = src T
        err = gemm(true, false, src, k, ws->t, k, dst, k, rows, k, k, nullptr, nullptr, 0, nullptr, ws->status, ws->gemm_ws,
                   ws->gemm_ws_bytes, ws->sm_count, st);
        if (err != cudaSuccess) return err;
        std::swap(src, dst);
    }
    *out = src;
    return cudaSuccess;
}

// C[rows_out x k] = W * X or W^T * X for the working matrix W of the workspace.
// X is row-major unless x_colmajor (Omega).
cudaError_t times_w(SvdWorkspace *ws, const float *A, bool w_transposed_product, const float *X, bool x_colmajor, float *C,
                    cudaStream_t st) {
    // W = A (not transposed) or A^T.  "W * X" contracts over W's columns, "W^T * X" over its rows.
    const bool use_a_as_stored = (w_transposed_product == ws->transposed);   // W*X with W=A, or W^T*X with W=A^T
    const int rows_out = w_transposed_product ? ws->N : ws->M;
    const int contract = w_transposed_product ? ws->M : ws->N;
    const long ldx = x_colmajor ? contract : ws->k;
    const int sp = span_begin(ws, 0, st);
    cudaError_t err = gemm(use_a_as_stored, x_colmajor, A, ws->n, X, ldx, C, ws->k, rows_out, ws->k, contract, nullptr,
                           nullptr, 0, nullptr, ws->status, ws->gemm_ws, ws->gemm_ws_bytes, ws->sm_count, st, ws->a_absmax_valid ? ws->a_absmax_use : nullptr,
                           // what X can hold: standard normal draws from 32-bit uniforms stay below 6.7, the columns of an
                           // orthonormalised panel have norm 1 (a loose bound costs FP16 range, not precision)
                           x_colmajor ? 16.0f : 1024.0f);
    span_end(ws, sp, st);
    // row-sharded W: W^T X contracts over the sharded rows, so the shards' partial products are summed
    if (err == cudaSuccess && w_transposed_product && ws->allreduce) err = timed_allreduce(ws, C, (size_t)rows_out * ws->k, st);
    return err;
}

}  // namespace

SvdWorkspace *svd_workspace_create(int m, int n, int k, int niter, int sm_count) {
    return svd_workspace_create_sharded(m, n, k, niter, sm_count, nullptr, nullptr, 0);
}

// Row-sharded: this rank holds m of the m_total rows (all n columns); the working matrix is never the
// transpose, so that the sharded dimension is the tall one that only GEMMs touch.
SvdWorkspace *svd_workspace_create_sharded(int m, int n, int k, int niter, int sm_count, SvdAllReduce allreduce,
                                           void *allreduce_ctx, int m_total) {
    if (m <= 0 || n <= 0 || k <= 0 || niter < 0) return nullptr;
    SvdWorkspace *ws = new (std::nothrow) SvdWorkspace();
    if (!ws) return nullptr;
    ws->m = m; ws->n = n; ws->niter = niter; ws->sm_count = sm_count;
    ws->allreduce = allreduce;
    ws->allreduce_ctx = allreduce_ctx;
    ws->k = std::max(1, std::min(k, std::min(allreduce ? m_total : m, n)));
    ws->transposed = allreduce ? false : m < n;
    ws->M = ws->transposed ? n : m;
    ws->N = ws->transposed ? m : n;
    const size_t kk = (size_t)ws->k * ws->k;
    bool ok = alloc_f(&ws->omega, (size_t)ws->N * ws->k + 2) && alloc_f(&ws->y, (size_t)ws->M * ws->k) &&
              alloc_f(&ws->y2, (size_t)ws->M * ws->k) && alloc_f(&ws->z, (size_t)ws->N * ws->k) &&
              alloc_f(&ws->z2, (size_t)ws->N * ws->k) && alloc_f(&ws->g, kk) && alloc_f(&ws->w, ws->k) &&
              alloc_f(&ws->t, kk) && alloc_f(&ws->tinv1, kk) && alloc_f(&ws->tinv2, kk) && alloc_f(&ws->core, kk) &&
              alloc_f(&ws->uc, kk) && alloc_f(&ws->vc, kk);
    // split-K partials: up to 2 * SMs tiles' worth of the largest skinny product, and of the Gram matrix
    // K-split partials, and behind them room for the images of a product's second operand split beforehand
    ws->gemm_ws_bytes = std::max((size_t)ws->M * ws->k * 8, kk * 2 * (size_t)sm_count) * sizeof(float) +
                        gemm_tc_image_bytes(ws->k, ws->k <= 256 ? ws->k : 128, std::max(ws->M, ws->N)) + 256;
    ok = ok && alloc_f(&ws->gemm_ws, ws->gemm_ws_bytes / sizeof(float));
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&ws->dev_info), sizeof(int)) == cudaSuccess;
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&ws->own_status), sizeof(unsigned)) == cudaSuccess;
    ok = ok && cudaMalloc(reinterpret_cast<void **>(&ws->a_absmax), sizeof(unsigned)) == cudaSuccess;
    ok = ok && curandCreateGenerator(&ws->rng, CURAND_RNG_PSEUDO_DEFAULT) == CURAND_STATUS_SUCCESS;
    ok = ok && cusolverDnCreate(&ws->solver) == CUSOLVER_STATUS_SUCCESS;
    ok = ok && cusolverDnCreateGesvdjInfo(&ws->svdj) == CUSOLVER_STATUS_SUCCESS;
    {
        // Jacobi stops when the columns are orthogonal to this tolerance; the library's default is machine epsilon.
        // The factors only have to carry FP32 products to ~1e-6, and every sweep over a 256 x 256 core costs 0.4 ms.
        double tol = 1.0e-6;
        if (const char *e = getenv("BSQ_CORE_SVD_TOL")) {
            const double v = atof(e);
            if (v >= 1.0e-8 && v <= 1.0e-2) tol = v;          // anything else: keep the default
        }
        ok = ok && cusolverDnXgesvdjSetTolerance(ws->svdj, tol) == CUSOLVER_STATUS_SUCCESS;
    }
    if (ok) {
        int l1 = 0, l2 = 0;
        ok = cusolverDnSsyevd_bufferSize(ws->solver, CUSOLVER_EIG_MODE_VECTOR, CUBLAS_FILL_MODE_LOWER, ws->k, ws->g, ws->k,
                                         ws->w, &l1) == CUSOLVER_STATUS_SUCCESS &&
             cusolverDnSgesvdj_bufferSize(ws->solver, CUSOLVER_EIG_MODE_VECTOR, 0, ws->k, ws->k, ws->core, ws->k, ws->w,
                                          ws->uc, ws->k, ws->vc, ws->k, &l2, ws->svdj) == CUSOLVER_STATUS_SUCCESS;
        ws->lwork = std::max(1, std::max(l1, l2));
        ok = ok && alloc_f(&ws->solver_work, (size_t)ws->lwork);
    }
    {
        const char *e = getenv("BSQ_CORE_SVD");              // "cusolver": keep the library solver (A/B comparisons)
        ws->own_core_svd = ws->k <= kJacobiClusterMaxK && !(e && e[0] == 'c');
    }
    if (ok && ws->own_core_svd && ws->k <= kJacobiSingleMaxK)
        ok = cudaFuncSetAttribute(jacobi_svd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)jacobi_smem_bytes(ws->k)) == cudaSuccess;
    if (ok && ws->own_core_svd && ws->k > kJacobiSingleMaxK) {
        const char *e = getenv("BSQ_JACOBI_LPP");
        ws->jc_lanes = ws->k <= 128 || (e && atoi(e) == 4) ? 4 : 2;
        {
            const char *v = getenv("BSQ_JACOBI_V");           // 1 / 0: with / without the accumulated right factor (A/B comparisons)
            ws->jc_with_v = v ? v[0] == '1' : false;
        }
        ok = cudaFuncSetAttribute(jacobi_cluster_fn(ws->k, ws->jc_lanes, ws->jc_with_v), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)jacobi_cluster_smem_bytes(ws->k)) == cudaSuccess;
        if (ok) {
            // a device (or partition of one) that cannot place a cluster of 8 such CTAs keeps the library solver
            cudaLaunchConfig_t cfg = {};
            cudaLaunchAttribute attr[1];
            jacobi_cluster_config(&cfg, attr, ws->k, ws->jc_lanes, nullptr);
            int clusters = 0;
            const cudaError_t q = cudaOccupancyMaxActiveClusters(&clusters, jacobi_cluster_fn(ws->k, ws->jc_lanes, ws->jc_with_v), &cfg);
            if (q != cudaSuccess || clusters < 1) {
                cudaGetLastError();
                ws->own_core_svd = false;
            }
        }
    }
    if (ok && ws->k <= kCholeskyBlockedMaxK)
        ok = cudaFuncSetAttribute(cholesky_inverse_blocked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)cholesky_blocked_smem_bytes(ws->k)) == cudaSuccess;
    else if (ok && ws->k <= kCholeskySmemMaxK)
        ok = cudaFuncSetAttribute(cholesky_inverse_smem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)cholesky_smem_bytes(ws->k)) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        svd_workspace_destroy(ws);
        return nullptr;
    }
    return ws;
}

void svd_workspace_destroy(SvdWorkspace *ws) {
    if (!ws) return;
    float *bufs[] = {ws->omega, ws->y, ws->y2, ws->z, ws->z2, ws->g, ws->w, ws->t, ws->tinv1, ws->tinv2,
                     ws->core, ws->uc, ws->vc, ws->gemm_ws, ws->solver_work};
    for (float *p : bufs)
        if (p) cudaFree(p);
    if (ws->dev_info) cudaFree(ws->dev_info);
    if (ws->own_status) cudaFree(ws->own_status);
    if (ws->a_absmax) cudaFree(ws->a_absmax);
    for (cudaEvent_t e : ws->span_ev)
        if (e) cudaEventDestroy(e);
    if (ws->svdj) cusolverDnDestroyGesvdjInfo(ws->svdj);
    if (ws->solver) cusolverDnDestroy(ws->solver);
    if (ws->rng) curandDestroyGenerator(ws->rng);
    cudaGetLastError();
    delete ws;
}

// Timing of the big products and all-reduces of the calls that follow (events on the call's stream).
cudaError_t svd_workspace_profile(SvdWorkspace *ws, bool on) {
    if (!ws) return cudaErrorInvalidValue;
    if (on)
        for (cudaEvent_t &e : ws->span_ev)
            if (!e && cudaEventCreate(&e) != cudaSuccess) return cudaErrorUnknown;
    ws->profile = on;
    ws->spans = 0;
    return cudaSuccess;
}
// Durations of the last call's spans, in call order; the call's stream must have been waited for.
int svd_workspace_spans(SvdWorkspace *ws, float *ms, int *kinds, int capacity) {
    if (!ws || !ws->profile) return 0;
    int n = 0;
    for (int i = 0; i < ws->spans && n < capacity; ++i) {
        float t = 0.0f;
        if (cudaEventElapsedTime(&t, ws->span_ev[2 * i], ws->span_ev[2 * i + 1]) != cudaSuccess) { cudaGetLastError(); continue; }
        if (ms) ms[n] = t;
        if (kinds) kinds[n] = ws->span_kind[i];
        ++n;
    }
    return n;
}

// Waits for the stream and reads the workspace's own status word (calls made without a caller status word).
cudaError_t svd_workspace_finish(SvdWorkspace *ws, cudaStream_t st) {
    unsigned h = 0;
    cudaError_t err = cudaMemcpyAsync(&h, ws->own_status, sizeof(unsigned), cudaMemcpyDeviceToHost, st);
    if (err == cudaSuccess) err = cudaStreamSynchronize(st);
    if (err != cudaSuccess) return err;
    return h == 0 ? cudaSuccess : cudaErrorLaunchTimeout;
}

cudaError_t svd_lowrank(SvdWorkspace *ws, const float *d_A, float *d_U, float *d_S, float *d_V, unsigned long long seed,
                        unsigned *d_status, cudaStream_t st, unsigned long long offset, const unsigned *d_abs_bound) {
    if (!ws || !d_A || !d_U || !d_S || !d_V) return cudaErrorInvalidValue;
    const int k = ws->k;
    ws->spans = 0;
    ws->status = d_status ? d_status : ws->own_status;    // bounded waits of the tensor-core GEMMs report here
    if (!d_status && cudaMemsetAsync(ws->own_status, 0, sizeof(unsigned), st) != cudaSuccess) return cudaErrorUnknown;
    if (curandSetStream(ws->rng, st) != CURAND_STATUS_SUCCESS) return cudaErrorUnknown;
    if (cusolverDnSetStream(ws->solver, st) != CUSOLVER_STATUS_SUCCESS) return cudaErrorUnknown;
    // Omega depends on the seed and the shape only (the generator is set back to the start of the seed's sequence for
    // every call), so it is drawn once per workspace and seed and kept: re-seeding costs a kernel of its own.
    if (!ws->seeded || ws->seed != seed || ws->offset != offset) {
        if (curandSetPseudoRandomGeneratorSeed(ws->rng, seed) != CURAND_STATUS_SUCCESS) return cudaErrorUnknown;
        if (curandSetGeneratorOffset(ws->rng, offset) != CURAND_STATUS_SUCCESS) return cudaErrorUnknown;
        size_t count = (size_t)ws->N * k;
        count += count & 1;                               // the normal generator wants an even count
        if (curandGenerateNormal(ws->rng, ws->omega, count, 0.0f, 1.0f) != CURAND_STATUS_SUCCESS) return cudaErrorUnknown;
        ws->seeded = true;
        ws->seed = seed;
        ws->offset = offset;
    }

    cudaError_t err;
    float *q = nullptr, *qz = nullptr, *spare = nullptr;
    // the largest |A|, once per call: the six products with A split it into FP16 halves scaled by a power of two from it
    // (or a bound that the caller already has)
    ws->a_absmax_use = d_abs_bound ? d_abs_bound : ws->a_absmax;
    ws->a_absmax_valid = k > 128 && (d_abs_bound != nullptr ||
                                     (ws->n % 4 == 0 && reinterpret_cast<uintptr_t>(d_A) % 16 == 0 &&
                                      gemm_absmax_bits(d_A, ws->n, ws->m, ws->n, ws->a_absmax, st) == cudaSuccess));
    // Y = W Omega, Q = orth(Y).  Panels ping-pong between the two buffers of their size.
    if ((err = times_w(ws, d_A, false, ws->omega, true, ws->y, st)) != cudaSuccess) return err;
    const int last_passes = 2;
    if ((err = orthonormalise(ws, ws->y, ws->y2, ws->M, ws->niter == 0 ? last_passes : 1, nullptr, nullptr, &q, true, st)) != cudaSuccess)
        return err;
    for (int it = 0; it < ws->niter; ++it) {
        if ((err = times_w(ws, d_A, true, q, false, ws->z, st)) != cudaSuccess) return err;               // Z = W^T Q
        if ((err = orthonormalise(ws, ws->z, ws->z2, ws->N, 1, nullptr, nullptr, &qz, false, st)) != cudaSuccess) return err;
        spare = (q == ws->y) ? ws->y2 : ws->y;
        if ((err = times_w(ws, d_A, false, qz, false, spare, st)) != cudaSuccess) return err;             // Y = W Qz
        float *other = (spare == ws->y) ? ws->y2 : ws->y;
        if ((err = orthonormalise(ws, spare, other, ws->M, it + 1 == ws->niter ? last_passes : 1, nullptr, nullptr, &q, true, st)) !=
            cudaSuccess)
            return err;
    }
    // B^T = W^T Q = Q2 C with C = R2 R1.  With the cluster Jacobi kernel the right factor comes from the panel B^T
    // itself (B^T v_j / S(j)), so Q2 is never formed: the second pass only has to deliver R2.
    const bool from_panel = ws->own_core_svd && k > kJacobiSingleMaxK && !ws->jc_with_v;
    if ((err = times_w(ws, d_A, true, q, false, ws->z, st)) != cudaSuccess) return err;
    if ((err = orthonormalise(ws, ws->z, ws->z2, ws->N, 2, ws->tinv1, ws->tinv2, &qz, false, st, from_panel)) != cudaSuccess) return err;
    if (from_panel) qz = ws->z;
    if ((err = gemm(true, false, ws->tinv2, k, ws->tinv1, k, ws->core, k, k, k, k, nullptr, nullptr, 0, nullptr, ws->status, nullptr, 0,
                    ws->sm_count, st)) != cudaSuccess)
        return err;
    // The row-major C read as column-major is C^T = Vc S Uc^T: the solver's "U" is Vc, its "V" is Uc.
    if (ws->own_core_svd && k > kJacobiSingleMaxK) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        jacobi_cluster_config(&cfg, attr, k, ws->jc_lanes, st);
        const float *core = ws->core;
        float *vc = ws->vc, *uc = ws->uc;
        unsigned *status = ws->status;
        err = cudaLaunchKernelEx(&cfg, jacobi_cluster_fn(k, ws->jc_lanes, ws->jc_with_v), core, k, d_S, vc, uc, status);
        if (err != cudaSuccess) return err;
    } else if (ws->own_core_svd) {
        jacobi_svd_kernel<<<1, 512, jacobi_smem_bytes(k), st>>>(ws->core, k, d_S, ws->vc, ws->uc);
        if ((err = cudaGetLastError()) != cudaSuccess) return err;
    } else if (cusolverDnSgesvdj(ws->solver, CUSOLVER_EIG_MODE_VECTOR, 0, k, k, ws->core, k, d_S, ws->vc, k, ws->uc, k,
                                 ws->solver_work, ws->lwork, ws->dev_info, ws->svdj) != CUSOLVER_STATUS_SUCCESS) {
        return cudaErrorUnknown;
    }
    // W = (Q Vc) S (Q2 Uc)^T; both k x k factors are column-major, i.e. K-major B operands.  (from_panel: qz is the
    // panel B^T itself and column j of uc is Vc(:, j) / S(j): B^T Vc(:, j) / S(j) is the vector Q2 Uc(:, j).)
    float *d_left = ws->transposed ? d_V : d_U;            // M x k factor
    float *d_right = ws->transposed ? d_U : d_V;           // N x k factor
    if ((err = gemm(true, true, q, k, ws->vc, k, d_left, k, ws->M, k, k, nullptr, nullptr, 0, nullptr, ws->status, ws->gemm_ws, ws->gemm_ws_bytes,
                    ws->sm_count, st)) != cudaSuccess)
        return err;
    return gemm(true, true, qz, k, ws->uc, k, d_right, k, ws->N, k, k, nullptr, nullptr, 0, nullptr, ws->status, ws->gemm_ws, ws->gemm_ws_bytes,
                ws->sm_count, st);
}

size_t reconstruct_workspace_bytes(int m, int n, int k) {
    // V's images, and in front of them U diag(S) split beforehand (the persistent product of bsq_gemm.cu)
    return n > 256 ? gemm_tc_image_bytes(n, 256, k) + ((gemm_tc_a_image_bytes(m, k) + 127) & ~(size_t)127) + 1024 : 0;
}

cudaError_t reconstruct_lowrank(const float *d_U, const float *d_S, const float *d_V, int m, int n, int k,
                                const float *d_minuend, float *d_out, unsigned *d_flag, unsigned *d_status, float *d_workspace,
                                size_t workspace_bytes, int sm_count, cudaStream_t st) {
    if (!d_U || !d_S || !d_V || !d_out || m <= 0 || n <= 0 || k <= 0) return cudaErrorInvalidValue;
    // out(i, j) = sum_t (U(i, t) S(t)) V(j, t): A = U as stored with a per-k scale, B = V^T (K-major)
    return gemm(true, true, d_U, k, d_V, k, d_out, n, m, n, k, d_S, d_minuend, n, d_flag, d_status, d_workspace, workspace_bytes, sm_count, st);
}

}  // namespace bsq
