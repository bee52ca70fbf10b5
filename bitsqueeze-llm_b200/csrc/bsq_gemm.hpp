// Argument block shared by the two GEMM kernels of the low-rank stages (bsq_gemm.cu: FP32 pipes,
// bsq_gemm_tc.cu: tcgen05 tensor cores with 3xTF32 splitting).
#pragma once

#include <cuda_runtime.h>

namespace bsq {

// C[M x N] = opA[M x K] * opB[K x N]; see bsq_gemm.cu for the operand conventions.
struct GemmArgs {
    const float *A, *B;
    float *C;                  // output, or partial tiles when splits > 1
    int M, N, K;
    long lda, ldb, ldc;
    const float *kscale;       // nullable: opA(i, kk) *= kscale[kk]
    int splits;                // K splits (grid.z)
    int k_per_split;           // multiple of BK
    long split_stride;         // elements between partial results
    const float *minuend;      // nullable (only without splits): C = minuend - acc
    long ldm;
    unsigned *flag;            // nullable: |= 1 when some |C| > FLT_EPSILON (with minuend)
    int n_tile;                // tensor-core kernel: columns per CTA (a multiple of 16, <= 256); grid.y tiles N
    const float4 *b_image;     // tensor-core kernel, nullable: room for B split beforehand (gemm_tc_image_bytes, 128-byte aligned)
    int a_stages, b_stages;    // with b_image: ring lengths in shared memory (gemm_tc_image_rings / gemm_tc_tma_rings)
    int raw_stages;            // TMA-fed kernel, A contiguous along M: slots of boxes as they come from memory
    bool use_tma;              // with b_image: the kernel that brings A in by TMA (bsq_gemm_tma.cu)
    bool persistent;           // with use_tma, no K split: one CTA per SM walks over all tiles (wide products)
    float *a_image;            // with persistent and A contiguous along K, nullable: room for A (times kscale) split beforehand into
                               // two row-major a_image_rows x K matrices, hi then lo (gemm_tc_a_image_bytes): a small A that every
                               // column tile reads again then comes in by TMA ready for the tensor core, and nobody splits in the kernel
    int a_image_rows;          // M rounded up to the tile height
    bool wide_tiles;           // with a_image: 256-column tiles whose three products share one accumulator (two accumulator sets
                               // then fit tensor memory), their epilogue shared by the warps that have nothing to split: per
                               // column of C half as many barrier waits, descriptors and commits for the one thread that issues
                               // the MMAs, which is what bounds a product with a short K
    int sm_count;
    bool f16;                      // TMA-fed kernel: operands split into two FP16 halves (bsq_gemm_tc.cuh) instead of two TF32
    const unsigned *a_absmax_bits; // halves; device words with the bits of the largest |A| and |B| (finite), from which the
    const unsigned *b_absmax_bits; // power-of-two scales of the split come
    float b_scale_fixed;           // > 0: the scale of B given by the caller (from a bound it knows) instead of *b_absmax_bits
    bool lo_unscaled;              // the low halves are fp16(x s - hi) without the factor 2^11, so that all three products of a
                                   // term can share ONE accumulator (the persistent product's 256-column tiles); elements more
                                   // than 2^18 below the operand's largest then lose bits of their low half
};

// Tensor-core path: true if the shape qualifies (N a multiple of 16, 16-byte aligned operands with leading
// dimensions that are multiples of 4; the fused scale / minuend epilogue only without K splits).  Launches with
// grid (M tiles, N tiles, splits).
bool gemm_tc_eligible(const GemmArgs &g, bool a_kmajor, bool b_kmajor);
// With g.b_image set, B is first split into per-chunk hi / lo images there (one small kernel) and the product kernel
// fetches them by bulk copies; gemm_tc_image_bytes is the room that takes.
size_t gemm_tc_image_bytes(int N, int n_tile, int K);
size_t gemm_tc_a_image_bytes(int M, int K);
// bits of the largest |x| of a rows x cols matrix into *d_out (the scale of the FP16 split comes from it)
cudaError_t gemm_absmax_bits(const float *x, long ld, int rows, int cols, unsigned *d_out, cudaStream_t stream);
int gemm_tc_image_ctas_per_sm(int n_tile);
void gemm_tc_image_rings(int n_tile, int *sa, int *nb);
cudaError_t gemm_tc_launch(const GemmArgs &g, bool a_kmajor, bool b_kmajor, unsigned *status, cudaStream_t stream);

// The TMA-fed kernel (bsq_gemm_tma.cu): A in either orientation, B split into images beforehand (g.b_image filled by
// the caller of gemm_tc_tma_launch), one CTA per SM.  gemm_tc_tma_usable looks at the shape, the alignment and the
// BSQ_GEMM_TMA switch; gemm_tc_tma_rings gives the ring lengths for raw_stages / a_stages / b_stages.
bool gemm_tc_tma_enabled();
bool gemm_tc_tma_usable(const GemmArgs &g, bool a_kmajor);
void gemm_tc_tma_rings(int n_tile, bool a_kmajor, int *nraw, int *nr, int *nb, bool f16 = false);
cudaError_t gemm_tc_tma_launch(const GemmArgs &g, bool a_kmajor, unsigned *status, cudaStream_t stream);

}  // namespace bsq
