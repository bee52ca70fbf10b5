/*
 * bitsqz_llm -- C ABI of the compress/decompress hot path (plain pointers and sizes only).
 *
 * The reference library has C++ linkage (include/bitsqz_llm.hpp has no extern "C" and
 * overloads bitsqz_llm_compress), so a foreign-function binding cannot name its symbols
 * portably.  This header gives every entry point of that interface, and every stage function
 * of the reference's four CUDA modules that the path is built from, a C name.  The library
 * exports both sets: the C++ symbols for callers that relink, these for cgo / ctypes / JNI.
 *
 * Conventions: int results are 0 on success and 1 on failure (the reference's convention);
 * nothing throws; `d_` pointers are device memory of the calling thread's current CUDA device;
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream); stage functions
 * only enqueue work on `stream` and do not synchronise.  Enum arguments are passed as int with
 * the values of bitsqz_llm.hpp: method -1 none, 10 NF4_DQ, 11 NF4; location 0 host, 1 device.
 */
#ifndef BITSQZ_LLM_C_H
#define BITSQZ_LLM_C_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

struct bitsqz_llm_array;                /* 200-byte header + payload, see bitsqz_llm.hpp */
struct bitsqz_llm_compress_profile;     /* seven doubles, see bitsqz_llm.hpp */

/* ---- the public interface (include/bitsqz_llm.hpp:95-141 of the reference) ---------------- */

/* bitsqz_llm_compress_initialize, include/bitsqz_llm.hpp:95-105 */
int bsq_compress_initialize(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio,
                            float error_correction_topk_ratio, int svd_ranks, int svd_niters, int svd_uv_format,
                            int svd_s_format, int quantization_only_format, int input_location);
/* bitsqz_llm_compress_release, :107 */
void bsq_compress_release(void);
/* bitsqz_llm_decompress_initialize, :109-117 */
int bsq_decompress_initialize(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio,
                              float error_correction_topk_ratio, int svd_ranks, int svd_uv_format, int svd_s_format,
                              int quantization_only_format);
/* bitsqz_llm_decompress_release, :119 */
void bsq_decompress_release(void);
/* bitsqz_llm_compress, :121-124.  *out must be NULL on entry; profile may be NULL. */
int bsq_compress(const float *row_major_matrix, struct bitsqz_llm_array **out, void *profile);
/* bitsqz_llm_decompress, :132-135 */
int bsq_decompress(const struct bitsqz_llm_array *compressed, float *d_dst, uint32_t dst_num_elements);
/* bitsqz_llm_get_packed_size, :137 */
uint64_t bsq_get_packed_size(const struct bitsqz_llm_array *compressed);
/* load_bitsqz_llm_from_buffer, :139 */
struct bitsqz_llm_array *bsq_load_from_buffer(const void *buffer, uint64_t buffer_size);
/* bitsqz_llm_free, :141 */
void bsq_free(struct bitsqz_llm_array *compressed);

/* ---- per-row top-k (modules/topk_cuda/include/topk_cuda.cuh:47-107) ----------------------- */

/* topk_compute_num_topk_columns, topk_cuda.cuh:47; -1 for a ratio outside [0, 1] */
int bsq_topk_num_columns(uint16_t num_columns, float topk_ratio);
/* topk_extraction (d_residual NULL) / topk_separation (d_residual = zeroed copy, may equal d_in),
 * topk_cuda.cuh:68-76.  d_idx, d_val: [rows][k], ordered by (|x| descending, column ascending).
 * d_status: one device word that receives error bits (0 = fine); may be NULL. */
int bsq_topk_rows(const float *d_in, float *d_residual, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                  float *d_val, uint32_t *d_status, void *stream);
/* topk_apply, topk_cuda.cuh:83-86: dense[row, idx] += val */
int bsq_topk_apply(const uint16_t *d_idx, const float *d_val, uint32_t rows, uint32_t cols, uint32_t k, float *d_dense,
                   uint32_t *d_status, void *stream);

/* ---- NF4 / NF4_DQ (modules/quantization_cuda/include/quantization_cuda/quantization_cuda.cuh:58-112) */

/* quantization_cuda_compress with an NF4 array, quantization_cuda.cuh:86-89.  d_scales: ceil(n/64)
 * floats, d_data: ceil(n/2) bytes, d_deq_out: NULL or n floats (dequantised values, may equal d_x). */
int bsq_nf4_quantize(const float *d_x, uint64_t n, float *d_scales, uint8_t *d_data, float *d_deq_out, void *stream);
/* bytes of device scratch bsq_nf4dq_quantize needs for n elements */
size_t bsq_nf4dq_scratch_bytes(uint64_t n);
/* quantization_cuda_compress with an NF4_DQ array.  d_dq: 1 float, d_scale_codes: ceil(n/64) bytes. */
int bsq_nf4dq_quantize(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                       float *d_deq_out, void *d_scratch, void *stream);
/* NF4_DQ quantiser for callers that cannot allocate device memory.  It has no counterpart in the
 * reference (there every quantiser context owns cudaMalloc'ed scratch).  Some callers hold a fixed
 * memory budget carved out at start-up, or run where an allocation would stall or break them
 * (inside a serving loop that must not touch the allocator, under a memory pool that owns the whole
 * device); this entry point needs only the caller's input and output buffers.  Its scratch (one
 * float per 64-element block) is a fixed array inside the library, so n is limited to
 * bsq_nf4dq_quantize_static_max_elements() (2^24 elements, 1 MiB of scratch per device); larger n
 * returns 1.  The first call on a device looks up the array's device address and should happen
 * outside stream capture.  All calls on a device share the array: do not let two of them overlap
 * on the GPU.  Results are identical to bsq_nf4dq_quantize. */
uint64_t bsq_nf4dq_quantize_static_max_elements(void);
int bsq_nf4dq_quantize_static(const float *d_x, uint64_t n, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                              void *stream);
/* quantization_cuda_decompress, quantization_cuda.cuh:91-94 */
int bsq_nf4_dequantize(const float *d_scales, const uint8_t *d_data, uint64_t n, float *d_out, void *stream);
int bsq_nf4dq_dequantize(const float *d_dq, const uint8_t *d_scale_codes, const uint8_t *d_data, uint64_t n,
                         float *d_out, void *stream);
/* quantization_cuda_decompress followed by topk_apply on the same rows x cols matrix (the no-SVD branch of
 * bitsqz_llm_decompress, src/bitsqz_llm.cu:1304-1393) in one pass over the output: d_out = dequantise(...) and then
 * d_out[row, idx] += val for the row's k entries.  method 11: d_scales_f32; method 10: d_dq and d_scale_codes.
 * Columns out of range are skipped and reported in d_status (bit 1), as by bsq_topk_apply. */
int bsq_dequantize_add_topk(int method, const float *d_scales_f32, const float *d_dq, const uint8_t *d_scale_codes,
                            const uint8_t *d_data, uint32_t rows, uint32_t cols, const uint16_t *d_idx, const float *d_val,
                            uint32_t k, float *d_out, uint32_t *d_status, void *stream);

/* ---- fused outlier separation + quantiser: the no-SVD branch of bitsqz_llm_compress
 * (src/bitsqz_llm.cu:1045-1056,1183-1195) as one stage --------------------------------------- */
int bsq_frontend_supported(uint32_t rows, uint32_t cols, uint32_t k);
/* d_scratch of bsq_frontend_quantize.  Its fourth 32-bit word carries a selection bound from one call to the next
 * on the same scratch area (a speed-up for runs of alike matrices; results never depend on it); zero the first 16
 * bytes once after allocating it.  Calls that overlap on the GPU need scratch areas of their own. */
size_t bsq_frontend_scratch_bytes(uint32_t rows, uint32_t cols);
int bsq_frontend_quantize(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k, uint16_t *d_idx,
                          float *d_val, float *d_scales_f32, float *d_dq, uint8_t *d_scale_codes, uint8_t *d_data,
                          void *d_scratch, uint32_t *d_status, void *stream);

/* Same call, bracketed by CUDA events on `stream`: ms_pass[0] = pass 1 (selection + block maxima, or the
 * whole NF4 kernel), ms_pass[1] = pass 2 (NF4_DQ encode; 0 for NF4).  Synchronises; for measurement. */
int bsq_frontend_quantize_timed(int method, const float *d_in, uint32_t rows, uint32_t cols, uint32_t k,
                                uint16_t *d_idx, float *d_val, float *d_scales_f32, float *d_dq,
                                uint8_t *d_scale_codes, uint8_t *d_data, void *d_scratch, uint32_t *d_status,
                                void *stream, float *ms_pass);

/* ---- error stage (src/bitsqz_llm.cu:164-184,375-423): e = a - b, *d_flag |= any(|e| > FLT_EPSILON) */
int bsq_residual_error(const float *d_a, const float *d_b, uint64_t n, float *d_e, uint32_t *d_flag, void *stream);

/* ---- low-rank stages ------------------------------------------------------------------------- */

/* svd_lowrank_cuda_initialize + svd_lowrank_cuda + svd_lowrank_cuda_release
 * (modules/svd_lowrank_cuda/include/svd_lowrank_cuda/svd_lowrank_cuda.cuh:54-68) in one call:
 * rank-k randomized SVD of the row-major m x n matrix d_A.  d_U: m x k, d_S: k, d_V: n x k. */
int bsq_svd_lowrank(const float *d_A, int m, int n, int k, int niter, unsigned long long seed, float *d_U, float *d_S,
                    float *d_V, void *stream);
/* The same with the random matrix taken `offset` values into the generator's sequence for `seed` (bsq_svd_lowrank is
 * offset 0): the range finder's random matrix is the N_work x k block of XORWOW normals that starts there. */
int bsq_svd_lowrank_at(const float *d_A, int m, int n, int k, int niter, unsigned long long seed, unsigned long long offset,
                       float *d_U, float *d_S, float *d_V, void *stream);
/* reconstruct_lowrank_cuda (reconstruct_lowrank_cuda.cuh:73-78): d_out = (U diag(S)) V^T.
 * d_minuend non-NULL: d_out = d_minuend - (U diag(S)) V^T and *d_flag |= any(|d_out| > FLT_EPSILON).
 * d_status (nullable) receives bit 0 if a bounded wait inside the product kernel gave up (d_out is then incomplete). */
int bsq_reconstruct(const float *d_U, const float *d_S, const float *d_V, int m, int n, int k, const float *d_minuend,
                    float *d_out, uint32_t *d_flag, uint32_t *d_status, void *stream);

/* The FP32 matrix product inside the two stages above, where the reference calls cublasSgemm
 * (svd_lowrank_cuda.cu:293-309, reconstruct_lowrank_cuda.cu:46-61): C[M x N] = opA[M x K] * opB[K x N], all row-major
 * device arrays.  a_kmajor: opA(i,kk) = A[i*lda+kk], else A[kk*lda+i]; b_kmajor: opB(kk,j) = B[j*ldb+kk], else B[kk*ldb+j].
 * d_workspace (nullable) allows a deterministic split of K and, above 128 columns, holds opB split once into the
 * tensor cores' operand format (room for 8 K N bytes makes that possible).  allow_tensor_cores = 0 keeps the product on the FP32 pipes;
 * otherwise products with N a multiple of 16 up to 256 run as 3xTF32 on the tensor cores (FP32-level accuracy).
 * d_status (nullable) receives bit 0 if a bounded wait inside the tensor-core kernel gave up.  Exported so that the
 * kernel can be tested and timed on its own. */
int bsq_gemm(int a_kmajor, int b_kmajor, const float *d_A, long lda, const float *d_B, long ldb, float *d_C, long ldc, int M,
             int N, int K, float *d_workspace, size_t workspace_bytes, int allow_tensor_cores, uint32_t *d_status, void *stream);

/* The same product when the caller knows an upper bound of |A| (a device word holding the bits of a finite, non-negative
 * float): 256-column products on the TMA-fed kernel then split their operands into two FP16 halves, scaled by powers of
 * two taken from that bound and from the largest |B|, instead of two TF32 halves (same accuracy class, twice the
 * tensor rate); every other shape runs as in bsq_gemm.  A bound below the true maximum overflows FP16: the result
 * holds Inf / NaN then. */
int bsq_gemm_bounded(int a_kmajor, int b_kmajor, const float *d_A, long lda, const float *d_B, long ldb, float *d_C, long ldc, int M,
                     int N, int K, float *d_workspace, size_t workspace_bytes, const uint32_t *d_a_absmax_bits, uint32_t *d_status,
                     void *stream);

/* ---- row-sharded SVD over several GPUs, one process per GPU (no counterpart in the reference, which is
 * single-GPU; the sharded form of svd_lowrank_cuda, svd_lowrank_cuda.cuh:54-68).  A is split by rows; each
 * rank passes its m_local x n slice and receives its rows of U; S and V are replicated and bit-identical
 * on all ranks.  Collectives: NCCL all-reduce of the k x k Gram matrices and the n x k partial products.
 * Rank 0 makes the 128-byte id and hands it to the others (any side channel), then every rank creates
 * its communicator with the device it will use current. */
int bsq_shard_unique_id(void *out, size_t bytes);
void *bsq_shard_comm_create(const void *unique_id, int rank, int world);
void bsq_shard_comm_destroy(void *comm);
int bsq_svd_lowrank_sharded(void *comm, const float *d_A_local, int m_local, int m_total, int n, int k, int niter,
                            unsigned long long seed, float *d_U_local, float *d_S, float *d_V, void *stream);
/* The same with a workspace that lives across calls (created once per communicator and shape; every rank creates its
 * own, with its own m_local).  bsq_shard_svd_run waits for `stream` before it returns (it checks the kernels' status).
 * bsq_shard_compress runs the SVD and returns THIS rank's shard as an ordinary packed object (FP32 sections: its
 * m_local rows of U, and the replicated S and V; m_local and n at most 65 535), which the unchanged
 * bitsqz_llm_decompress -- initialised with (m_local, n, 0, 0, k, none, none, none) -- turns back into the shard's
 * rows: a matrix with more rows than one object can hold (include/bitsqz_llm.hpp:56, uint16_t num_rows, of the
 * reference) becomes one object per shard.  Release it with bsq_free.
 * bsq_shard_svd_profile / _read: as bsq_lane_profile; kind 0 = product with the local rows, kind 1 = all-reduce. */
typedef struct bsq_shard_svd bsq_shard_svd_t;
bsq_shard_svd_t *bsq_shard_svd_create(void *comm, int m_local, int m_total, int n, int k, int niter);
void bsq_shard_svd_destroy(bsq_shard_svd_t *handle);
int bsq_shard_svd_run(bsq_shard_svd_t *handle, const float *d_A_local, unsigned long long seed, float *d_U_local, float *d_S,
                      float *d_V, void *stream);
int bsq_shard_compress(bsq_shard_svd_t *handle, const float *d_A_local, unsigned long long seed, struct bitsqz_llm_array **out,
                       void *stream);
/* 1 if this communicator's k x k all-reduces run as one kernel over peer memory (ranks that can map each other's memory
 * through CUDA IPC: the GPUs of one node), 0 if they go through NCCL like the large ones (BSQ_SHARD_PEER=0 forces that) */
int bsq_shard_uses_peer_exchange(void *comm);
int bsq_shard_svd_profile(bsq_shard_svd_t *handle, int on);
int bsq_shard_svd_profile_read(bsq_shard_svd_t *handle, float *ms, int *kinds, int capacity);

/* ---- lanes and batches: several independent matrices in flight on one device -----------------------------------
 * No counterpart in the reference, whose compress and decompress calls are synchronous and keep one pair of runtimes
 * per process (src/bitsqz_llm.cu:981-1302, 1304-1393 are the calls these split in two).  A lane owns a compress and a
 * decompress runtime of one configuration on the device that was current when it was created, with a CUDA stream of
 * its own.  "begin" enqueues a whole call on that stream and returns; "end" waits for the stream and finishes the
 * result.  Calls begun on different lanes overlap on the GPU.  One compress or decompress call per lane at a time;
 * lanes are not thread-safe (one host thread per lane, or one for all).
 *
 * Results of compress go to a pooled pinned host object exactly like bitsqz_llm_compress (d_packed NULL) or, with
 * d_packed set, to a device buffer of at least bsq_lane_packed_capacity() bytes that receives the same bytes in the
 * same layout (200-byte header, then the payload): copying packed_size bytes from it to the host gives a buffer that
 * load_bitsqz_llm_from_buffer accepts.  For such a device-resident object bsq_lane_compress_end fills *device_header,
 * a host copy of the header whose `payload` member is the DEVICE address of the payload; pass that header to
 * bsq_lane_decompress_begin with payload_on_device = 1. */
typedef struct bsq_lane bsq_lane_t;
bsq_lane_t *bsq_lane_create(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio, float error_correction_topk_ratio,
                            int svd_ranks, int svd_niters, int svd_uv_format, int svd_s_format, int quantization_only_format);
void bsq_lane_destroy(bsq_lane_t *lane);
/* upper bound of the packed size (header + payload) of this lane's configuration */
uint64_t bsq_lane_packed_capacity(bsq_lane_t *lane);
/* the lane's cudaStream_t (compress side or decompress side), e.g. to make other work wait for it with an event */
void *bsq_lane_stream(bsq_lane_t *lane, int decompress_side);
/* matrix: host (input_location 0; pinned memory makes the copy asynchronous) or device (1) */
int bsq_lane_compress_begin(bsq_lane_t *lane, const float *matrix, int input_location, void *d_packed, uint64_t capacity);
/* host object: *out (must be NULL on entry) receives it, release with bsq_free; device object: device_header (nullable) */
int bsq_lane_compress_end(bsq_lane_t *lane, struct bitsqz_llm_array **out, struct bitsqz_llm_array *device_header,
                          uint64_t *packed_size);
int bsq_lane_decompress_begin(bsq_lane_t *lane, const struct bitsqz_llm_array *header, int payload_on_device, float *d_dst,
                              uint64_t dst_num_elements);
int bsq_lane_decompress_end(bsq_lane_t *lane);
/* Measurement aid for lanes with an SVD stage: with `on`, the compress calls that follow bracket every product with
 * the big matrix (kind 0) by CUDA events on the lane's stream; after bsq_lane_compress_end, bsq_lane_profile_read
 * returns how many spans the last call had and their milliseconds, in call order. */
int bsq_lane_profile(bsq_lane_t *lane, int on);
int bsq_lane_profile_read(bsq_lane_t *lane, float *ms, int *kinds, int capacity);

/* A batch is `lanes` lanes (1..16) of one configuration; matrix i of a call runs on lane i % lanes, so up to `lanes`
 * matrices are in flight.  bsq_batch_compress: d_packed NULL -> outs[i] receive host objects (bsq_free each);
 * d_packed set -> object i goes to the device buffer d_packed[i] (capacity bytes each), device_headers[i] and
 * packed_sizes[i] (both nullable arrays) describe it.  Matrices are independent, results do not depend on the lane. */
typedef struct bsq_batch bsq_batch_t;
bsq_batch_t *bsq_batch_create(uint16_t num_rows, uint16_t num_columns, float outlier_topk_ratio, float error_correction_topk_ratio,
                              int svd_ranks, int svd_niters, int svd_uv_format, int svd_s_format, int quantization_only_format,
                              int lanes);
void bsq_batch_destroy(bsq_batch_t *batch);
int bsq_batch_lanes(bsq_batch_t *batch);
bsq_lane_t *bsq_batch_lane(bsq_batch_t *batch, int i);
int bsq_batch_compress(bsq_batch_t *batch, const float *const *matrices, int count, int input_location, void *const *d_packed,
                       uint64_t capacity, struct bitsqz_llm_array **outs, struct bitsqz_llm_array *device_headers,
                       uint64_t *packed_sizes);
int bsq_batch_decompress(bsq_batch_t *batch, const struct bitsqz_llm_array *const *headers, int count, int payload_on_device,
                         float *const *d_dsts, uint64_t dst_num_elements);

/* Test hook (no counterpart in the reference): the next bsq_compress (which = 0) or bsq_decompress (which = 1) on the
 * current device starts with `bits` set in its device status word, as if a kernel had reported them; that call must
 * return 1.  Lets the error path be tested without making a kernel fail. */
void bsq_test_inject_status(int which, uint32_t bits);

/* library build tag: "sm_100a" plus the compile date */
const char *bsq_build_info(void);

#ifdef __cplusplus
}
#endif
#endif /* BITSQZ_LLM_C_H */
