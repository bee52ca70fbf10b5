/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the bitsqz_llm compress/decompress
 * hot path.  Nothing in the shipped library links, loads or calls this file; only
 * the test-suite, the smoke check and the bench's CPU-baseline leg may use it, and
 * there only as the checker / the timed baseline.
 *
 * Every function restates, in plain C, the arithmetic of one reference routine and
 * cites the reference file:line it follows (paths relative to the reference tree).
 * Parity pins: the NF4 / NF4_DQ routines are checked byte-for-byte against the
 * reference's own CPU library (legacy_modules/quantization, compiled unmodified into
 * oracle/_ref) and against fixtures generated from it (tests/golden); the top-k,
 * reconstruct and packing routines have no CPU twin in the reference and are checked
 * against the reference's CUDA build on a GPU box and against the properties the
 * reference's own tests assert.
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp -ffp-contract=off -shared -fPIC).
 * -ffp-contract=off matters: the reference CPU build (g++ -O3, generic x86-64) never
 * fuses x*inv - level into an FMA, and neither may this file.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define BSQ_BLOCK 64u
#define BSQ_E4M3_MAX 448.0f

/* quantization_cuda.cu:20-37 == nf4_impl.cpp:3-20 == nf4_dq_impl.cpp:7-24 */
static const float kLevels[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

/* nf4_impl.cpp:73-86 / quantization_cuda.cu:43-58: non-finite -> 0, then the first
 * level (lowest index) that attains the minimum of |v - L[i]| in FP32. */
uint8_t bsq_oracle_nf4_code(float v) {
    if (!isfinite(v)) v = 0.0f;
    int best = 0;
    float best_err = fabsf(v - kLevels[0]);
    for (int i = 1; i < 16; ++i) {
        float err = fabsf(v - kLevels[i]);
        if (err < best_err) { best_err = err; best = i; }
    }
    return (uint8_t)best;
}

float bsq_oracle_nf4_level(uint8_t code) { return kLevels[code & 0xF]; }

/* nf4_dq_impl.cpp:83-112 / quantization_cuda.cu:64-109 */
uint8_t bsq_oracle_e4m3_encode(float x) {
    if (!isfinite(x)) x = (x < 0.0f) ? -BSQ_E4M3_MAX : BSQ_E4M3_MAX;
    const int sign = signbit(x) ? 1 : 0;
    float ax = fabsf(x);
    if (ax == 0.0f) return (uint8_t)(sign << 7);
    if (ax > BSQ_E4M3_MAX) ax = BSQ_E4M3_MAX;
    int e2 = 0;
    const float frac = frexpf(ax, &e2);          /* ax = frac * 2^e2, frac in [0.5,1) */
    int efield = e2 - 1 + 7;
    if (efield <= 0) {                            /* subnormal range: multiples of 2^-9 */
        int m = (int)lrintf(ax * 512.0f);
        if (m > 7) m = 7;
        return (uint8_t)((sign << 7) | (m & 7));
    }
    int m = (int)lrintf((frac * 2.0f - 1.0f) * 8.0f);
    if (m > 7) { m = 0; efield += 1; }
    if (efield >= 16) { efield = 15; m = 7; }
    return (uint8_t)((sign << 7) | ((efield & 0xF) << 3) | (m & 7));
}

/* nf4_dq_impl.cpp:114-129 / quantization_cuda.cu:111-128 */
float bsq_oracle_e4m3_decode(uint8_t c) {
    const int sign = (c >> 7) & 1, efield = (c >> 3) & 0xF, m = c & 7;
    float r;
    if (efield == 0) r = ((float)m / 8.0f) * ldexpf(1.0f, -6);
    else r = (1.0f + (float)m / 8.0f) * ldexpf(1.0f, efield - 7);
    return sign ? -r : r;
}

static float block_absmax_or_one(const float *x, uint64_t start, uint64_t n) {
    /* nf4_impl.cpp:110-118: non-finite inputs count as 0; empty/all-zero block -> 1.0 */
    const uint64_t remain = (start + BSQ_BLOCK <= n) ? BSQ_BLOCK : (n - start);
    float amax = 0.0f;
    for (uint64_t i = 0; i < remain; ++i) {
        float v = x[start + i];
        if (!isfinite(v)) v = 0.0f;
        const float av = fabsf(v);
        if (av > amax) amax = av;
    }
    return amax > 0.0f ? amax : 1.0f;
}

static void encode_block(const float *x, uint64_t start, uint64_t n, float scale, uint8_t *data) {
    /* nf4_impl.cpp:119-131: inv = 1/scale (IEEE divide), v = x*inv (IEEE multiply),
     * even flat index -> high nibble, odd -> low nibble. */
    const uint64_t remain = (start + BSQ_BLOCK <= n) ? BSQ_BLOCK : (n - start);
    const float inv = 1.0f / scale;
    for (uint64_t i = 0; i < remain; ++i) {
        const float v = x[start + i] * inv;
        const uint8_t code = bsq_oracle_nf4_code(v) & 0xF;
        const uint64_t p = (start + i) >> 1;
        if (((start + i) & 1) == 0) data[p] = (uint8_t)(code << 4);
        else data[p] |= code;
    }
}

/* nf4_compress, nf4_impl.cpp:92-135.  scales: ceil(n/64) floats, data: ceil(n/2) bytes. */
int bsq_oracle_nf4_quantize(const float *x, uint64_t n, float *scales, uint8_t *data) {
    if (!x || !n || !scales || !data) return 1;
    const uint64_t nb = (n + BSQ_BLOCK - 1) / BSQ_BLOCK;
    memset(data, 0, (size_t)((n + 1) / 2));
#pragma omp parallel for schedule(static)
    for (uint64_t b = 0; b < nb; ++b) {
        const float s = block_absmax_or_one(x, b * BSQ_BLOCK, n);
        scales[b] = s;
        encode_block(x, b * BSQ_BLOCK, n, s, data);
    }
    return 0;
}

/* nf4_decompress, nf4_impl.cpp:137-164 / quantization_cuda.cu:287-310 */
int bsq_oracle_nf4_dequantize(const float *scales, const uint8_t *data, uint64_t n, float *out) {
    if (!scales || !data || !n || !out) return 1;
    const uint64_t nb = (n + BSQ_BLOCK - 1) / BSQ_BLOCK;
#pragma omp parallel for schedule(static)
    for (uint64_t b = 0; b < nb; ++b) {
        float s = scales[b];
        if (s == 0.0f || !isfinite(s)) s = 1.0f;
        const uint64_t start = b * BSQ_BLOCK;
        const uint64_t remain = (start + BSQ_BLOCK <= n) ? BSQ_BLOCK : (n - start);
        for (uint64_t i = 0; i < remain; ++i) {
            const uint8_t byte = data[(start + i) >> 1];
            const uint8_t code = ((start + i) & 1) ? (byte & 0xF) : (byte >> 4);
            out[start + i] = s * kLevels[code];
        }
    }
    return 0;
}

/* _quantize_nf4_dq, nf4_dq_impl.cpp:161-225 (CUDA twin quantization_cuda.cu:186-285):
 * dq = max_b(absmax_or_one_b)/448 (1.0 when the max is 0), scale code = e4m3(absmax/dq),
 * effective scale = dq*decode(code) (1.0 when 0 or non-finite). */
int bsq_oracle_nf4dq_quantize(const float *x, uint64_t n, float *dq_out, uint8_t *scale_codes,
                              uint8_t *data) {
    if (!x || !n || !dq_out || !scale_codes || !data) return 1;
    const uint64_t nb = (n + BSQ_BLOCK - 1) / BSQ_BLOCK;
    float *amax = (float *)malloc((size_t)nb * sizeof(float));
    if (!amax) return 1;
    memset(data, 0, (size_t)((n + 1) / 2));
#pragma omp parallel for schedule(static)
    for (uint64_t b = 0; b < nb; ++b) amax[b] = block_absmax_or_one(x, b * BSQ_BLOCK, n);
    float gmax = 0.0f;                       /* choose_dq_scale, nf4_dq_impl.cpp:149-159 */
    for (uint64_t b = 0; b < nb; ++b) {
        if (!isfinite(amax[b])) continue;
        if (fabsf(amax[b]) > gmax) gmax = fabsf(amax[b]);
    }
    float dq = (gmax == 0.0f) ? 1.0f : gmax / BSQ_E4M3_MAX;
    if (dq == 0.0f) dq = 1.0f;
    *dq_out = dq;
#pragma omp parallel for schedule(static)
    for (uint64_t b = 0; b < nb; ++b) {
        const uint8_t c = bsq_oracle_e4m3_encode(amax[b] / dq);
        scale_codes[b] = c;
        float s = dq * bsq_oracle_e4m3_decode(c);
        if (s == 0.0f || !isfinite(s)) s = 1.0f;
        encode_block(x, b * BSQ_BLOCK, n, s, data);
    }
    free(amax);
    return 0;
}

/* nf4_dq_decompress, nf4_dq_impl.cpp:243-275 / quantization_cuda.cu:312-341 */
int bsq_oracle_nf4dq_dequantize(float dq, const uint8_t *scale_codes, const uint8_t *data,
                                uint64_t n, float *out) {
    if (!scale_codes || !data || !n || !out) return 1;
    /* quantization_cuda.cu:325-328 guards dq itself; the CPU twin does not, and the two
     * agree for every dq a compressor can emit (dq is never 0 or non-finite there). */
    if (dq == 0.0f || !isfinite(dq)) dq = 1.0f;
    const uint64_t nb = (n + BSQ_BLOCK - 1) / BSQ_BLOCK;
#pragma omp parallel for schedule(static)
    for (uint64_t b = 0; b < nb; ++b) {
        float s = dq * bsq_oracle_e4m3_decode(scale_codes[b]);
        if (s == 0.0f || !isfinite(s)) s = 1.0f;
        const uint64_t start = b * BSQ_BLOCK;
        const uint64_t remain = (start + BSQ_BLOCK <= n) ? BSQ_BLOCK : (n - start);
        for (uint64_t i = 0; i < remain; ++i) {
            const uint8_t byte = data[(start + i) >> 1];
            const uint8_t code = ((start + i) & 1) ? (byte & 0xF) : (byte >> 4);
            out[start + i] = s * kLevels[code];
        }
    }
    return 0;
}

/* topk_compute_num_topk_columns, topk_cuda.cu:53-69: FP32 product, roundf (half away
 * from zero), clamp to cols, at least 1 when ratio > 0.  Returns 0xFFFFFFFF for a ratio
 * outside [0,1] (the reference throws there). */
uint32_t bsq_oracle_topk_num_columns(uint16_t cols, float ratio) {
    if (cols == 0) return 0;
    if (!(ratio >= 0.0f && ratio <= 1.0f)) return 0xFFFFFFFFu;
    const float raw = (float)cols * ratio;
    uint16_t k = (uint16_t)roundf(raw);
    if (k > cols) k = cols;
    else if (k == 0 && ratio > 0.0f) k = 1;
    return k;
}

/* Sort key of topk_cuda_utils.cuh:51-69 mapped onto an unsigned integer that orders the
 * same way as the reference's float key under a descending sort: key = |x| with NaN -> -inf,
 * so every NaN ranks below every number (including 0), and +0/-0 tie. */
static uint32_t topk_ukey(float x) {
    uint32_t b;
    memcpy(&b, &x, 4);
    b &= 0x7FFFFFFFu;
    return (b > 0x7F800000u) ? 0u : b + 1u;
}

/* run_topk_extraction, topk_cuda_utils.cuh:275-295 (build keys :51-69, stable descending
 * segmented radix sort :254-273, gather of the first k :71-93) and, when `zero_selected`,
 * zero_selected_entries_kernel :95-111 on the caller's matrix.
 * Order within a row: key descending, ties by ascending column (stable sort of the
 * column-ordered segment).  Values keep their sign and bit pattern. */
int bsq_oracle_topk_rows(float *x, uint32_t rows, uint32_t cols, uint32_t k, int zero_selected,
                         uint16_t *idx_out, float *val_out) {
    if (!x || !rows || !cols || k > cols) return 1;
    if (k == 0) return 0;
    if (!idx_out || !val_out) return 1;
    int failed = 0;
#pragma omp parallel
    {
        uint64_t *comp = (uint64_t *)malloc((size_t)cols * sizeof(uint64_t));
        uint64_t *tmp = (uint64_t *)malloc((size_t)cols * sizeof(uint64_t));
        if (!comp || !tmp) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(static)
            for (uint32_t r = 0; r < rows; ++r) {
                float *row = x + (size_t)r * cols;
                /* composite = key in the high half, (0xFFFF - col) below it: descending
                 * order of the composite == (key desc, col asc). */
                for (uint32_t c = 0; c < cols; ++c)
                    comp[c] = ((uint64_t)topk_ukey(row[c]) << 16) | (uint64_t)(0xFFFFu - c);
                /* LSD radix sort, 6 passes of 8 bits over the 48-bit composite, ascending */
                uint64_t *src = comp, *dst = tmp;
                for (int pass = 0; pass < 6; ++pass) {
                    uint32_t hist[257];
                    memset(hist, 0, sizeof(hist));
                    const int sh = pass * 8;
                    for (uint32_t c = 0; c < cols; ++c) hist[((src[c] >> sh) & 0xFF) + 1]++;
                    for (int d = 0; d < 256; ++d) hist[d + 1] += hist[d];
                    for (uint32_t c = 0; c < cols; ++c) dst[hist[(src[c] >> sh) & 0xFF]++] = src[c];
                    uint64_t *t = src; src = dst; dst = t;
                }
                for (uint32_t j = 0; j < k; ++j) {
                    const uint64_t e = src[cols - 1 - j];
                    const uint32_t c = 0xFFFFu - (uint32_t)(e & 0xFFFFu);
                    idx_out[(size_t)r * k + j] = (uint16_t)c;
                    val_out[(size_t)r * k + j] = row[c];
                }
                if (zero_selected)
                    for (uint32_t j = 0; j < k; ++j) row[idx_out[(size_t)r * k + j]] = 0.0f;
            }
        }
        free(comp);
        free(tmp);
    }
    return failed;
}

/* scatter_add_topk_kernel, topk_cuda_utils.cuh:132-149 (topk_apply, topk_cuda.cu:221-233) */
int bsq_oracle_topk_apply(const uint16_t *idx, const float *val, uint32_t rows, uint32_t cols,
                          uint32_t k, float *dense) {
    if (!dense || !rows || !cols) return 1;
    if (k == 0) return 0;
    if (!idx || !val) return 1;
    for (uint32_t r = 0; r < rows; ++r)
        for (uint32_t j = 0; j < k; ++j) {
            const uint32_t c = idx[(size_t)r * k + j];
            if (c < cols) dense[(size_t)r * cols + c] += val[(size_t)r * k + j];
        }
    return 0;
}

/* subtract_kernel + has_nonzero_kernel, src/bitsqz_llm.cu:164-184: e = a - b and the flag
 * "some |e| > FLT_EPSILON". */
int bsq_oracle_residual(const float *a, const float *b, uint64_t n, float *e) {
    int any = 0;
    for (uint64_t i = 0; i < n; ++i) {
        float d = a[i] - b[i];
        if (d != d) {
            /* The reference subtracts on the GPU (subtract_kernel, src/bitsqz_llm.cu:164-170), whose FP32 arithmetic
             * returns the canonical NaN 0x7fffffff whatever the NaN operand's payload was; a CPU keeps the payload.
             * The bits matter: a NaN error value is stored in the error top-k section as it is. */
            const uint32_t canonical = 0x7fffffffu;
            memcpy(&d, &canonical, 4);
        }
        e[i] = d;
        if (fabsf(d) > 1.1920928955078125e-07f) any = 1;
    }
    return any;
}

/* reconstruct_lowrank_cuda.cu:21-62: out = (U diag(S)) V^T, row-major m x n; U m x k and
 * V n x k row-major.  Accumulated in double and rounded once, so it serves as the
 * higher-precision reference the FP32 GEMM results are compared against by tolerance. */
int bsq_oracle_reconstruct(const float *U, const float *S, const float *V, uint32_t m, uint32_t n,
                           uint32_t k, float *out) {
    if (!U || !S || !V || !out || !m || !n || !k) return 1;
#pragma omp parallel for schedule(static)
    for (uint32_t i = 0; i < m; ++i) {
        for (uint32_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (uint32_t t = 0; t < k; ++t) {
                const float us = U[(size_t)i * k + t] * S[t]; /* cublasSdgmm rounds U*S to FP32 */
                acc += (double)us * (double)V[(size_t)j * k + t];
            }
            out[(size_t)i * n + j] = (float)acc;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------
 * Packed sections (byte layouts the reference writes into bitsqz_llm_array_t.payload).
 * ---------------------------------------------------------------------------------- */

/* quantization_cuda_packed_header_t, quantization_cuda.cuh:15-26 (48 bytes) followed by
 * scales and nibbles, quantization_cuda.cu:736-807.  method: 11 = NF4, 10 = NF4_DQ. */
uint64_t bsq_oracle_quant_section_size(int method, uint64_t n) {
    const uint64_t nb = (n + BSQ_BLOCK - 1) / BSQ_BLOCK;
    return 48u + (method == 11 ? nb * 4u : nb) + (n + 1) / 2;
}

int bsq_oracle_pack_quant_section(int method, const float *x, uint64_t n, uint8_t *dst) {
    if ((method != 10 && method != 11) || !x || !n || !dst) return 1;
    const uint64_t nb = (n + BSQ_BLOCK - 1) / BSQ_BLOCK;
    memset(dst, 0, 48);
    const uint32_t magic = 0x51544355u;
    const uint16_t version = 1;
    const int32_t m32 = method;
    const uint64_t bs = BSQ_BLOCK;
    memcpy(dst + 0, &magic, 4);
    memcpy(dst + 4, &version, 2);
    memcpy(dst + 8, &m32, 4);
    memcpy(dst + 16, &n, 8);
    memcpy(dst + 24, &nb, 8);
    memcpy(dst + 32, &bs, 8);
    if (method == 11) {
        float *scales = (float *)malloc((size_t)nb * 4);
        if (!scales) return 1;
        const int rc = bsq_oracle_nf4_quantize(x, n, scales, dst + 48 + nb * 4);
        memcpy(dst + 48, scales, (size_t)nb * 4);
        free(scales);
        return rc;
    }
    float dq = 0.0f;
    const int rc = bsq_oracle_nf4dq_quantize(x, n, &dq, dst + 48, dst + 48 + nb);
    memcpy(dst + 40, &dq, 4);
    return rc;
}

/* topk_packed_header_t, topk_cuda.cuh:16-21 (8 bytes) + rows*k u16 + rows*k f32,
 * topk_cuda.cu:294-330. */
uint64_t bsq_oracle_topk_section_size(uint32_t rows, uint32_t k) {
    return 8u + (uint64_t)rows * k * 6u;
}

int bsq_oracle_pack_topk_section(uint32_t rows, uint32_t cols, uint32_t k, const uint16_t *idx,
                                 const float *val, uint8_t *dst) {
    if (!dst) return 1;
    const uint16_t h[4] = {(uint16_t)rows, (uint16_t)cols, (uint16_t)k, 0};
    memcpy(dst, h, 8);
    const uint64_t cnt = (uint64_t)rows * k;
    if (cnt) {
        memcpy(dst + 8, idx, (size_t)cnt * 2);
        memcpy(dst + 8 + cnt * 2, val, (size_t)cnt * 4);
    }
    return 0;
}

/* ------------------------------------------------------------------------------------
 * bitsqz_llm_compress without SVD, src/bitsqz_llm.cu:981-1302 (branch :1181-1235):
 * copy -> outlier separation -> quantise (or dense FP32) -> optional error top-k of
 * (residual - dequantised) -> sections direct | outlier | error.  Writes the 200-byte
 * header followed by the payload into `dst` (capacity `cap`); returns the packed size,
 * or 0 on failure.  quant_method: -1 none, 10 NF4_DQ, 11 NF4.
 * ---------------------------------------------------------------------------------- */
static void put_section(uint8_t *hdr, int slot, uint64_t off, uint64_t size, uint8_t storage) {
    uint8_t *p = hdr + 48 + 24 * slot;
    memcpy(p, &off, 8);
    memcpy(p + 8, &size, 8);
    p[16] = storage;
}

uint64_t bsq_oracle_compress_nosvd(const float *input, uint16_t rows, uint16_t cols,
                                   float outlier_ratio, float error_ratio, int quant_method,
                                   uint8_t *dst, uint64_t cap) {
    if (!input || !rows || !cols || !dst || cap < 200) return 0;
    const uint32_t n = (uint32_t)rows * cols;
    const uint32_t ko = bsq_oracle_topk_num_columns(cols, outlier_ratio);
    const uint32_t ke = bsq_oracle_topk_num_columns(cols, error_ratio);
    if (ko == 0xFFFFFFFFu || ke == 0xFFFFFFFFu) return 0;
    float *res = (float *)malloc((size_t)n * 4);
    float *deq = NULL, *err = NULL;
    uint16_t *oi = NULL, *ei = NULL;
    float *ov = NULL, *ev = NULL;
    uint64_t total = 0;
    if (!res) return 0;
    memcpy(res, input, (size_t)n * 4);
    memset(dst, 0, 200);
    uint8_t *pay = dst + 200;
    uint64_t off = 0;
    uint32_t flags = 0;
    if (ko) {
        oi = (uint16_t *)malloc((size_t)rows * ko * 2);
        ov = (float *)malloc((size_t)rows * ko * 4);
        if (!oi || !ov || bsq_oracle_topk_rows(res, rows, cols, ko, 1, oi, ov)) goto done;
        flags |= 2u;
    }
    if (quant_method == 10 || quant_method == 11) {
        const uint64_t sz = bsq_oracle_quant_section_size(quant_method, n);
        if (200 + off + sz > cap) goto done;
        if (bsq_oracle_pack_quant_section(quant_method, res, n, pay + off)) goto done;
        put_section(dst, 3, off, sz, 2);
        const uint8_t *sec = pay + off;
        off += sz;
        if (ke) {
            const uint64_t nb = (n + BSQ_BLOCK - 1) / BSQ_BLOCK;
            deq = (float *)malloc((size_t)n * 4);
            err = (float *)malloc((size_t)n * 4);
            if (!deq || !err) goto done;
            if (quant_method == 11) {
                float *sc = (float *)malloc((size_t)nb * 4);
                if (!sc) goto done;
                memcpy(sc, sec + 48, (size_t)nb * 4);
                bsq_oracle_nf4_dequantize(sc, sec + 48 + nb * 4, n, deq);
                free(sc);
            } else {
                float dq;
                memcpy(&dq, sec + 40, 4);
                bsq_oracle_nf4dq_dequantize(dq, sec + 48, sec + 48 + nb, n, deq);
            }
            if (bsq_oracle_residual(res, deq, n, err)) {
                ei = (uint16_t *)malloc((size_t)rows * ke * 2);
                ev = (float *)malloc((size_t)rows * ke * 4);
                if (!ei || !ev || bsq_oracle_topk_rows(err, rows, cols, ke, 0, ei, ev)) goto done;
                flags |= 4u;
            }
        }
    } else {
        const uint64_t sz = (uint64_t)n * 4;
        if (200 + off + sz > cap) goto done;
        memcpy(pay + off, res, (size_t)sz);
        put_section(dst, 3, off, sz, 1);
        off += sz;
    }
    if (flags & 2u) {
        const uint64_t sz = bsq_oracle_topk_section_size(rows, ko);
        if (200 + off + sz > cap) goto done;
        bsq_oracle_pack_topk_section(rows, cols, ko, oi, ov, pay + off);
        put_section(dst, 4, off, sz, 3);
        off += sz;
    }
    if (flags & 4u) {
        const uint64_t sz = bsq_oracle_topk_section_size(rows, ke);
        if (200 + off + sz > cap) goto done;
        bsq_oracle_pack_topk_section(rows, cols, ke, ei, ev, pay + off);
        put_section(dst, 5, off, sz, 3);
        off += sz;
    }
    {   /* header fields, src/bitsqz_llm.cu:1253-1271; `payload` pointer left 0 here */
        const int16_t m1 = -1, one = 1, zero = 0;
        const int32_t none = -1, q = (quant_method == 10 || quant_method == 11) ? quant_method : -1;
        memcpy(dst + 0, &rows, 2);
        memcpy(dst + 2, &cols, 2);
        memcpy(dst + 4, &n, 4);
        memcpy(dst + 8, &outlier_ratio, 4);
        memcpy(dst + 12, &error_ratio, 4);
        memcpy(dst + 16, &m1, 2);      /* svd_ranks  */
        memcpy(dst + 18, &one, 2);     /* svd_niters */
        memcpy(dst + 20, &zero, 2);    /* effective_rank */
        memcpy(dst + 24, &none, 4);
        memcpy(dst + 28, &none, 4);
        memcpy(dst + 32, &q, 4);
        memcpy(dst + 40, &flags, 4);
    }
    total = 200 + off;
done:
    free(res); free(deq); free(err); free(oi); free(ov); free(ei); free(ev);
    return total;
}

/* bitsqz_llm_decompress without SVD, src/bitsqz_llm.cu:1360-1387: direct section, then
 * += error top-k, then += outlier top-k.  `packed` is header + payload as written above. */
int bsq_oracle_decompress_nosvd(const uint8_t *packed, uint64_t size, float *out) {
    if (!packed || size < 200 || !out) return 1;
    uint16_t rows, cols;
    uint32_t n, flags;
    int32_t q;
    memcpy(&rows, packed, 2);
    memcpy(&cols, packed + 2, 2);
    memcpy(&n, packed + 4, 4);
    memcpy(&q, packed + 32, 4);
    memcpy(&flags, packed + 40, 4);
    if (flags & 1u) return 1;
    const uint8_t *pay = packed + 200;
    uint64_t off, sz;
    memcpy(&off, packed + 48 + 24 * 3, 8);
    memcpy(&sz, packed + 48 + 24 * 3 + 8, 8);
    const uint8_t storage = packed[48 + 24 * 3 + 16];
    if (200 + off + sz > size) return 1;
    const uint64_t nb = ((uint64_t)n + BSQ_BLOCK - 1) / BSQ_BLOCK;
    if (storage == 1) {
        memcpy(out, pay + off, (size_t)n * 4);
    } else if (storage == 2 && q == 11) {
        float *sc = (float *)malloc((size_t)nb * 4);
        if (!sc) return 1;
        memcpy(sc, pay + off + 48, (size_t)nb * 4);
        bsq_oracle_nf4_dequantize(sc, pay + off + 48 + nb * 4, n, out);
        free(sc);
    } else if (storage == 2 && q == 10) {
        float dq;
        memcpy(&dq, pay + off + 40, 4);
        bsq_oracle_nf4dq_dequantize(dq, pay + off + 48, pay + off + 48 + nb, n, out);
    } else {
        return 1;
    }
    for (int pass = 0; pass < 2; ++pass) {           /* error first, outlier second */
        const int slot = pass == 0 ? 5 : 4;
        const uint32_t bit = pass == 0 ? 4u : 2u;
        if (!(flags & bit)) continue;
        memcpy(&off, packed + 48 + 24 * slot, 8);
        memcpy(&sz, packed + 48 + 24 * slot + 8, 8);
        if (200 + off + sz > size || sz < 8) return 1;
        uint16_t h[4];
        memcpy(h, pay + off, 8);
        const uint64_t cnt = (uint64_t)h[0] * h[2];
        if (h[0] != rows || h[1] != cols || sz != 8 + cnt * 6) return 1;
        uint16_t *idx = (uint16_t *)malloc((size_t)cnt * 2 + 2);
        float *val = (float *)malloc((size_t)cnt * 4 + 4);
        if (!idx || !val) { free(idx); free(val); return 1; }
        memcpy(idx, pay + off + 8, (size_t)cnt * 2);
        memcpy(val, pay + off + 8 + cnt * 2, (size_t)cnt * 4);
        bsq_oracle_topk_apply(idx, val, rows, cols, h[2], out);
        free(idx);
        free(val);
    }
    return 0;
}

void bsq_oracle_set_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int bsq_oracle_max_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
