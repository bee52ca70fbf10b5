/*
 * TEST INFRASTRUCTURE / one-off generator.  Walks every finite FP32 value in ascending
 * order, applies the reference's literal 16-level nearest-code scan (nf4_impl.cpp:73-86,
 * quantization_cuda.cu:43-58) and records every place where the code changes.  It prints
 * the transitions below 2^23+1 (there must be exactly 15, each stepping the code up by
 * one: those are the thresholds the CUDA encoder binary-searches) and the number of
 * transitions above it (where FP32 rounding of v - L[i] makes the scan non-monotone and
 * the encoder must fall back to the literal scan).
 *
 *   gcc -O2 -fopenmp -ffp-contract=off gen_nf4_thresholds.c -o _ref/gen_nf4_thresholds -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static const float L[16] = {
    -1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

static inline int scan(float v) {
    int best = 0;
    float be = fabsf(v - L[0]);
    for (int i = 1; i < 16; ++i) {
        float e = fabsf(v - L[i]);
        if (e < be) { be = e; best = i; }
    }
    return best;
}
static inline float from_key(uint32_t key) {
    uint32_t bits = (key & 0x80000000u) ? (key ^ 0x80000000u) : ~key;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

#define CHUNKS 4096
typedef struct { uint32_t key; int from, to; } tr_t;
static tr_t tr[CHUNKS][64];
static int ntr[CHUNKS];
static int first_code[CHUNKS], last_code[CHUNKS];

int main(void) {
    const uint64_t per = (1ull << 32) / CHUNKS;
#pragma omp parallel for schedule(dynamic)
    for (int c = 0; c < CHUNKS; ++c) {
        int prev = -1;
        ntr[c] = 0;
        first_code[c] = -1;
        for (uint64_t k = (uint64_t)c * per; k < (uint64_t)(c + 1) * per; ++k) {
            const float v = from_key((uint32_t)k);
            if (!isfinite(v)) continue;
            const int code = scan(v);
            if (first_code[c] < 0) first_code[c] = code;
            if (prev >= 0 && code != prev && ntr[c] < 64) {
                tr[c][ntr[c]].key = (uint32_t)k; tr[c][ntr[c]].from = prev; tr[c][ntr[c]].to = code; ntr[c]++;
            }
            prev = code;
        }
        last_code[c] = prev;
    }
    int low = 0, high = 0, prev = -1, bad = 0;
    const float limit = 8388609.0f;
    for (int c = 0; c < CHUNKS; ++c) {
        if (first_code[c] < 0) continue;
        if (prev >= 0 && first_code[c] != prev) {   /* transition exactly on a chunk edge */
            const float v = from_key((uint32_t)((uint64_t)c * per));
            uint32_t b; memcpy(&b, &v, 4);
            if (v < limit) { printf("T[%d] = 0x%08x  /* %.9g */ (chunk edge)\n", first_code[c], b, v); low++; if (first_code[c] != prev + 1) bad++; }
            else high++;
        }
        for (int t = 0; t < ntr[c]; ++t) {
            const float v = from_key(tr[c][t].key);
            uint32_t b; memcpy(&b, &v, 4);
            if (v < limit) { printf("T[%d] = 0x%08x  /* %.9g */\n", tr[c][t].to, b, v); low++; if (tr[c][t].to != tr[c][t].from + 1) bad++; }
            else high++;
        }
        if (ntr[c] >= 64) high += 1000000;  /* overflowed: erratic region */
        prev = last_code[c];
    }
    printf("transitions below 2^23+1: %d (non-unit steps: %d); transitions at or above: %d%s\n", low, bad, high,
           high >= 1000000 ? " (capped)" : "");
    return (low == 15 && bad == 0) ? 0 : 1;
}
