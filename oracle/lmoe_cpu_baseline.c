/*
 * Timed CPU baseline of the MoE block -- TEST INFRASTRUCTURE ONLY (the benchmark's CPU leg and
 * its `--impl reference` arm time it; nothing in the shipped library may call or link it).
 *
 * The reference runs its CPU path through candle's k-quant `QMatMul` (src/gguf.rs:230,
 * `ReferenceExperts`, src/moe.rs:142-187).  candle is a Cargo dependency that is not vendored with
 * the reference (huggingface/candle 0.11.0, rev 25188553ba2ff0251bfe8c6a5e64496f93a2c48a), so this
 * file RESTATES the published ggml/candle CPU convention for k-quant mat-vecs instead of running
 * it: the activation row is quantized to 8-bit blocks of 256 values (one f32 scale per block and
 * the sums of every 16 values), and each super-block of a weight row contributes an integer dot
 * product scaled by d (and, for Q4_K, a "min" term against the block sums).  "Restated, unverified
 * against candle."  It is never the parity oracle: int8 activations alone move a product by about
 * 7e-3 relative L2, outside the 2e-3 bound the kernels are held to.
 *
 * Unlike lmoe_oracle.c (bit-specified routing: -O2 -ffp-contract=off) this unit is built for speed
 * with -O3 -march=native: where the host has 256-bit integer SIMD the int8 dot products use the pairwise
 * multiply-add instructions a production CPU build of candle/ggml relies on (plain loops otherwise).  Rows of a
 * projection are spread over all host threads with OpenMP.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "lmoe_oracle.h"

typedef struct {
    float d;
    int8_t qs[QK_K];
    int16_t bsums[16];
} q8k_block;

static int nearest_int(float v) { return (int)lrintf(v); }

/* x[k] -> k/256 blocks: scale = max-magnitude value / -127 (the ggml convention keeps the sign). */
static void quantize_q8k(const float *x, int k, q8k_block *y) {
    for (int b = 0; b < k / QK_K; b++) {
        float amax = 0.f, vmax = 0.f;
        for (int i = 0; i < QK_K; i++) {
            const float a = fabsf(x[b * QK_K + i]);
            if (a > amax) { amax = a; vmax = x[b * QK_K + i]; }
        }
        if (amax == 0.f) { memset(&y[b], 0, sizeof y[b]); continue; }
        const float iscale = -127.f / vmax;
        for (int i = 0; i < QK_K; i++) {
            int v = nearest_int(iscale * x[b * QK_K + i]);
            y[b].qs[i] = (int8_t)(v > 127 ? 127 : v < -128 ? -128 : v);
        }
        for (int j = 0; j < 16; j++) {
            int s = 0;
            for (int i = 0; i < 16; i++) s += y[b].qs[16 * j + i];
            y[b].bsums[j] = (int16_t)s;
        }
        y[b].d = 1.f / iscale;
    }
}

#ifdef __AVX2__
#include <immintrin.h>
#ifdef __F16C__
#define lmo_h2f(h) _cvtsh_ss(h) /* the hardware conversion; the same value as the table-free routine */
#endif

static inline int32_t hsum_epi32(__m256i v) {
    __m128i a = _mm_add_epi32(_mm256_castsi256_si128(v), _mm256_extracti128_si256(v, 1));
    a = _mm_add_epi32(a, _mm_shuffle_epi32(a, 0x4e));
    a = _mm_add_epi32(a, _mm_shuffle_epi32(a, 0xb1));
    return _mm_cvtsi128_si32(a);
}

/* 256-bit form: unsigned 4-bit fields times signed activation bytes through the u8 x s8 pairwise
 * multiply-add (sums of two products fit 16 bits: 2 * 15 * 127), then the 6-bit sub-block scale through
 * the 16-bit multiply-add into 32-bit lanes. */
static float dot_q4k_q8k(const uint8_t *row, const q8k_block *y, int nb) {
    const __m256i m4 = _mm256_set1_epi8(0x0f);
    float sum = 0.f;
    for (int b = 0; b < nb; b++) {
        const uint8_t *blk = row + b * Q4K_BYTES;
        uint16_t dh, mh;
        memcpy(&dh, blk, 2);
        memcpy(&mh, blk + 2, 2);
        const float d = lmo_h2f(dh) * y[b].d, dmin = lmo_h2f(mh) * y[b].d;
        __m256i acc = _mm256_setzero_si256();
        int32_t msum = 0;
        for (int j = 0; j < 4; j++) {
            int s0, m0, s1, m1;
            q4k_scale_min(blk + 4, 2 * j, &s0, &m0);
            q4k_scale_min(blk + 4, 2 * j + 1, &s1, &m1);
            const __m256i q = _mm256_loadu_si256((const __m256i *)(blk + 16 + 32 * j));
            const __m256i lo = _mm256_and_si256(q, m4), hi = _mm256_and_si256(_mm256_srli_epi16(q, 4), m4);
            const __m256i y0 = _mm256_loadu_si256((const __m256i *)(y[b].qs + 64 * j));
            const __m256i y1 = _mm256_loadu_si256((const __m256i *)(y[b].qs + 64 * j + 32));
            acc = _mm256_add_epi32(acc, _mm256_madd_epi16(_mm256_maddubs_epi16(lo, y0), _mm256_set1_epi16((short)s0)));
            acc = _mm256_add_epi32(acc, _mm256_madd_epi16(_mm256_maddubs_epi16(hi, y1), _mm256_set1_epi16((short)s1)));
            msum += m0 * (y[b].bsums[4 * j] + y[b].bsums[4 * j + 1]) + m1 * (y[b].bsums[4 * j + 2] + y[b].bsums[4 * j + 3]);
        }
        sum += d * (float)hsum_epi32(acc) - dmin * (float)msum;
    }
    return sum;
}

/* Q6_K: the 6-bit values (0..63) stay unsigned for the pairwise multiply-add (2 * 63 * 127 fits 16 bits);
 * the "-32" offset comes in through the activation sums of each 16-wide sub-block. */
static float dot_q6k_q8k(const uint8_t *row, const q8k_block *y, int nb) {
    const __m256i m4 = _mm256_set1_epi8(0x0f), m2 = _mm256_set1_epi8(0x30);
    float sum = 0.f;
    for (int b = 0; b < nb; b++) {
        const uint8_t *blk = row + b * Q6K_BYTES;
        const int8_t *sc = (const int8_t *)(blk + 192);
        uint16_t dh;
        memcpy(&dh, blk + 208, 2);
        const float d = lmo_h2f(dh) * y[b].d;
        __m256i acc = _mm256_setzero_si256();
        int32_t off = 0;
        for (int j = 0; j < 16; j++) off += sc[j] * y[b].bsums[j];
        for (int n = 0; n < 2; n++) {
            const __m256i qa = _mm256_loadu_si256((const __m256i *)(blk + 64 * n));
            const __m256i qb = _mm256_loadu_si256((const __m256i *)(blk + 64 * n + 32));
            const __m256i h = _mm256_loadu_si256((const __m256i *)(blk + 128 + 32 * n));
            const __m256i q1 = _mm256_or_si256(_mm256_and_si256(qa, m4), _mm256_and_si256(_mm256_slli_epi16(h, 4), m2));
            const __m256i q2 = _mm256_or_si256(_mm256_and_si256(qb, m4), _mm256_and_si256(_mm256_slli_epi16(h, 2), m2));
            const __m256i q3 = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(qa, 4), m4), _mm256_and_si256(h, m2));
            const __m256i q4 = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(qb, 4), m4), _mm256_and_si256(_mm256_srli_epi16(h, 2), m2));
            const __m256i qq[4] = {q1, q2, q3, q4};
            for (int i = 0; i < 4; i++) {
                const __m256i yv = _mm256_loadu_si256((const __m256i *)(y[b].qs + 128 * n + 32 * i));
                /* 16-bit lanes 0-7 belong to sub-block scale 2i, lanes 8-15 to 2i+1 */
                const __m256i sv = _mm256_set_m128i(_mm_set1_epi16(sc[8 * n + 2 * i + 1]), _mm_set1_epi16(sc[8 * n + 2 * i]));
                acc = _mm256_add_epi32(acc, _mm256_madd_epi16(_mm256_maddubs_epi16(qq[i], yv), sv));
            }
        }
        sum += d * (float)(hsum_epi32(acc) - 32 * off);
    }
    return sum;
}
#else
/* n a multiple of 16; written so the compiler widens to 16 bits and uses multiply-add pairs */
static inline int32_t dot_u8_s8(const uint8_t *restrict a, const int8_t *restrict b, int n) {
    int32_t s = 0;
    for (int i = 0; i < n; i++) s += (int32_t)a[i] * (int32_t)b[i];
    return s;
}
static inline int32_t dot_s8_s8(const int8_t *restrict a, const int8_t *restrict b, int n) {
    int32_t s = 0;
    for (int i = 0; i < n; i++) s += (int32_t)a[i] * (int32_t)b[i];
    return s;
}

/* Q4_K row . q8 activations: nibbles unpacked to bytes, eight 32-wide integer dots per super-block. */
static float dot_q4k_q8k(const uint8_t *row, const q8k_block *y, int nb) {
    float sum = 0.f;
    uint8_t q[QK_K];
    for (int b = 0; b < nb; b++) {
        const uint8_t *blk = row + b * Q4K_BYTES;
        uint16_t dh, mh;
        memcpy(&dh, blk, 2);
        memcpy(&mh, blk + 2, 2);
        const float d = lmo_h2f(dh) * y[b].d, dmin = lmo_h2f(mh) * y[b].d;
        const uint8_t *qs = blk + 16;
        for (int j = 0; j < 4; j++) {
            for (int l = 0; l < 32; l++) {
                q[64 * j + l] = qs[32 * j + l] & 0x0f;
                q[64 * j + 32 + l] = qs[32 * j + l] >> 4;
            }
        }
        int32_t isum = 0, msum = 0;
        for (int j = 0; j < 8; j++) {
            int sc, mn;
            q4k_scale_min(blk + 4, j, &sc, &mn);
            isum += sc * dot_u8_s8(q + 32 * j, y[b].qs + 32 * j, 32);
            msum += mn * (y[b].bsums[2 * j] + y[b].bsums[2 * j + 1]);
        }
        sum += d * (float)isum - dmin * (float)msum;
    }
    return sum;
}

/* Q6_K row . q8 activations: 6-bit values rebuilt as signed bytes, sixteen 16-wide integer dots. */
static float dot_q6k_q8k(const uint8_t *row, const q8k_block *y, int nb) {
    float sum = 0.f;
    int8_t q[QK_K];
    for (int b = 0; b < nb; b++) {
        const uint8_t *blk = row + b * Q6K_BYTES;
        const uint8_t *ql = blk, *qh = blk + 128;
        const int8_t *sc = (const int8_t *)(blk + 192);
        uint16_t dh;
        memcpy(&dh, blk + 208, 2);
        const float d = lmo_h2f(dh) * y[b].d;
        for (int n = 0; n < 2; n++) {
            for (int l = 0; l < 32; l++) {
                const uint8_t h = qh[32 * n + l];
                q[128 * n + l] = (int8_t)((ql[64 * n + l] & 0x0f) | ((h & 3) << 4)) - 32;
                q[128 * n + 32 + l] = (int8_t)((ql[64 * n + 32 + l] & 0x0f) | (((h >> 2) & 3) << 4)) - 32;
                q[128 * n + 64 + l] = (int8_t)((ql[64 * n + l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
                q[128 * n + 96 + l] = (int8_t)((ql[64 * n + 32 + l] >> 4) | (((h >> 6) & 3) << 4)) - 32;
            }
        }
        int32_t isum = 0;
        for (int j = 0; j < 16; j++) isum += sc[j] * dot_s8_s8(q + 16 * j, y[b].qs + 16 * j, 16);
        sum += d * (float)isum;
    }
    return sum;
}

#endif /* __AVX2__ */

static float dot_q8k(int dtype, const uint8_t *row, const q8k_block *y, int nb) {
    return dtype == LMO_Q4_K ? dot_q4k_q8k(row, y, nb) : dot_q6k_q8k(row, y, nb);
}

/* One SwiGLU expert for one token, rows spread over the OpenMP team. */
static void expert_ffn_q8(const lmo_layer *L, const uint8_t *g, const uint8_t *u, const uint8_t *d,
                          const q8k_block *xq, float wgt, float *out, float *act, q8k_block *aq) {
    const int H = L->hidden, F = L->expert_ff;
    const int64_t grow = (int64_t)(H / QK_K) * lmo_type_size(L->gate_dtype);
    const int64_t drow = (int64_t)(F / QK_K) * lmo_type_size(L->down_dtype);
#pragma omp parallel for schedule(static)
    for (int f = 0; f < F; f++) {
        const float gv = dot_q8k(L->gate_dtype, g + f * grow, xq, H / QK_K);
        const float uv = dot_q8k(L->gate_dtype, u + f * grow, xq, H / QK_K);
        act[f] = (gv / (1.0f + expf(-gv))) * uv;
    }
    quantize_q8k(act, F, aq);
#pragma omp parallel for schedule(static)
    for (int h = 0; h < H; h++) out[h] += wgt * dot_q8k(L->down_dtype, d + h * drow, aq, F / QK_K);
}

/* Whole block (route, routed experts, shared expert) through the int8-activation convention. */
int lmo_moe_forward_q8(const lmo_layer *L, const float *x, int t, float *out) {
    const int H = L->hidden, F = L->expert_ff, K = L->top_k;
    if (H % QK_K || F % QK_K) return -1;
    uint32_t *ids = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)t * K);
    float *w = (float *)malloc(sizeof(float) * (size_t)t * K);
    lmo_route(L->router, L->bias, x, t, H, L->n_expert, K, L->scale, L->norm, ids, w);
    const int64_t gexp = (int64_t)F * (H / QK_K) * lmo_type_size(L->gate_dtype);
    const int64_t dexp = (int64_t)H * (F / QK_K) * lmo_type_size(L->down_dtype);
    q8k_block *xq = (q8k_block *)malloc(sizeof(q8k_block) * (size_t)(H / QK_K));
    q8k_block *aq = (q8k_block *)malloc(sizeof(q8k_block) * (size_t)(F / QK_K));
    float *act = (float *)malloc(sizeof(float) * (size_t)F);
    for (int i = 0; i < t; i++) {
        float *o = out + (int64_t)i * H;
        for (int h = 0; h < H; h++) o[h] = 0.0f;
        quantize_q8k(x + (int64_t)i * H, H, xq);
        for (int k = 0; k < K; k++) {
            const uint32_t e = ids[(int64_t)i * K + k];
            expert_ffn_q8(L, L->gate + e * gexp, L->up + e * gexp, L->down + e * dexp, xq,
                          w[(int64_t)i * K + k], o, act, aq);
        }
        if (L->sh_gate) expert_ffn_q8(L, L->sh_gate, L->sh_up, L->sh_down, xq, 1.0f, o, act, aq);
    }
    free(ids); free(w); free(xq); free(aq); free(act);
    return 0;
}
