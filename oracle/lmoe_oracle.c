/*
 * CPU oracle for the quantized indexed MoE path -- TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's MoE hot
 * path so the CUDA kernels can be checked against it.  Nothing in the shipped
 * library may call, link or import it; only the test-suite, the smoke check and
 * the benchmark's CPU-baseline leg do.
 *
 * What each function follows (paths are relative to the reference project):
 *   - super-block formats            src/ops/mv.metal:55-75, src/ops/mm_id.metal:51-56
 *   - Q4_K / Q6_K decode             src/ops/mm_id.metal:89-111, 136-167
 *   - routing                        src/moe.rs:84-119 (floor constant src/moe.rs:14)
 *   - per-row dot oracle             src/ops/dispatch.rs:2273-2300 (testutil::oracle)
 *   - per-expert map (map0)          src/ops/mm_id.metal:207-269
 *   - silu(g)*u                      src/ops/silu_mul.metal:57-72
 *   - weighted combine               src/ops/combine.metal:70-133
 *   - ReferenceExperts / shared      src/moe.rs:142-187, 369-374, 73-78
 *
 * The k-quant arithmetic of the reference lives in a third-party dependency
 * that is not vendored with it (huggingface/candle 0.11.0, git rev
 * 25188553ba2ff0251bfe8c6a5e64496f93a2c48a).  The decode below restates the
 * published GGUF k-quant format and is pinned against gguf-py's independent
 * numpy decoder through committed golden vectors; the routing is pinned
 * against the known-answer cases of src/moe.rs:405-484.  The ENCODER here is
 * NOT candle's quantizer (its source is absent): it is a deterministic
 * encoder that emits valid super-blocks; parity is defined on identical bytes
 * fed to both sides, so byte-identity with a candle run is "parity unpinned".
 *
 * Build:  make -C oracle      (gcc -O2 -ffp-contract=off -fopenmp -shared; the timed CPU
 *         baseline is a separate unit, lmoe_cpu_baseline.c, with its own flags)
 * -ffp-contract=off matters: the router reduction below is specified to the
 * bit and must not be re-associated or fused by the compiler.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "lmoe_oracle.h"

/* ---------------------------------------------------------------- f16 ---- */

static float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even float -> half */
static uint16_t f2h(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* overflows to inf */
    if (x < 0x33000001u) return (uint16_t)sign;              /* rounds to zero */
    int32_t e = (int32_t)(x >> 23) - 127;
    uint32_t m = (x & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffffu; }
    uint32_t r = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (r & 1))) r++;
    return (uint16_t)(sign | (base + r));
}

float lmo_h2f(uint16_t h) { return h2f(h); }
uint16_t lmo_f2h(float f) { return f2h(f); }

/* ------------------------------------------------------------- formats ---- */

int lmo_type_size(int dtype) {
    return dtype == LMO_Q4_K ? Q4K_BYTES : dtype == LMO_Q6_K ? Q6K_BYTES : 0;
}

/* One Q4_K super-block -> 256 floats: w = (d*sc_j)*q - (dmin*m_j). */
static void deq_q4k_block(const uint8_t *b, float *y) {
    uint16_t dh, mh;
    memcpy(&dh, b, 2);
    memcpy(&mh, b + 2, 2);
    const float d = h2f(dh), dmin = h2f(mh);
    const uint8_t *sc = b + 4, *qs = b + 16;
    for (int j = 0; j < 4; j++) {
        int s1, m1, s2, m2;
        q4k_scale_min(sc, 2 * j, &s1, &m1);
        q4k_scale_min(sc, 2 * j + 1, &s2, &m2);
        const float d1 = d * (float)s1, n1 = dmin * (float)m1;
        const float d2 = d * (float)s2, n2 = dmin * (float)m2;
        for (int l = 0; l < 32; l++) y[64 * j + l] = d1 * (float)(qs[32 * j + l] & 0x0f) - n1;
        for (int l = 0; l < 32; l++) y[64 * j + 32 + l] = d2 * (float)(qs[32 * j + l] >> 4) - n2;
    }
}

/* One Q6_K super-block -> 256 floats: w = d*sc_j*(q-32). */
static void deq_q6k_block(const uint8_t *b, float *y) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    uint16_t dh;
    memcpy(&dh, b + 208, 2);
    const float d = h2f(dh);
    for (int n = 0; n < 2; n++) {
        for (int l = 0; l < 32; l++) {
            const int is = l / 16;
            const int q1 = (int)((ql[64 * n + l] & 0x0f) | (((qh[32 * n + l] >> 0) & 3) << 4)) - 32;
            const int q2 = (int)((ql[64 * n + 32 + l] & 0x0f) | (((qh[32 * n + l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)((ql[64 * n + l] >> 4) | (((qh[32 * n + l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)((ql[64 * n + 32 + l] >> 4) | (((qh[32 * n + l] >> 6) & 3) << 4)) - 32;
            y[128 * n + l] = d * (float)sc[8 * n + is] * (float)q1;
            y[128 * n + 32 + l] = d * (float)sc[8 * n + is + 2] * (float)q2;
            y[128 * n + 64 + l] = d * (float)sc[8 * n + is + 4] * (float)q3;
            y[128 * n + 96 + l] = d * (float)sc[8 * n + is + 6] * (float)q4;
        }
    }
}

/* Decode `nblocks` consecutive super-blocks. */
int lmo_dequantize(int dtype, const uint8_t *blocks, int64_t nblocks, float *out) {
    const int ts = lmo_type_size(dtype);
    if (!ts) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nblocks; i++) {
        if (dtype == LMO_Q4_K) deq_q4k_block(blocks + i * ts, out + i * QK_K);
        else deq_q6k_block(blocks + i * ts, out + i * QK_K);
    }
    return 0;
}

static int nearest_int(float v) { return (int)lrintf(v); }

/* Deterministic Q4_K encoder (not candle's): per 32-weight sub-block an
 * affine [min,max] -> 0..15 map, sub-block scales/mins to 6 bits against the
 * super-block maxima. */
static void enc_q4k_block(const float *x, uint8_t *b) {
    float scale[8], mins[8];
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; j++) {
        float lo = 0.f, hi = 0.f; /* the representable range must include 0 */
        for (int l = 0; l < 32; l++) {
            const float v = x[32 * j + l];
            if (v < lo) lo = v;
            if (v > hi) hi = v;
        }
        scale[j] = (hi - lo) / 15.f;
        mins[j] = -lo;
        if (scale[j] > max_scale) max_scale = scale[j];
        if (mins[j] > max_min) max_min = mins[j];
    }
    const float inv_s = max_scale > 0.f ? 63.f / max_scale : 0.f;
    const float inv_m = max_min > 0.f ? 63.f / max_min : 0.f;
    const uint16_t dh = f2h(max_scale / 63.f), mh = f2h(max_min / 63.f);
    const float d = h2f(dh), dmin = h2f(mh);
    uint8_t *s = b + 4, *qs = b + 16;
    int sc[8], mn[8];
    memset(s, 0, 12);
    for (int j = 0; j < 8; j++) {
        sc[j] = nearest_int(inv_s * scale[j]);
        mn[j] = nearest_int(inv_m * mins[j]);
        if (sc[j] > 63) sc[j] = 63;
        if (mn[j] > 63) mn[j] = 63;
        if (j < 4) {
            s[j] = (uint8_t)sc[j];
            s[j + 4] = (uint8_t)mn[j];
        } else {
            s[j + 4] = (uint8_t)((sc[j] & 0x0f) | ((mn[j] & 0x0f) << 4));
            s[j - 4] |= (uint8_t)((sc[j] >> 4) << 6);
            s[j] |= (uint8_t)((mn[j] >> 4) << 6);
        }
    }
    memcpy(b, &dh, 2);
    memcpy(b + 2, &mh, 2);
    uint8_t q[QK_K];
    for (int j = 0; j < 8; j++) {
        const float dj = d * (float)sc[j], mj = dmin * (float)mn[j];
        for (int l = 0; l < 32; l++) {
            int v = 0;
            if (dj > 0.f) v = nearest_int((x[32 * j + l] + mj) / dj);
            q[32 * j + l] = (uint8_t)(v < 0 ? 0 : v > 15 ? 15 : v);
        }
    }
    for (int j = 0; j < 4; j++)
        for (int l = 0; l < 32; l++) qs[32 * j + l] = (uint8_t)(q[64 * j + l] | (q[64 * j + 32 + l] << 4));
}

/* Deterministic Q6_K encoder (not candle's): per 16-weight sub-block a
 * symmetric absmax -> [-32,31] map, sub-block scales to int8. */
static void enc_q6k_block(const float *x, uint8_t *b) {
    float scale[16];
    float max_abs_scale = 0.f;
    for (int j = 0; j < 16; j++) {
        float amax = 0.f, vmax = 0.f;
        for (int l = 0; l < 16; l++) {
            const float a = fabsf(x[16 * j + l]);
            if (a > amax) { amax = a; vmax = x[16 * j + l]; }
        }
        scale[j] = -vmax / 32.f; /* the extreme value lands on q-32 = -32 */
        if (fabsf(scale[j]) > max_abs_scale) max_abs_scale = fabsf(scale[j]);
    }
    uint8_t *ql = b, *qh = b + 128;
    int8_t *sc = (int8_t *)(b + 192);
    memset(b, 0, Q6K_BYTES);
    const uint16_t dh = f2h(max_abs_scale / 127.f);
    const float d = h2f(dh);
    memcpy(b + 208, &dh, 2);
    if (!(d > 0.f)) {
        for (int i = 0; i < 128; i++) ql[i] = 0; /* q = 32 -> value 0 */
        for (int i = 0; i < 64; i++) qh[i] = 0xaa;
        return;
    }
    uint8_t q[QK_K];
    for (int j = 0; j < 16; j++) {
        int s = nearest_int(scale[j] / d);
        s = s < -128 ? -128 : s > 127 ? 127 : s;
        sc[j] = (int8_t)s;
        const float dj = d * (float)s;
        for (int l = 0; l < 16; l++) {
            int v = 0;
            if (dj != 0.f) v = nearest_int(x[16 * j + l] / dj);
            v = v < -32 ? -32 : v > 31 ? 31 : v;
            q[16 * j + l] = (uint8_t)(v + 32);
        }
    }
    for (int n = 0; n < 2; n++) {
        for (int l = 0; l < 32; l++) {
            const uint8_t q1 = q[128 * n + l], q2 = q[128 * n + 32 + l];
            const uint8_t q3 = q[128 * n + 64 + l], q4 = q[128 * n + 96 + l];
            ql[64 * n + l] = (uint8_t)((q1 & 0x0f) | ((q3 & 0x0f) << 4));
            ql[64 * n + 32 + l] = (uint8_t)((q2 & 0x0f) | ((q4 & 0x0f) << 4));
            qh[32 * n + l] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
        }
    }
}

/* Encode `nblocks*256` floats into consecutive super-blocks. */
int lmo_quantize(int dtype, const float *x, int64_t nblocks, uint8_t *out) {
    const int ts = lmo_type_size(dtype);
    if (!ts) return -1;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < nblocks; i++) {
        if (dtype == LMO_Q4_K) enc_q4k_block(x + i * QK_K, out + i * ts);
        else enc_q6k_block(x + i * QK_K, out + i * ts);
    }
    return 0;
}

/* ------------------------------------------------------------- routing ---- */

/* exp(x) for |x| <= 87 with a fixed sequence of IEEE-754 binary32 operations
 * (round-to-nearest-even; every fused step written as fmaf, nothing else
 * contracted).  The same sequence is used on the GPU, so selection scores --
 * and therefore expert ids -- agree to the bit.  Accuracy is ~1 ulp, well
 * inside the reference's 1e-5 weight tolerance (src/moe.rs:428-431). */
static float exp_fixed(float x) {
    const float LOG2E = 1.44269502162933349609375f;
    const float LN2_HI = 0.693145751953125f;           /* 0x3f317200 */
    const float LN2_LO = 1.42860676533018704e-06f;     /* 0x35bfbe8e */
    float n = rintf(x * LOG2E);
    float r = fmaf(n, -LN2_HI, x);
    r = fmaf(n, -LN2_LO, r);
    float p = 1.0f / 5040.0f;
    p = fmaf(p, r, 1.0f / 720.0f);
    p = fmaf(p, r, 1.0f / 120.0f);
    p = fmaf(p, r, 1.0f / 24.0f);
    p = fmaf(p, r, 1.0f / 6.0f);
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    int32_t e = (int32_t)n; /* in [-126, 126] for |x| <= 87 */
    uint32_t bits = (uint32_t)(e + 127) << 23;
    float s;
    memcpy(&s, &bits, 4);
    return p * s;
}

/* sigmoid(v) = 1 / (1 + exp(-v)), src/moe.rs:101 (candle_nn::ops::sigmoid). */
static float sigmoid_fixed(float v) {
    float a = -v;
    if (a > 87.0f) a = 87.0f;
    if (a < -87.0f) a = -87.0f;
    return 1.0f / (1.0f + exp_fixed(a));
}

float lmo_sigmoid(float v) { return sigmoid_fixed(v); }

/* Router logit with a fully specified reduction order (src/moe.rs:84-87 is a
 * plain f32 matmul; the order is this build's definition, shared with the
 * GPU):  128 partial sums p_c over the elements c, c+128, c+256, ... each
 * accumulated in index order with fmaf; lane l = c/4 folds its four partials
 * as (p0+p1)+(p2+p3); the 32 lane values are folded by a butterfly with
 * strides 16, 8, 4, 2, 1. */
static float router_dot(const float *x, const float *w, int h) {
    float p[128];
    for (int c = 0; c < 128; c++) {
        float acc = 0.0f;
        for (int i = c; i < h; i += 128) acc = fmaf(x[i], w[i], acc);
        p[c] = acc;
    }
    float v[32];
    for (int l = 0; l < 32; l++) v[l] = (p[4 * l] + p[4 * l + 1]) + (p[4 * l + 2] + p[4 * l + 3]);
    for (int off = 16; off >= 1; off >>= 1) {
        float nv[32];
        for (int l = 0; l < 32; l++) nv[l] = v[l] + v[l ^ off];
        memcpy(v, nv, sizeof v);
    }
    return v[0];
}

/* logits[t,e] = <x[t], router[e]>; router is [n_expert, hidden] row-major
 * (the GGUF `ffn_gate_inp` orientation; the reference transposes it once at
 * load, src/moe.rs:43, only to feed candle's matmul). */
void lmo_route_logits(const float *router, const float *x, int t, int hidden, int n_expert, float *logits) {
#pragma omp parallel for schedule(static) collapse(2)
    for (int i = 0; i < t; i++)
        for (int e = 0; e < n_expert; e++)
            logits[(int64_t)i * n_expert + e] = router_dot(x + (int64_t)i * hidden, router + (int64_t)e * hidden, hidden);
}

/* `ffn_norm`, src/model.rs:340 (candle RmsNorm: x * 1/sqrt(mean(x^2) + eps) * weight, f32).  The sum of
 * squares uses the router's reduction order (this build's definition, shared with the GPU). */
void lmo_rms_norm(const float *x, const float *w, float eps, int t, int hidden, float *out) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < t; i++) {
        const float *xr = x + (int64_t)i * hidden;
        const float ss = router_dot(xr, xr, hidden);
        const float mean = ss / (float)hidden;
        const float inv = 1.0f / sqrtf(mean + eps);
        for (int c = 0; c < hidden; c++) {
            const float v = xr[c] * inv;
            out[(int64_t)i * hidden + c] = v * w[c];
        }
    }
}

/* src/moe.rs:94-119.  ids ordered by descending selection score, ties to the
 * lower expert index (stable sort, src/moe.rs:104-105); weights gathered from
 * the UNBIASED probabilities, divided by max(sum, 2^-14) when `norm`, then
 * multiplied by `scale` unless it is 0 or 1 (src/moe.rs:115). */
void lmo_route_from_logits(const float *logits, const float *bias, int t, int n_expert, int top_k,
                           float scale, int norm, uint32_t *ids, float *weights) {
    const float floor_v = 6.103515625e-5f;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < t; i++) {
        float *probs = (float *)malloc(sizeof(float) * (size_t)n_expert * 2);
        float *sel = probs + n_expert;
        uint8_t *taken = (uint8_t *)calloc((size_t)n_expert, 1);
        for (int e = 0; e < n_expert; e++) {
            probs[e] = sigmoid_fixed(logits[(int64_t)i * n_expert + e]);
            sel[e] = probs[e] + (bias ? bias[e] : 0.0f);
        }
        for (int k = 0; k < top_k; k++) {
            int best = -1;
            for (int e = 0; e < n_expert; e++) {
                if (taken[e]) continue;
                if (best < 0 || sel[e] > sel[best]) best = e; /* strict > keeps the lower index on ties */
            }
            taken[best] = 1;
            ids[(int64_t)i * top_k + k] = (uint32_t)best;
            weights[(int64_t)i * top_k + k] = probs[best];
        }
        float *w = weights + (int64_t)i * top_k;
        if (norm) {
            float sum = 0.0f;
            for (int k = 0; k < top_k; k++) sum = sum + w[k];
            if (sum < floor_v) sum = floor_v;
            for (int k = 0; k < top_k; k++) w[k] = w[k] / sum;
        }
        if (scale != 0.0f && scale != 1.0f)
            for (int k = 0; k < top_k; k++) w[k] = w[k] * scale;
        free(probs);
        free(taken);
    }
}

void lmo_route(const float *router, const float *bias, const float *x, int t, int hidden, int n_expert,
               int top_k, float scale, int norm, uint32_t *ids, float *weights) {
    float *logits = (float *)malloc(sizeof(float) * (size_t)t * n_expert);
    lmo_route_logits(router, x, t, hidden, n_expert, logits);
    lmo_route_from_logits(logits, bias, t, n_expert, top_k, scale, norm, ids, weights);
    free(logits);
}

/* ------------------------------------------------------------ matmuls ----- */

/* Decode one weight row (k values) of a stack. */
static void deq_row(int dtype, const uint8_t *row, int k, float *out) {
    const int ts = lmo_type_size(dtype);
    for (int b = 0; b < k / QK_K; b++) {
        if (dtype == LMO_Q4_K) deq_q4k_block(row + b * ts, out + b * QK_K);
        else deq_q6k_block(row + b * ts, out + b * QK_K);
    }
}

/* out[t,s,:] = W[ids[t,s]] . x[t, (x_per_row==1 ? 0 : s), :] with a
 * sequential f32 dot per output row -- src/ops/dispatch.rs:2273-2300.
 * `accum64` != 0 accumulates in double instead (error attribution only). */
int lmo_mul_id(int dtype, const uint8_t *stack, int n_expert, int n_out, int k, const float *x,
               int x_per_row, const uint32_t *ids, int t, int top_k, float *out, int accum64) {
    const int ts = lmo_type_size(dtype);
    if (!ts || k % QK_K) return -1;
    const int64_t row_bytes = (int64_t)(k / QK_K) * ts;
    for (int64_t i = 0; i < (int64_t)t * top_k; i++)
        if (ids[i] >= (uint32_t)n_expert) return -2;
#pragma omp parallel
    {
        float *wrow = (float *)malloc(sizeof(float) * (size_t)k);
#pragma omp for schedule(static) collapse(2)
        for (int64_t pair = 0; pair < (int64_t)t * top_k; pair++) {
            for (int o = 0; o < n_out; o++) {
                const int token = (int)(pair / top_k), slot = (int)(pair % top_k);
                const uint32_t e = ids[pair];
                const float *xr = x + ((int64_t)token * x_per_row + (x_per_row == 1 ? 0 : slot)) * k;
                deq_row(dtype, stack + ((int64_t)e * n_out + o) * row_bytes, k, wrow);
                if (accum64) {
                    double acc = 0.0;
                    for (int i = 0; i < k; i++) acc += (double)wrow[i] * (double)xr[i];
                    out[pair * n_out + o] = (float)acc;
                } else {
                    float acc = 0.0f;
                    for (int i = 0; i < k; i++) acc += wrow[i] * xr[i];
                    out[pair * n_out + o] = acc;
                }
            }
        }
        free(wrow);
    }
    return 0;
}

/* Plain (non-indexed) quantized mat-vec: out[t,:] = W . x[t,:]. */
int lmo_mul_mv(int dtype, const uint8_t *w, int n_out, int k, const float *x, int t, float *out) {
    uint32_t *ids = (uint32_t *)calloc((size_t)t, sizeof(uint32_t));
    int rc = lmo_mul_id(dtype, w, 1, n_out, k, x, 1, ids, t, 1, out, 0);
    free(ids);
    return rc;
}

/* act = (g / (1 + exp(-g))) * u with the two roundings kept separate --
 * src/ops/silu_mul.metal:68-71.  exp is libm's here (the reference's is the
 * Metal one): compared under a tolerance, not bitwise. */
void lmo_silu_mul(const float *gate, const float *up, int64_t n, float *out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++) {
        const float g = gate[i];
        const float s = g / (1.0f + expf(-g));
        out[i] = s * up[i];
    }
}

/* dst[s,c] = sum_k down[s,k,c] * (col_l2[s,k] * 2^-15) * w[s,k]; each multiply
 * rounded separately -- src/ops/combine.metal:70-133.  Summation order: the
 * reference strides k over an 8-wide (next_pow2(top_k/2)) group and folds the
 * group with a hardware reduction whose order Metal does not specify; here the
 * group is folded as a butterfly with strides width/2 ... 1. */
void lmo_combine(const float *down, const float *col_l2, const float *w, int seq, int top_k, int n_out,
                 float *dst) {
    int width = 1;
    while (width < top_k / 2) width <<= 1;
    if (width > 32) width = 32;
#pragma omp parallel for schedule(static)
    for (int s = 0; s < seq; s++) {
        for (int c = 0; c < n_out; c++) {
            float lane[32];
            for (int l = 0; l < 32; l++) lane[l] = 0.0f;
            for (int l = 0; l < width; l++) {
                float value = 0.0f;
                for (int k = l; k < top_k; k += width) {
                    float d = down[((int64_t)s * top_k + k) * n_out + c];
                    if (col_l2) {
                        d = d * col_l2[(int64_t)s * top_k + k];
                        d = d * 0x1p-15f;
                    }
                    const float r = d * w[(int64_t)s * top_k + k];
                    value = value + r;
                }
                lane[l] = value;
            }
            for (int off = 16; off >= 1; off >>= 1) {
                float nv[32];
                for (int l = 0; l < 32; l++) nv[l] = lane[l] + lane[l ^ off];
                memcpy(lane, nv, sizeof lane);
            }
            dst[(int64_t)s * n_out + c] = lane[0];
        }
    }
}

/* Per-expert compacted lists of flat `token*top_k + slot` ids in scan order,
 * and their lengths -- src/ops/mm_id.metal:207-269.  ids_map is
 * [n_expert, t]; entries past tpe[e] are left untouched. */
int lmo_map0(const uint32_t *ids, int t, int top_k, int n_expert, uint32_t *tpe, int32_t *ids_map) {
    for (int e = 0; e < n_expert; e++) tpe[e] = 0;
    for (int token = 0; token < t; token++) {
        for (int slot = 0; slot < top_k; slot++) {
            const uint32_t e = ids[(int64_t)token * top_k + slot];
            if (e >= (uint32_t)n_expert) return -2;
            ids_map[(int64_t)e * t + tpe[e]] = token * top_k + slot;
            tpe[e]++;
            /* the reference's kernel takes at most one slot per (token, expert) */
        }
    }
    return 0;
}

/* --------------------------------------------------------- whole block ---- */


/* One SwiGLU expert on one token: out += wgt * down(silu(gate x) * up x).
 * f32 dequantize-then-dot, src/moe.rs:173-183; `accum64` as above. */
static void expert_ffn(const lmo_layer *L, const uint8_t *g, const uint8_t *u, const uint8_t *d,
                       const float *x, float wgt, float *out, float *act, float *wrow, int accum64) {
    const int H = L->hidden, F = L->expert_ff;
    const int64_t grow = (int64_t)(H / QK_K) * lmo_type_size(L->gate_dtype);
    const int64_t drow = (int64_t)(F / QK_K) * lmo_type_size(L->down_dtype);
    for (int f = 0; f < F; f++) {
        float gv, uv;
        deq_row(L->gate_dtype, g + f * grow, H, wrow);
        if (accum64) { double a = 0; for (int i = 0; i < H; i++) a += (double)wrow[i] * x[i]; gv = (float)a; }
        else { float a = 0; for (int i = 0; i < H; i++) a += wrow[i] * x[i]; gv = a; }
        deq_row(L->gate_dtype, u + f * grow, H, wrow);
        if (accum64) { double a = 0; for (int i = 0; i < H; i++) a += (double)wrow[i] * x[i]; uv = (float)a; }
        else { float a = 0; for (int i = 0; i < H; i++) a += wrow[i] * x[i]; uv = a; }
        const float s = gv / (1.0f + expf(-gv));
        act[f] = s * uv;
    }
    for (int h = 0; h < H; h++) {
        float dv;
        deq_row(L->down_dtype, d + h * drow, F, wrow);
        if (accum64) { double a = 0; for (int i = 0; i < F; i++) a += (double)wrow[i] * act[i]; dv = (float)a; }
        else { float a = 0; for (int i = 0; i < F; i++) a += wrow[i] * act[i]; dv = a; }
        out[h] += dv * wgt;
    }
}

/* MoeBlock::forward, src/moe.rs:73-78: route, routed experts weighted by the
 * routing weights (src/moe.rs:142-187), plus the unscaled shared expert
 * (src/moe.rs:369-374).  Writes ids/weights too when non-NULL. */
int lmo_moe_forward(const lmo_layer *L, const float *x, int t, float *out, uint32_t *ids_out,
                    float *w_out, int accum64) {
    const int H = L->hidden, F = L->expert_ff, K = L->top_k;
    if (H % QK_K || F % QK_K) return -1;
    uint32_t *ids = ids_out ? ids_out : (uint32_t *)malloc(sizeof(uint32_t) * (size_t)t * K);
    float *w = w_out ? w_out : (float *)malloc(sizeof(float) * (size_t)t * K);
    lmo_route(L->router, L->bias, x, t, H, L->n_expert, K, L->scale, L->norm, ids, w);
    const int64_t gexp = (int64_t)F * (H / QK_K) * lmo_type_size(L->gate_dtype);
    const int64_t dexp = (int64_t)H * (F / QK_K) * lmo_type_size(L->down_dtype);
#pragma omp parallel
    {
        float *act = (float *)malloc(sizeof(float) * (size_t)F);
        float *wrow = (float *)malloc(sizeof(float) * (size_t)(H > F ? H : F));
#pragma omp for schedule(dynamic, 1)
        for (int i = 0; i < t; i++) {
            float *o = out + (int64_t)i * H;
            for (int h = 0; h < H; h++) o[h] = 0.0f;
            for (int k = 0; k < K; k++) {
                const uint32_t e = ids[(int64_t)i * K + k];
                expert_ffn(L, L->gate + e * gexp, L->up + e * gexp, L->down + e * dexp, x + (int64_t)i * H,
                           w[(int64_t)i * K + k], o, act, wrow, accum64);
            }
            if (L->sh_gate)
                expert_ffn(L, L->sh_gate, L->sh_up, L->sh_down, x + (int64_t)i * H, 1.0f, o, act, wrow, accum64);
        }
        free(act);
        free(wrow);
    }
    if (!ids_out) free(ids);
    if (!w_out) free(w);
    return 0;
}

/* `ExpertFfn::forward`, src/moe.rs:19-21, as `ReferenceExperts` implements it (src/moe.rs:142-187):
 * the routing decision comes from the caller.  out[t] = sum over slots, in slot order, of
 * weights[t,k] * FFN_{ids[t,k]}(x[t]); an id >= n_expert is an empty slot; the same expert may
 * appear more than once in a row (each slot is evaluated on its own).  No shared expert. */
int lmo_experts_forward(const lmo_layer *L, const float *x, const uint32_t *ids, const float *w, int t, int top_k,
                        float *out, int accum64) {
    const int H = L->hidden, F = L->expert_ff;
    if (H % QK_K || F % QK_K) return -1;
    const int64_t gexp = (int64_t)F * (H / QK_K) * lmo_type_size(L->gate_dtype);
    const int64_t dexp = (int64_t)H * (F / QK_K) * lmo_type_size(L->down_dtype);
#pragma omp parallel
    {
        float *act = (float *)malloc(sizeof(float) * (size_t)F);
        float *wrow = (float *)malloc(sizeof(float) * (size_t)(H > F ? H : F));
#pragma omp for schedule(dynamic, 1)
        for (int i = 0; i < t; i++) {
            float *o = out + (int64_t)i * H;
            for (int h = 0; h < H; h++) o[h] = 0.0f;
            for (int k = 0; k < top_k; k++) {
                const uint32_t e = ids[(int64_t)i * top_k + k];
                if (e >= (uint32_t)L->n_expert) continue;
                expert_ffn(L, L->gate + e * gexp, L->up + e * gexp, L->down + e * dexp, x + (int64_t)i * H,
                           w[(int64_t)i * top_k + k], o, act, wrow, accum64);
            }
        }
        free(act);
        free(wrow);
    }
    return 0;
}

int lmo_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp master
        n = omp_get_num_threads();
    }
#endif
    return n;
}
