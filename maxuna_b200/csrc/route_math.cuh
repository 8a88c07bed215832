// Bit-specified routing arithmetic shared by the stand-alone routing kernels
// and the fused decode / prefill kernels.
//
// The expert ids must agree with the CPU definition to the bit, so every
// floating-point step that feeds the selection is written with explicit
// round-to-nearest intrinsics (never contracted, never re-associated):
//   * router logit: 128 partial sums p_c over elements c, c+128, c+256, ...
//     accumulated in index order with fmaf; lane l folds its four partials as
//     (p0+p1)+(p2+p3); the 32 lane values are folded by a butterfly with
//     strides 16, 8, 4, 2, 1;
//   * exp: n = rint(x*log2e); r = fma(n,-ln2_hi,x); r = fma(n,-ln2_lo,r);
//     degree-7 Horner polynomial in fmaf; scaled by 2^n;
//   * sigmoid(v) = 1 / (1 + exp(clamp(-v, -87, 87))).
// Routing rule: src/moe.rs:94-119 of the reference.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

__device__ __forceinline__ float lmoe_exp_fixed(float x) {
    const float LOG2E = 1.44269502162933349609375f;
    const float LN2_HI = 0.693145751953125f;
    const float LN2_LO = 1.42860676533018704e-06f;
    const float n = rintf(__fmul_rn(x, LOG2E));
    float r = __fmaf_rn(n, -LN2_HI, x);
    r = __fmaf_rn(n, -LN2_LO, r);
    float p = 1.0f / 5040.0f;
    p = __fmaf_rn(p, r, 1.0f / 720.0f);
    p = __fmaf_rn(p, r, 1.0f / 120.0f);
    p = __fmaf_rn(p, r, 1.0f / 24.0f);
    p = __fmaf_rn(p, r, 1.0f / 6.0f);
    p = __fmaf_rn(p, r, 0.5f);
    p = __fmaf_rn(p, r, 1.0f);
    p = __fmaf_rn(p, r, 1.0f);
    const int e = (int)n;
    return __fmul_rn(p, __int_as_float((e + 127) << 23));
}

__device__ __forceinline__ float lmoe_sigmoid_fixed(float v) {
    float a = -v;
    a = a > 87.0f ? 87.0f : a;
    a = a < -87.0f ? -87.0f : a;
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, lmoe_exp_fixed(a)));
}

// Fold four partial sums and reduce over the warp in the specified order.
__device__ __forceinline__ float lmoe_router_fold(float p0, float p1, float p2, float p3) {
    float v = __fadd_rn(__fadd_rn(p0, p1), __fadd_rn(p2, p3));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// One warp turns `n_expert` selection scores (shared memory, destroyed) into
// the ordered top_k: descending score, ties to the lower expert index.
// probs: unbiased probabilities (shared memory). Writes ids/weights rows.
__device__ __forceinline__ void lmoe_warp_select(float *sel, const float *probs, int n_expert, int top_k,
                                                 float scale, int norm, uint32_t *ids_row, float *w_row,
                                                 int lane) {
    float my_w = 0.0f; // lane k keeps weight k (top_k <= 32)
    for (int k = 0; k < top_k; k++) {
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        for (int e = lane; e < n_expert; e += 32) {
            const float v = sel[e];
            if (v > best || (v == best && e < best_i)) { best = v; best_i = e; }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        if (best_i == 0x7fffffff) best_i = 0; // only reachable with NaN scores
        if (lane == k) my_w = probs[best_i];
        if (lane == 0) {
            ids_row[k] = (uint32_t)best_i;
            sel[best_i] = -INFINITY;
        }
        __syncwarp();
    }
    if (norm) {
        float sum = 0.0f; // sequential in slot order, like a plain CPU sum
        for (int k = 0; k < top_k; k++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_w, k));
        sum = sum < 6.103515625e-5f ? 6.103515625e-5f : sum;
        my_w = __fdiv_rn(my_w, sum);
    }
    if (scale != 0.0f && scale != 1.0f) my_w = __fmul_rn(my_w, scale);
    if (lane < top_k) w_row[lane] = my_w;
}

// Register-resident variant of the selection for n_expert <= 512: each lane keeps
// experts lane, lane+32, ... ; every round is two warp-wide integer reductions
// (maximum of an order-preserving key, then the lowest expert index holding it).
// `logit_of(e)` supplies the pre-sigmoid logit.  Same result as lmoe_warp_select.
template <typename LogitFn>
__device__ __forceinline__ void lmoe_warp_select_regs(LogitFn logit_of, const float *__restrict__ bias,
                                                      int n_expert, int top_k, float scale, int norm,
                                                      uint32_t *ids_row, float *w_row, int lane) {
    constexpr int EPL = 16;
    float p[EPL];
    uint32_t key[EPL];
    float lg[EPL];
#pragma unroll
    for (int i = 0; i < EPL; i++) {
        const int e = lane + 32 * i;
        lg[i] = e < n_expert ? logit_of(e) : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < EPL; i++) {
        const int e = lane + 32 * i;
        key[i] = 0u;
        p[i] = 0.0f;
        if (e < n_expert) {
            p[i] = lmoe_sigmoid_fixed(lg[i]);
            float sv = bias ? __fadd_rn(p[i], __ldg(bias + e)) : p[i];
            sv = __fadd_rn(sv, 0.0f); // -0 -> +0 so the integer order equals the float order
            const uint32_t u = __float_as_uint(sv);
            key[i] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
            if (key[i] == 0u) key[i] = 1u; // 0 marks "taken / absent"
        }
    }
    float my_w = 0.0f;
    for (int k = 0; k < top_k; k++) {
        uint32_t best = 0u;
#pragma unroll
        for (int i = 0; i < EPL; i++) best = key[i] > best ? key[i] : best;
        const uint32_t m = __reduce_max_sync(0xffffffffu, best);
        uint32_t cand = 0xffffffffu;
#pragma unroll
        for (int i = EPL - 1; i >= 0; i--)
            if (key[i] == m) cand = (uint32_t)(lane + 32 * i);
        const uint32_t idx = __reduce_min_sync(0xffffffffu, cand);
        float pw = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; i++)
            if ((uint32_t)(lane + 32 * i) == idx) { pw = p[i]; key[i] = 0u; }
        pw = __shfl_sync(0xffffffffu, pw, idx & 31);
        if (lane == k) my_w = pw;
        if (lane == 0) ids_row[k] = idx;
    }
    if (norm) {
        float sum = 0.0f;
        for (int k = 0; k < top_k; k++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_w, k));
        sum = sum < 6.103515625e-5f ? 6.103515625e-5f : sum;
        my_w = __fdiv_rn(my_w, sum);
    }
    if (scale != 0.0f && scale != 1.0f) my_w = __fmul_rn(my_w, scale);
    if (lane < top_k) w_row[lane] = my_w;
}
