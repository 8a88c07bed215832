// Small kernels around the expert matmuls: silu(g)*u, the weighted top-k
// combine, and the per-expert token-slot map ("map0").
// Reference: src/ops/silu_mul.metal:57-72, src/ops/combine.metal:70-133,
// src/ops/mm_id.metal:207-269.
#include "common.cuh"
#include "route_math.cuh"

namespace {

__global__ void silu_mul_kernel(const float *__restrict__ g, const float *__restrict__ u, int64_t n,
                                float *__restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float a = g[i];
    const float s = __fdiv_rn(a, __fadd_rn(1.0f, expf(-a))); // two separate roundings, then the product
    out[i] = __fmul_rn(s, u[i]);
}

__global__ void add_inplace_kernel(float *__restrict__ out, const float *__restrict__ b, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(out[i], b[i]);
}

// One thread per output element. The top_k terms are summed in the order of
// the reference's launch geometry: k strided over W lanes, then a butterfly.
template <int W>
__global__ void combine_kernel(const float *__restrict__ down, const float *__restrict__ col_l2,
                               const float *__restrict__ w, int seq, int top_k, int n_out,
                               float *__restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)seq * n_out) return;
    const int s = (int)(i / n_out), c = (int)(i % n_out);
    float v[W];
#pragma unroll
    for (int l = 0; l < W; l++) {
        float value = 0.0f;
        for (int k = l; k < top_k; k += W) {
            float d = down[((size_t)s * top_k + k) * n_out + c];
            if (col_l2) {
                d = __fmul_rn(d, col_l2[(size_t)s * top_k + k]);
                d = __fmul_rn(d, 0x1p-15f);
            }
            value = __fadd_rn(value, __fmul_rn(d, w[(size_t)s * top_k + k]));
        }
        v[l] = value;
    }
#pragma unroll
    for (int off = W / 2; off >= 1; off >>= 1)
#pragma unroll
        for (int l = 0; l < off; l++) v[l] = __fadd_rn(v[l], v[l + off]);
    out[i] = v[0];
}

// One block per expert: scan the tokens in chunks of 1024 (four consecutive tokens per thread), keep the
// token order, write flat ids `token*top_k + slot`.
__global__ void __launch_bounds__(256)
map0_kernel(const uint32_t *__restrict__ ids, int t, int top_k, int n_expert, uint32_t *__restrict__ tpe,
            int32_t *__restrict__ ids_map) {
    __shared__ int warp_count[8];
    __shared__ int base;
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) base = 0;
    __syncthreads();
    int32_t *dst = ids_map + (size_t)e * t;
    for (int t0 = 0; t0 < t; t0 += 1024) {
        int slot[4], mine = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int token = t0 + 4 * (int)threadIdx.x + j;
            slot[j] = -1;
            if (token < t) {
                for (int s = 0; s < top_k; s++)
                    if (ids[(size_t)token * top_k + s] == (uint32_t)e) { slot[j] = s; break; }
            }
            mine += slot[j] >= 0;
        }
        // exclusive prefix of the per-thread counts inside the warp, then over the warps
        int pre = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, pre, o);
            if (lane >= o) pre += v;
        }
        if (lane == 31) warp_count[warp] = pre;
        __syncthreads();
        int off = base + pre - mine;
        for (int wv = 0; wv < warp; wv++) off += warp_count[wv];
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (slot[j] >= 0) dst[off++] = (t0 + 4 * (int)threadIdx.x + j) * top_k + slot[j];
        __syncthreads();
        if (threadIdx.x == 0) {
            int tot = 0;
            for (int wv = 0; wv < 8; wv++) tot += warp_count[wv];
            base += tot;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) tpe[e] = (uint32_t)base;
}

// RMS norm of one row per warp (`ffn_norm`, src/model.rs:340): out = (x * inv) * weight with
// inv = 1 / sqrt(sum(x^2) / hidden + eps).  The sum of squares runs in the router's reduction order
// (128 fmaf chains over elements c, c + 128, ..., folded per lane and by the warp butterfly), so the
// router input - and with it the expert selection - does not depend on the launch geometry.
__global__ void __launch_bounds__(256) rms_norm_kernel(const float *__restrict__ x, const float *__restrict__ w, float eps,
                                                       int t, int hidden, float *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= t) return;
    const float *xr = x + (size_t)row * hidden;
    float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
    for (int i = lane * 4; i < hidden; i += 128) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        p0 = __fmaf_rn(v.x, v.x, p0);
        p1 = __fmaf_rn(v.y, v.y, p1);
        p2 = __fmaf_rn(v.z, v.z, p2);
        p3 = __fmaf_rn(v.w, v.w, p3);
    }
    const float ss = lmoe_router_fold(p0, p1, p2, p3);
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)hidden), eps)));
    float *orow = out + (size_t)row * hidden;
    for (int i = lane * 4; i < hidden; i += 128) {
        const float4 v = *reinterpret_cast<const float4 *>(xr + i);
        const float4 g = __ldg(reinterpret_cast<const float4 *>(w + i));
        float4 o;
        o.x = __fmul_rn(__fmul_rn(v.x, inv), g.x);
        o.y = __fmul_rn(__fmul_rn(v.y, inv), g.y);
        o.z = __fmul_rn(__fmul_rn(v.z, inv), g.z);
        o.w = __fmul_rn(__fmul_rn(v.w, inv), g.w);
        *reinterpret_cast<float4 *>(orow + i) = o;
    }
}

} // namespace

cudaError_t launch_rms_norm(const float *x, const float *w, float eps, int64_t t, int hidden, float *out, cudaStream_t s) {
    if (t == 0) return cudaSuccess;
    rms_norm_kernel<<<(unsigned)((t + 7) / 8), 256, 0, s>>>(x, w, eps, (int)t, hidden, out);
    return cudaGetLastError();
}

cudaError_t launch_silu_mul(const float *g, const float *u, int64_t n, float *out, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(g, u, n, out);
    return cudaGetLastError();
}

cudaError_t launch_add_inplace(float *out, const float *b, int64_t n, cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out, b, n);
    return cudaGetLastError();
}

cudaError_t launch_combine(const float *down, const float *col_l2, const float *w, int seq, int top_k,
                           int n_out, float *out, cudaStream_t s) {
    const int64_t n = (int64_t)seq * n_out;
    if (n == 0) return cudaSuccess;
    int width = 1;
    while (width < top_k / 2) width <<= 1;
    const unsigned grid = (unsigned)((n + 255) / 256);
    switch (width) {
    case 1: combine_kernel<1><<<grid, 256, 0, s>>>(down, col_l2, w, seq, top_k, n_out, out); break;
    case 2: combine_kernel<2><<<grid, 256, 0, s>>>(down, col_l2, w, seq, top_k, n_out, out); break;
    case 4: combine_kernel<4><<<grid, 256, 0, s>>>(down, col_l2, w, seq, top_k, n_out, out); break;
    case 8: combine_kernel<8><<<grid, 256, 0, s>>>(down, col_l2, w, seq, top_k, n_out, out); break;
    case 16: combine_kernel<16><<<grid, 256, 0, s>>>(down, col_l2, w, seq, top_k, n_out, out); break;
    default: combine_kernel<32><<<grid, 256, 0, s>>>(down, col_l2, w, seq, top_k, n_out, out); break;
    }
    return cudaGetLastError();
}

cudaError_t launch_map0(const uint32_t *ids, int t, int top_k, int n_expert, uint32_t *tpe, int32_t *ids_map,
                        cudaStream_t s) {
    if (n_expert == 0) return cudaSuccess;
    map0_kernel<<<n_expert, 256, 0, s>>>(ids, t, top_k, n_expert, tpe, ids_map);
    return cudaGetLastError();
}

// Expert ids of the whole block -> ids relative to the experts [first, first + count) resident on one rank;
// every other id (other ranks' experts, or already-empty slots) becomes the empty-slot id `count`.
__global__ void ep_localize_ids_kernel(const uint32_t *__restrict__ ids, int64_t n, uint32_t first, uint32_t count,
                                       uint32_t *__restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint32_t e = ids[i] - first; // wraps for ids below `first`
    out[i] = e < count ? e : count;
}

cudaError_t launch_ep_localize_ids(const uint32_t *ids, int64_t n, uint32_t first, uint32_t count, uint32_t *out,
                                   cudaStream_t s) {
    if (n == 0) return cudaSuccess;
    ep_localize_ids_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(ids, n, first, count, out);
    return cudaGetLastError();
}
