// Stand-alone routing kernels: router logits (bit-specified f32 reduction) and
// the sigmoid / bias / ordered top-k / normalise step.
// Reference: `route_logits` and `route_from_logits`, src/moe.rs:84-119.
#include "common.cuh"
#include "route_math.cuh"

namespace {

constexpr int ROUTE_WARPS = 8;

// grid (ceil(n_expert / ROUTE_WARPS), ceil(t / TT)); one warp per expert row,
// TT tokens per pass so the router row is read once per token tile.
template <int TT>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_logits_kernel(const float *__restrict__ router, const float *__restrict__ x, int t, int hidden,
                    int n_expert, float *__restrict__ logits) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int e = blockIdx.x * ROUTE_WARPS + warp;
    const int t0 = blockIdx.y * TT;
    if (e >= n_expert) return;
    const float *w = router + (size_t)e * hidden;
    float acc[TT][4];
#pragma unroll
    for (int i = 0; i < TT; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f;

    if ((hidden & 3) == 0) {
        const int full = hidden / 128; // passes where every lane has a full float4
#pragma unroll 4
        for (int j = 0; j < full; j++) {
            const float4 wv = __ldg(reinterpret_cast<const float4 *>(w + 128 * j + 4 * lane));
#pragma unroll
            for (int i = 0; i < TT; i++) {
                if (t0 + i < t) {
                    const float4 xv =
                        __ldg(reinterpret_cast<const float4 *>(x + (size_t)(t0 + i) * hidden + 128 * j + 4 * lane));
                    acc[i][0] = __fmaf_rn(xv.x, wv.x, acc[i][0]);
                    acc[i][1] = __fmaf_rn(xv.y, wv.y, acc[i][1]);
                    acc[i][2] = __fmaf_rn(xv.z, wv.z, acc[i][2]);
                    acc[i][3] = __fmaf_rn(xv.w, wv.w, acc[i][3]);
                }
            }
        }
        const int base = 128 * full + 4 * lane; // ragged last pass (hidden % 128 != 0)
        if (base < hidden) {
            const float4 wv = __ldg(reinterpret_cast<const float4 *>(w + base));
#pragma unroll
            for (int i = 0; i < TT; i++) {
                if (t0 + i < t) {
                    const float4 xv = __ldg(reinterpret_cast<const float4 *>(x + (size_t)(t0 + i) * hidden + base));
                    acc[i][0] = __fmaf_rn(xv.x, wv.x, acc[i][0]);
                    acc[i][1] = __fmaf_rn(xv.y, wv.y, acc[i][1]);
                    acc[i][2] = __fmaf_rn(xv.z, wv.z, acc[i][2]);
                    acc[i][3] = __fmaf_rn(xv.w, wv.w, acc[i][3]);
                }
            }
        }
    } else {
        for (int j = 0; 128 * j < hidden; j++) {
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int idx = 128 * j + 4 * lane + c;
                if (idx < hidden) {
                    const float wv = w[idx];
#pragma unroll
                    for (int i = 0; i < TT; i++)
                        if (t0 + i < t) acc[i][c] = __fmaf_rn(x[(size_t)(t0 + i) * hidden + idx], wv, acc[i][c]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < TT; i++) {
        const float v = lmoe_router_fold(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        if (lane == 0 && t0 + i < t) logits[(size_t)(t0 + i) * n_expert + e] = v;
    }
}

// Prefill-sized variant for hidden = 128*HB: a block stages TTB tokens in shared memory; each of
// its 8 warps walks pairs of experts with both router rows in registers (all of their loads
// in flight together) and runs the same per-lane fmaf chains, so the logits are bit-identical.
template <int HB>
__global__ void __launch_bounds__(ROUTE_WARPS * 32, 1)
route_logits_tiled_kernel(const float *__restrict__ router, const float *__restrict__ x, int t, int n_expert, int ttb,
                          float *__restrict__ logits) {
    extern __shared__ float xs[];
    constexpr int H = 128 * HB;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t0 = blockIdx.x * ttb;
    const int nt = min(ttb, t - t0);
    for (int i = threadIdx.x; i < nt * (H / 4); i += ROUTE_WARPS * 32)
        reinterpret_cast<float4 *>(xs)[i] = __ldg(reinterpret_cast<const float4 *>(x + (size_t)t0 * H) + i);
    __syncthreads();
    // two router rows per pass: every hidden-state value read from shared memory feeds two chains
    for (int e = 2 * warp; e < n_expert; e += 2 * ROUTE_WARPS) {
        const bool two = e + 1 < n_expert;
        float4 wa[HB], wb[HB];
        const float4 *wr = reinterpret_cast<const float4 *>(router + (size_t)e * H) + lane;
        const float4 *wq = reinterpret_cast<const float4 *>(router + (size_t)(two ? e + 1 : e) * H) + lane;
#pragma unroll
        for (int j = 0; j < HB; j++) {
            wa[j] = __ldg(wr + 32 * j);
            wb[j] = __ldg(wq + 32 * j);
        }
        for (int i = 0; i < nt; i++) {
            const float4 *xr = reinterpret_cast<const float4 *>(xs + i * H) + lane;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, b0 = 0.f, b1 = 0.f, b2 = 0.f, b3 = 0.f;
#pragma unroll
            for (int j = 0; j < HB; j++) {
                const float4 xv = xr[32 * j];
                a0 = __fmaf_rn(xv.x, wa[j].x, a0);
                a1 = __fmaf_rn(xv.y, wa[j].y, a1);
                a2 = __fmaf_rn(xv.z, wa[j].z, a2);
                a3 = __fmaf_rn(xv.w, wa[j].w, a3);
                b0 = __fmaf_rn(xv.x, wb[j].x, b0);
                b1 = __fmaf_rn(xv.y, wb[j].y, b1);
                b2 = __fmaf_rn(xv.z, wb[j].z, b2);
                b3 = __fmaf_rn(xv.w, wb[j].w, b3);
            }
            const float va = lmoe_router_fold(a0, a1, a2, a3);
            const float vb = lmoe_router_fold(b0, b1, b2, b3);
            if (lane == 0) {
                logits[(size_t)(t0 + i) * n_expert + e] = va;
                if (two) logits[(size_t)(t0 + i) * n_expert + e + 1] = vb;
            }
        }
    }
}

// One warp per token; scores staged in shared memory (2 * n_expert floats per warp).
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_select_kernel(const float *__restrict__ logits, const float *__restrict__ bias, int t, int n_expert,
                    int top_k, float scale, int norm, uint32_t *__restrict__ ids, float *__restrict__ weights) {
    extern __shared__ float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int token = blockIdx.x * ROUTE_WARPS + warp;
    if (token >= t) return;
    float *probs = smem + (size_t)warp * 2 * n_expert;
    float *sel = probs + n_expert;
    for (int e = lane; e < n_expert; e += 32) {
        const float p = lmoe_sigmoid_fixed(logits[(size_t)token * n_expert + e]);
        probs[e] = p;
        sel[e] = bias ? __fadd_rn(p, bias[e]) : p;
    }
    __syncwarp();
    lmoe_warp_select(sel, probs, n_expert, top_k, scale, norm, ids + (size_t)token * top_k,
                     weights + (size_t)token * top_k, lane);
}

} // namespace

cudaError_t launch_route_logits(const float *router, const float *x, int t, int hidden, int n_expert,
                                float *logits, cudaStream_t s) {
    if (t == 0) return cudaSuccess;
    const unsigned gx = (unsigned)((n_expert + ROUTE_WARPS - 1) / ROUTE_WARPS);
    if (t <= 2) {
        route_logits_kernel<1><<<dim3(gx, t), ROUTE_WARPS * 32, 0, s>>>(router, x, t, hidden, n_expert, logits);
    } else if (t <= 64) {
        route_logits_kernel<4><<<dim3(gx, (t + 3) / 4), ROUTE_WARPS * 32, 0, s>>>(router, x, t, hidden, n_expert, logits);
    } else if (hidden == 128 * 24) {
        // Up to 16 tokens per block (one block per SM: 16 rows of f32 fill its shared memory); more tokens per
        // block mean fewer re-reads of the router from L2.  The token count per block is the smallest that
        // keeps the grid within whole waves of the device, so the last wave is not mostly empty
        // (4096 tokens: 293 blocks of 14 instead of 256 of 16 on 148 SMs).
        static int sms_of[64] = {0}; // per device: SM count, and the shared-memory opt-in done once
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
        if (!sms_of[dev]) {
            int n = 0;
            if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
            cudaFuncSetAttribute(route_logits_tiled_kernel<24>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(16 * hidden * sizeof(float)));
            sms_of[dev] = n;
        }
        const int sms = sms_of[dev];
        const int waves = (t + 16 * sms - 1) / (16 * sms);
        int ttb = (t + waves * sms - 1) / (waves * sms);
        if (ttb < 8) ttb = t >= 2048 ? ttb : 8;      // small inputs: 8 per block covers the SMs well enough
        if (ttb < 1) ttb = 1;
        if (ttb > 16) ttb = 16;
        const size_t smem = (size_t)ttb * hidden * sizeof(float);
        route_logits_tiled_kernel<24><<<(t + ttb - 1) / ttb, ROUTE_WARPS * 32, smem, s>>>(router, x, t, n_expert, ttb, logits);
    } else {
        route_logits_kernel<8><<<dim3(gx, (t + 7) / 8), ROUTE_WARPS * 32, 0, s>>>(router, x, t, hidden, n_expert, logits);
    }
    return cudaGetLastError();
}

cudaError_t launch_route_select(const float *logits, const float *bias, int t, int n_expert, int top_k,
                                float scale, int norm, uint32_t *ids, float *weights, cudaStream_t s) {
    if (t == 0) return cudaSuccess;
    const size_t smem = (size_t)ROUTE_WARPS * 2 * n_expert * sizeof(float);
    const unsigned grid = (unsigned)((t + ROUTE_WARPS - 1) / ROUTE_WARPS);
    route_select_kernel<<<grid, ROUTE_WARPS * 32, smem, s>>>(logits, bias, t, n_expert, top_k, scale, norm, ids,
                                                             weights);
    return cudaGetLastError();
}

// ---- routing without any allocation -------------------------------------------------------
// Some hosts of this library may not allocate device memory at the moment they route: an engine
// whose buffer pool owns the whole device and hands nothing to plugins, a serving loop running
// under a frozen memory budget, or code that is between cudaStreamBeginCapture and EndCapture.
// For them the logits scratch of `lmoe_route` lives in this fixed array instead of a caller
// workspace.  Every GPU that loads the library carries the array until the process exits.
#define LMOE_ROUTE_NOALLOC_MAX_LOGITS (64 * 512) /* t * n_expert floats, 128 KB */
static __device__ __align__(256) float g_route_noalloc_logits[LMOE_ROUTE_NOALLOC_MAX_LOGITS];

extern "C" lmoe_status lmoe_route_noalloc(const float *router, const float *bias, const float *x, int64_t t,
                                          int64_t hidden, int64_t n_expert, int64_t top_k, float scale, int32_t norm,
                                          uint32_t *ids_out, float *weights_out, void *stream) {
    lmoe_clear_error();
    if (t < 0 || n_expert < 1 || n_expert > 512 || top_k < 1 || top_k > 32 || top_k > n_expert)
        return lmoe_fail(LMOE_ERR_INVALID, "route_noalloc: t >= 0, n_expert in [1, 512], top_k in [1, min(32, n_expert)] required");
    if (hidden < 1 || hidden > (1 << 20)) return lmoe_fail(LMOE_ERR_INVALID, "hidden (%lld) out of range", (long long)hidden);
    // t is bounded before the product is formed, so the comparison below cannot wrap around
    if (t > LMOE_ROUTE_NOALLOC_MAX_LOGITS || t * n_expert > LMOE_ROUTE_NOALLOC_MAX_LOGITS)
        return lmoe_fail(LMOE_ERR_INVALID,
                         "route_noalloc: t * n_expert = %lld exceeds the built-in scratch of %d logits; use lmoe_route with a workspace",
                         t > LMOE_ROUTE_NOALLOC_MAX_LOGITS ? (long long)t : (long long)(t * n_expert), LMOE_ROUTE_NOALLOC_MAX_LOGITS);
    if (!router || !x || !ids_out || !weights_out) return lmoe_fail(LMOE_ERR_INVALID, "router/x/ids_out/weights_out is NULL");
    if (hidden % 4 == 0 && (((uintptr_t)router | (uintptr_t)x) & 15u))
        return lmoe_fail(LMOE_ERR_INVALID, "router and x must be 16-byte aligned");
    // In host code the array's name is only a stand-in; the kernels need its device address, which
    // differs per GPU.  It is looked up once per device, with that device current.
    static float *dev_ptr[64] = {nullptr};
    int dev = 0;
    LMOE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "device ordinal %d not supported", dev);
    if (!dev_ptr[dev]) {
        float *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_route_noalloc_logits);
        if (e != cudaSuccess || !p)
            return lmoe_fail(LMOE_ERR_CUDA, "cudaGetSymbolAddress(route scratch) failed: %s", cudaGetErrorString(e));
        dev_ptr[dev] = p;
    }
    float *logits = dev_ptr[dev];
    // nothing has to start at zero: every logit a launch reads was written by the same call
    LMOE_CUDA(launch_route_logits(router, x, (int)t, (int)hidden, (int)n_expert, logits, (cudaStream_t)stream));
    LMOE_CUDA(launch_route_select(logits, bias, (int)t, (int)n_expert, (int)top_k, scale, norm, ids_out, weights_out,
                                  (cudaStream_t)stream));
    return LMOE_OK;
}
