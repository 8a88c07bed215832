// Device-side Q4_K / Q6_K encoder and decoder (one warp per super-block).
//
// The encoder is a deterministic min/max (Q4_K) and absmax (Q6_K) quantizer
// used to build synthetic expert stacks directly in HBM; it emits valid
// super-blocks but makes no claim of byte-identity with candle's quantizer.
#include "common.cuh"
#include "kquant.cuh"

namespace {

constexpr int WARPS = 8;

__device__ __forceinline__ float warp_max(float v) {
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__global__ void __launch_bounds__(WARPS * 32) quantize_q4k_kernel(const float *__restrict__ src, int64_t nblocks,
                                                                   uint8_t *__restrict__ dst) {
    __shared__ uint8_t sq[WARPS][QK_K];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t blk = (int64_t)blockIdx.x * WARPS + warp;
    if (blk >= nblocks) return;
    const float *x = src + blk * QK_K + lane * 8;
    float v[8];
    *reinterpret_cast<float4 *>(v) = *reinterpret_cast<const float4 *>(x);
    *reinterpret_cast<float4 *>(v + 4) = *reinterpret_cast<const float4 *>(x + 4);
    float lo = 0.f, hi = 0.f;
    for (int i = 0; i < 8; i++) { lo = fminf(lo, v[i]); hi = fmaxf(hi, v[i]); }
    for (int o = 1; o <= 2; o <<= 1) { // sub-block = 4 lanes
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const float scale = (hi - lo) / 15.f, mins = -lo;
    const float max_scale = warp_max(scale), max_min = warp_max(mins);
    const float inv_s = max_scale > 0.f ? 63.f / max_scale : 0.f;
    const float inv_m = max_min > 0.f ? 63.f / max_min : 0.f;
    const __half dh = __float2half_rn(max_scale / 63.f), mh = __float2half_rn(max_min / 63.f);
    const float d = __half2float(dh), dmin = __half2float(mh);
    int sc = min(63, __float2int_rn(inv_s * scale));
    int mn = min(63, __float2int_rn(inv_m * mins));
    const float dj = d * (float)sc, mj = dmin * (float)mn;
    for (int i = 0; i < 8; i++) {
        int q = 0;
        if (dj > 0.f) q = __float2int_rn((v[i] + mj) / dj);
        sq[warp][lane * 8 + i] = (uint8_t)max(0, min(15, q));
    }
    __syncwarp();
    uint8_t *b = dst + blk * Q4K_BYTES;
    // qs: 128 bytes, 4 per lane
    for (int i = 0; i < 4; i++) {
        const int idx = lane * 4 + i; // byte 32j + l
        const int j = idx >> 5, l = idx & 31;
        b[16 + idx] = (uint8_t)(sq[warp][64 * j + l] | (sq[warp][64 * j + 32 + l] << 4));
    }
    // header: sub-block j's values live in lane 4j
    int scj[8], mnj[8];
    for (int j = 0; j < 8; j++) {
        scj[j] = __shfl_sync(0xffffffffu, sc, 4 * j);
        mnj[j] = __shfl_sync(0xffffffffu, mn, 4 * j);
    }
    if (lane == 0) {
        *reinterpret_cast<__half *>(b) = dh;
        *reinterpret_cast<__half *>(b + 2) = mh;
        uint8_t s[12];
        for (int j = 0; j < 4; j++) {
            s[j] = (uint8_t)(scj[j] | ((scj[j + 4] >> 4) << 6));
            s[j + 4] = (uint8_t)(mnj[j] | ((mnj[j + 4] >> 4) << 6));
            s[j + 8] = (uint8_t)((scj[j + 4] & 0x0f) | ((mnj[j + 4] & 0x0f) << 4));
        }
        for (int j = 0; j < 12; j++) b[4 + j] = s[j];
    }
}

__global__ void __launch_bounds__(WARPS * 32) quantize_q6k_kernel(const float *__restrict__ src, int64_t nblocks,
                                                                   uint8_t *__restrict__ dst) {
    __shared__ uint8_t sq[WARPS][QK_K];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t blk = (int64_t)blockIdx.x * WARPS + warp;
    if (blk >= nblocks) return;
    const float *x = src + blk * QK_K + lane * 8;
    float v[8];
    *reinterpret_cast<float4 *>(v) = *reinterpret_cast<const float4 *>(x);
    *reinterpret_cast<float4 *>(v + 4) = *reinterpret_cast<const float4 *>(x + 4);
    float amax = 0.f, vmax = 0.f;
    for (int i = 0; i < 8; i++)
        if (fabsf(v[i]) > amax) { amax = fabsf(v[i]); vmax = v[i]; }
    { // sub-block = 2 lanes; the lower lane wins exact ties
        const float oa = __shfl_xor_sync(0xffffffffu, amax, 1), ov = __shfl_xor_sync(0xffffffffu, vmax, 1);
        if (oa > amax || (oa == amax && (lane & 1))) { amax = oa; vmax = ov; }
    }
    const float scale = -vmax / 32.f;
    const float max_abs_scale = warp_max(fabsf(scale));
    const __half dh = __float2half_rn(max_abs_scale / 127.f);
    const float d = __half2float(dh);
    uint8_t *b = dst + blk * Q6K_BYTES;
    int s = 0;
    if (d > 0.f) s = max(-128, min(127, __float2int_rn(scale / d)));
    const float dj = d * (float)s;
    for (int i = 0; i < 8; i++) {
        int q = 0;
        if (dj != 0.f) q = max(-32, min(31, __float2int_rn(v[i] / dj)));
        sq[warp][lane * 8 + i] = (uint8_t)(q + 32);
    }
    __syncwarp();
    const uint8_t *q = sq[warp];
    for (int i = 0; i < 4; i++) { // ql: 128 bytes
        const int idx = lane * 4 + i;
        const int n = idx >> 6, r = idx & 63;
        const int l = r & 31;
        const int a = r < 32 ? q[128 * n + l] : q[128 * n + 32 + l];
        const int c = r < 32 ? q[128 * n + 64 + l] : q[128 * n + 96 + l];
        b[idx] = (uint8_t)((a & 0x0f) | ((c & 0x0f) << 4));
    }
    for (int i = 0; i < 2; i++) { // qh: 64 bytes
        const int idx = lane * 2 + i;
        const int n = idx >> 5, l = idx & 31;
        b[128 + idx] = (uint8_t)((q[128 * n + l] >> 4) | ((q[128 * n + 32 + l] >> 4) << 2) |
                                 ((q[128 * n + 64 + l] >> 4) << 4) | ((q[128 * n + 96 + l] >> 4) << 6));
    }
    if ((lane & 1) == 0) b[192 + (lane >> 1)] = (uint8_t)(int8_t)s;
    if (lane == 0) {
        b[208] = (uint8_t)(__half_as_ushort(dh) & 0xff);
        b[209] = (uint8_t)(__half_as_ushort(dh) >> 8);
    }
}

__global__ void __launch_bounds__(WARPS * 32) dequantize_kernel(int dtype, const uint8_t *__restrict__ src,
                                                                 int64_t nblocks, float *__restrict__ dst) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t blk = (int64_t)blockIdx.x * WARPS + warp;
    if (blk >= nblocks) return;
    float *y = dst + blk * QK_K;
    if (dtype == LMOE_Q4_K) {
        const uint8_t *b = src + blk * Q4K_BYTES;
        const float d = lmoe_h2f(*reinterpret_cast<const uint16_t *>(b));
        const float dmin = lmoe_h2f(*reinterpret_cast<const uint16_t *>(b + 2));
        for (int i = 0; i < 8; i++) {
            const int idx = lane + 32 * i; // weight index
            const int sb = idx >> 5, j = sb >> 1, l = idx & 31;
            int sc, mn;
            q4k_scale_min(b + 4, sb, sc, mn);
            const int q = (sb & 1) ? (b[16 + 32 * j + l] >> 4) : (b[16 + 32 * j + l] & 0x0f);
            y[idx] = d * (float)sc * (float)q - dmin * (float)mn;
        }
    } else {
        const uint8_t *b = src + blk * Q6K_BYTES;
        const float d = lmoe_h2f((uint16_t)(b[208] | (b[209] << 8)));
        const int8_t *sc = reinterpret_cast<const int8_t *>(b + 192);
        for (int i = 0; i < 8; i++) {
            const int idx = lane + 32 * i;
            const int n = idx >> 7, g = (idx >> 5) & 3, l = idx & 31;
            const int qlb = b[64 * n + 32 * (g & 1) + l];
            const int lo4 = (g & 2) ? (qlb >> 4) : (qlb & 0x0f);
            const int hi2 = (b[128 + 32 * n + l] >> (2 * g)) & 3;
            const int q = (lo4 | (hi2 << 4)) - 32;
            y[idx] = d * (float)sc[8 * n + 2 * g + l / 16] * (float)q;
        }
    }
}

} // namespace

cudaError_t launch_quantize(int dtype, const float *src, int64_t nblocks, uint8_t *dst, cudaStream_t s) {
    if (nblocks == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((nblocks + WARPS - 1) / WARPS);
    if (dtype == LMOE_Q4_K) quantize_q4k_kernel<<<grid, WARPS * 32, 0, s>>>(src, nblocks, dst);
    else quantize_q6k_kernel<<<grid, WARPS * 32, 0, s>>>(src, nblocks, dst);
    return cudaGetLastError();
}

cudaError_t launch_dequantize(int dtype, const uint8_t *src, int64_t nblocks, float *dst, cudaStream_t s) {
    if (nblocks == 0) return cudaSuccess;
    const unsigned grid = (unsigned)((nblocks + WARPS - 1) / WARPS);
    dequantize_kernel<<<grid, WARPS * 32, 0, s>>>(dtype, src, nblocks, dst);
    return cudaGetLastError();
}
