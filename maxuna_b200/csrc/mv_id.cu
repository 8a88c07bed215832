// Stand-alone indexed quantized mat-vec: out[t,s,:] = W[ids[t,s]] . x[t, s|0, :].
// Reference: `ops::mul_mv_id`, src/ops/mv_id.rs:37-45; kernels
// kernel_mul_mv_id_q{4,6}_K_f32_v, src/ops/mv.metal:181-290, 413-504, 638-717.
//
// One warp per output row; lanes stride over 16-byte pieces of the row, decode
// in registers, multiply f32 activations, reduce with warp shuffles.  The
// fused decode kernel (decode.cu) is the fast path; this entry point keeps the
// reference's op-level signature and serves the op-level parity tests.
#include "common.cuh"
#include "kquant.cuh"

namespace {

constexpr int MV_WARPS = 4;
constexpr int MV_ROWS_PER_WARP = 2;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float dot_row_q4k(const uint8_t *__restrict__ row, const float *__restrict__ x, int nb,
                                             int lane) {
    float acc = 0.f;
    for (int u = lane; u < nb * 8; u += 32) {
        const int b = u >> 3, c = u & 7, j = c >> 1, h = c & 1;
        const uint8_t *blk = row + (size_t)b * Q4K_BYTES;
        const uint32_t dm = __ldg(reinterpret_cast<const uint32_t *>(blk));
        const float d = lmoe_h2f((uint16_t)(dm & 0xffff)), dmin = lmoe_h2f((uint16_t)(dm >> 16));
        int sc0, mn0, sc1, mn1;
        q4k_scale_min(blk + 4, 2 * j, sc0, mn0);
        q4k_scale_min(blk + 4, 2 * j + 1, sc1, mn1);
        const uint4 qv = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 16 * c));
        const uint32_t qw[4] = {qv.x, qv.y, qv.z, qv.w};
        const float *xl = x + 256 * b + 64 * j + 16 * h;
        const float *xh = xl + 32;
        float slo = 0.f, shi = 0.f, xsl = 0.f, xsh = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float4 a = __ldg(reinterpret_cast<const float4 *>(xl + 4 * w));
            const float4 g = __ldg(reinterpret_cast<const float4 *>(xh + 4 * w));
            const uint32_t q = qw[w];
            slo += a.x * (float)(q & 15) + a.y * (float)((q >> 8) & 15) + a.z * (float)((q >> 16) & 15) +
                   a.w * (float)((q >> 24) & 15);
            shi += g.x * (float)((q >> 4) & 15) + g.y * (float)((q >> 12) & 15) + g.z * (float)((q >> 20) & 15) +
                   g.w * (float)(q >> 28);
            xsl += a.x + a.y + a.z + a.w;
            xsh += g.x + g.y + g.z + g.w;
        }
        acc += d * ((float)sc0 * slo + (float)sc1 * shi) - dmin * ((float)mn0 * xsl + (float)mn1 * xsh);
    }
    return acc;
}

__device__ __forceinline__ float dot_row_q6k(const uint8_t *__restrict__ row, const float *__restrict__ x, int nb,
                                             int lane) {
    float acc = 0.f;
    for (int u = lane; u < nb * 16; u += 32) {
        const int b = u >> 4, n = (u >> 3) & 1, lg = u & 7;
        const uint8_t *blk = row + (size_t)b * Q6K_BYTES;
        const uint32_t qa = ld_u32_unaligned2(blk + 64 * n + 4 * lg);
        const uint32_t qb = ld_u32_unaligned2(blk + 64 * n + 32 + 4 * lg);
        const uint32_t qh = ld_u32_unaligned2(blk + 128 + 32 * n + 4 * lg);
        const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192) + 8 * n + (lg >> 2);
        const float d = lmoe_h2f(*reinterpret_cast<const uint16_t *>(blk + 208));
        const float *xp = x + 256 * b + 128 * n + 4 * lg;
        const float4 x1 = __ldg(reinterpret_cast<const float4 *>(xp));
        const float4 x2 = __ldg(reinterpret_cast<const float4 *>(xp + 32));
        const float4 x3 = __ldg(reinterpret_cast<const float4 *>(xp + 64));
        const float4 x4 = __ldg(reinterpret_cast<const float4 *>(xp + 96));
        const float xa[4][4] = {{x1.x, x1.y, x1.z, x1.w}, {x2.x, x2.y, x2.z, x2.w},
                                {x3.x, x3.y, x3.z, x3.w}, {x4.x, x4.y, x4.z, x4.w}};
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int h = (qh >> (8 * i)) & 0xff;
            const int a = (qa >> (8 * i)) & 0xff, bq = (qb >> (8 * i)) & 0xff;
            const int q1 = ((a & 15) | ((h & 3) << 4)) - 32;
            const int q2 = ((bq & 15) | (((h >> 2) & 3) << 4)) - 32;
            const int q3 = ((a >> 4) | (((h >> 4) & 3) << 4)) - 32;
            const int q4 = ((bq >> 4) | (((h >> 6) & 3) << 4)) - 32;
            s[0] += xa[0][i] * (float)q1;
            s[1] += xa[1][i] * (float)q2;
            s[2] += xa[2][i] * (float)q3;
            s[3] += xa[3][i] * (float)q4;
        }
        acc += d * ((float)sc[0] * s[0] + (float)sc[2] * s[1] + (float)sc[4] * s[2] + (float)sc[6] * s[3]);
    }
    return acc;
}

// grid (ceil(n_out / (MV_WARPS*MV_ROWS_PER_WARP)), t*top_k)
template <int DT>
__global__ void __launch_bounds__(MV_WARPS * 32)
mul_mv_id_kernel(const uint8_t *__restrict__ w, int64_t expert_bytes, int n_expert, int n_out, int k,
                 const float *__restrict__ x, int x_per_row, const uint32_t *__restrict__ ids, int top_k,
                 float *__restrict__ out) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int pair = blockIdx.y;
    const int token = pair / top_k, slot = pair % top_k;
    const uint32_t e = ids ? ids[pair] : 0u;
    const int nb = k / QK_K;
    const int64_t row_bytes = (int64_t)nb * (DT == LMOE_Q4_K ? Q4K_BYTES : Q6K_BYTES);
    const float *xr = x + ((size_t)token * x_per_row + (x_per_row == 1 ? 0 : slot)) * k;
    const int r0 = (blockIdx.x * MV_WARPS + warp) * MV_ROWS_PER_WARP;
#pragma unroll
    for (int r = 0; r < MV_ROWS_PER_WARP; r++) {
        const int o = r0 + r;
        if (o >= n_out) break;
        float v = 0.f;
        if (e < (uint32_t)n_expert) { // an out-of-range id produces a zero row
            const uint8_t *row = w + (size_t)e * expert_bytes + (size_t)o * row_bytes;
            v = DT == LMOE_Q4_K ? dot_row_q4k(row, xr, nb, lane) : dot_row_q6k(row, xr, nb, lane);
            v = warp_sum(v);
        }
        if (lane == 0) out[(size_t)pair * n_out + o] = v;
    }
}

} // namespace

cudaError_t launch_mul_mv_id(int dtype, const uint8_t *w, int64_t expert_bytes, int n_expert, int n_out, int k,
                             const float *x, int t, int x_per_row, const uint32_t *ids, int top_k, float *out,
                             cudaStream_t s) {
    if (t == 0 || top_k == 0 || n_out == 0) return cudaSuccess;
    const int rows_per_block = MV_WARPS * MV_ROWS_PER_WARP;
    // grid.y is limited to 65535: fold large pair counts over several launches
    const int64_t pairs = (int64_t)t * top_k;
    for (int64_t p0 = 0; p0 < pairs; p0 += 65535 / top_k * top_k) {
        const int64_t np = pairs - p0 < 65535 / top_k * top_k ? pairs - p0 : 65535 / top_k * top_k;
        const dim3 grid((n_out + rows_per_block - 1) / rows_per_block, (unsigned)np);
        const int64_t tok0 = p0 / top_k;
        const float *xs = x + (size_t)tok0 * x_per_row * k;
        const uint32_t *is = ids ? ids + p0 : nullptr;
        float *os = out + (size_t)p0 * n_out;
        if (dtype == LMOE_Q4_K)
            mul_mv_id_kernel<LMOE_Q4_K><<<grid, MV_WARPS * 32, 0, s>>>(w, expert_bytes, n_expert, n_out, k, xs,
                                                                        x_per_row, is, top_k, os);
        else
            mul_mv_id_kernel<LMOE_Q6_K><<<grid, MV_WARPS * 32, 0, s>>>(w, expert_bytes, n_expert, n_out, k, xs,
                                                                        x_per_row, is, top_k, os);
    }
    return cudaGetLastError();
}
