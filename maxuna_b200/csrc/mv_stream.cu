// Plain Q6_K mat-vec for one activation row at a time, streamed: out[o] = W[o, :] . x.
// Reference: `ops::mul_mv`, src/ops/mv_id.rs:54-56 (kernel_mul_mv_q6_K_f32, src/ops/mv.metal), which the model
// calls once per decoded token for the vocabulary projection (src/model.rs:388-403): Q6_K [100352 x 3072],
// 253 MB that must all cross HBM, so the kernel is a pure bandwidth problem.
//
//   * One persistent CTA per SM.  A producer thread moves chunks of 16 weight rows (one MMA row tile,
//     16 * row_bytes contiguous bytes, always a multiple of 16) into a shared-memory ring with one bulk copy
//     each, completion counted on an mbarrier; as many stages as fit (five at k = 3072: 200 KB in flight per SM).
//   * Twelve consumer warps split the super-blocks of a chunk (the K dimension).  The six-bit values go to the
//     integer tensor-core path exactly as in the fused decode kernel: the activation row is quantized once per
//     CTA under the largest magnitude of each 256-wide block and carried as three signed base-128 digits
//     (21 bits) in three MMA columns, so the integer sums are exact; the "-32" offset is one f16 MMA per
//     super-block against the 16-wide activation sums.
//   * The warps' partial sums of the 16 rows meet in a double-buffered shared array; one named barrier per chunk.
//   * Every wait is bounded.  A wait that gives up marks the CTA (a shared-memory word) and the rows it still
//     writes become NaN, so a launch that went wrong cannot pass for a result.
#include "stream_math.cuh"

namespace {

constexpr int MVS_ROWS = 16;
constexpr int MVS_NCW = 12;
constexpr int MVS_CONS = 32 * MVS_NCW;
constexpr int MVS_THREADS = MVS_CONS + 32;
constexpr int MVS_NDIG = 3;
constexpr int MVS_MAX_STAGES = 8;
constexpr int MVS_MAX_CHUNK = 56 * 1024;
constexpr int MVS_SMEM_MAX = 227 * 1024;

struct MvsLayout {
    int chunk_bytes, stage_stride, nstage, xs, ss;
    int o_ring, o_xc, o_s, o_sx, o_red, o_bar, total;
    __host__ __device__ explicit MvsLayout(int k) {
        const int nb = k / QK_K;
        chunk_bytes = MVS_ROWS * nb * Q6K_BYTES;
        stage_stride = (chunk_bytes + 127) / 128 * 128;
        xs = k + 32;         // bytes per digit column (+32: the columns of one load cover different banks)
        ss = nb * 16;        // 16-wide sub-block sums per column
        int o = 0;
        o_xc = o; o += (MVS_NDIG * xs + 15) / 16 * 16;
        o_s = o; o += (MVS_NDIG * ss * 2 + 15) / 16 * 16;
        o_sx = o; o += nb * 8 * 4;
        o_red = o; o += 2 * MVS_NCW * MVS_ROWS * 4;
        o_bar = o; o += 2 * MVS_MAX_STAGES * 8 + 16; // full / empty barriers, then the CTA's failure word
        o = (o + 127) / 128 * 128;
        o_ring = o;
        int n = (MVS_SMEM_MAX - o - 16) / stage_stride; // 16 spare bytes: an aligned two-word read may end past the last block
        nstage = n > MVS_MAX_STAGES ? MVS_MAX_STAGES : n;
        total = o + (nstage > 0 ? nstage : 0) * stage_stride + 16;
    }
};

// The activation row as digits, sums and column scales (one 256-wide block per warp and step).
__device__ __forceinline__ void mvs_stage_x(const float *__restrict__ x, int nb, int8_t *xc, __half *sh, float *sxs,
                                            int xs, int ss, int warp, int lane) {
    constexpr float QMAX = 524287.f;
    for (int b = warp; b < nb; b += MVS_NCW) {
        const float4 a = __ldg(reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8));
        const float4 c = __ldg(reinterpret_cast<const float4 *>(x + b * QK_K + lane * 8) + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float inv = amax > 0.f ? QMAX / amax : 0.f;
        const float sx = amax * (1.0f / QMAX);
        int sum = 0;
        uint32_t dig[MVS_NDIG][2];
#pragma unroll
        for (int d = 0; d < MVS_NDIG; d++) dig[d][0] = dig[d][1] = 0u;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int X = __float2int_rn(v[j] * inv);
            sum += X;
#pragma unroll
            for (int d = MVS_NDIG - 1; d > 0; d--) { // least significant digit first; the last takes what is left
                const int dd = ((X + 64) & 127) - 64;
                dig[d][j >> 2] |= (uint32_t)(dd & 255) << (8 * (j & 3));
                X = (X - dd) >> 7;
            }
            dig[0][j >> 2] |= (uint32_t)(X & 255) << (8 * (j & 3));
        }
#pragma unroll
        for (int d = 0; d < MVS_NDIG; d++)
            *reinterpret_cast<uint2 *>(xc + d * xs + b * QK_K + lane * 8) = make_uint2(dig[d][0], dig[d][1]);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if ((lane & 1) == 0) {
            // the 16-wide integer sum times 2^-9 (|sum| <= 16 * QMAX fits f16 then), as a high and a low f16 part
            const float sf = (float)sum * 0x1p-9f;
            const __half h = __float2half_rn(sf);
            const int idx = b * 16 + (lane >> 1);
            sh[idx] = h;
            sh[ss + idx] = __float2half_rn(sf - __half2float(h));
            sh[2 * ss + idx] = __float2half_rn(0.f);
        }
        if (lane < 8) {
            // column scale: digit d (most significant first) weighs 128^(2-d); the other MMA columns count for nothing
            sxs[b * 8 + lane] = lane == 0 ? sx * 16384.f : (lane == 1 ? sx * 128.f : (lane == 2 ? sx : 0.f));
        }
    }
}

__global__ void __launch_bounds__(MVS_THREADS, 1)
mv_q6k_stream_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ out, int k, int n_chunks) {
    extern __shared__ __align__(128) uint8_t smem[];
    const MvsLayout L(k);
    const int nb = k / QK_K, row_bytes = nb * Q6K_BYTES, nstage = L.nstage;
    int8_t *xc = reinterpret_cast<int8_t *>(smem + L.o_xc);
    __half *sh = reinterpret_cast<__half *>(smem + L.o_s);
    float *sxs = reinterpret_cast<float *>(smem + L.o_sx);
    float *red = reinterpret_cast<float *>(smem + L.o_red);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.o_bar);
    uint64_t *empty = full + MVS_MAX_STAGES;
    uint32_t *fail = reinterpret_cast<uint32_t *>(empty + MVS_MAX_STAGES); // [0] flag, [1] where, [2] CTA
    uint8_t *ring = smem + L.o_ring;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < nstage; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, MVS_NCW);
        }
        fail[0] = fail[1] = fail[2] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == MVS_NCW) {
        // ---- producer: one bulk copy per chunk, running ahead by the depth of the ring
        if (lane == 0) {
            int i = 0;
            for (int c = blockIdx.x; c < n_chunks; c += gridDim.x, i++) {
                const int s = i % nstage;
                if (i >= nstage) mbar_wait<32>(empty + s, (uint32_t)((i / nstage - 1) & 1), fail, 1u);
                mbar_expect_tx(full + s, (uint32_t)L.chunk_bytes);
                bulk_g2s(ring + (size_t)s * L.stage_stride, w + (size_t)c * L.chunk_bytes, (uint32_t)L.chunk_bytes, full + s);
            }
            // leave only when the last copies have landed (they have been waited for already unless a consumer gave up)
            for (int j = i > nstage ? i - nstage : 0; j < i; j++)
                mbar_wait<32>(full + j % nstage, (uint32_t)((j / nstage) & 1), fail, 2u);
        }
        return;
    }

    // ---- consumers
    mvs_stage_x(x, nb, xc, sh, sxs, L.xs, L.ss, warp, lane);
    bar_sync(1, MVS_CONS);
    const int g = lane >> 2, t = lane & 3;
    const int col = g < MVS_NDIG ? g : MVS_NDIG - 1; // the unused MMA columns repeat the last digit; their scale is zero
    const int8_t *xcol = xc + col * L.xs;
    const __half *scol = sh + col * L.ss;
    // 32 * 2^9 / 128^(2-d) for the columns 2t and 2t+1 (d = column, three digits): the "-32" of a Q6_K value against
    // sums that are stored times 2^-9
    const float r0 = t == 0 ? 1.0f : (t == 1 ? 16384.f : 0.f);
    const float r1 = t == 0 ? 128.f : 0.f;
    int i = 0;
    for (int c = blockIdx.x; c < n_chunks; c += gridDim.x, i++) {
        const int s = i % nstage;
        mbar_wait(full + s, (uint32_t)((i / nstage) & 1), fail, 3u);
        const uint8_t *rg = ring + (size_t)s * L.stage_stride + g * row_bytes;
        const uint8_t *rG = rg + 8 * row_bytes;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int b = warp; b < nb; b += MVS_NCW) {
            const uint8_t *bg = rg + b * Q6K_BYTES, *bG = rG + b * Q6K_BYTES;
            if (row_bytes & 2) q6k_block<2>(bg, bG, b, t, xcol, scol, sxs, r0, r1, acc);
            else if (b & 1) q6k_block<1>(bg, bG, b, t, xcol, scol, sxs, r0, r1, acc);
            else q6k_block<0>(bg, bG, b, t, xcol, scol, sxs, r0, r1, acc);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        float v0 = acc[0] + acc[1], v1 = acc[2] + acc[3];
        v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
        v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
        float *rb = red + (i & 1) * MVS_NCW * MVS_ROWS;
        if (t == 0) {
            rb[warp * MVS_ROWS + g] = v0;
            rb[warp * MVS_ROWS + g + 8] = v1;
        }
        // the buffer of chunk i is written again at chunk i + 2, after the barrier of chunk i + 1, which warp 0
        // reaches only when it has read this one
        bar_sync(1, MVS_CONS);
        if (warp == 0 && lane < MVS_ROWS) {
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < MVS_NCW; q++) sum += rb[q * MVS_ROWS + lane];
            if (*reinterpret_cast<volatile uint32_t *>(fail) != 0u) sum = __int_as_float(0x7fc00000);
            out[(size_t)c * MVS_ROWS + lane] = sum;
        }
    }
}

} // namespace

// True when the streamed kernel serves this shape: whole 16-row chunks that fit the ring at least three deep.
bool mv_q6k_stream_available(int64_t n_out, int64_t k) {
    if (k <= 0 || k % QK_K != 0 || n_out < MVS_ROWS) return false;
    if (k / QK_K * Q6K_BYTES * MVS_ROWS > MVS_MAX_CHUNK) return false;
    const MvsLayout L((int)k);
    return L.nstage >= 3;
}

// Rows [0, n_out - n_out % 16) of one activation row; the caller serves the tail rows with the row-per-warp kernel.
cudaError_t launch_mv_q6k_stream(const uint8_t *w, int n_out, int k, const float *x, float *out, cudaStream_t s) {
    static std::mutex mu;
    static bool ready[64] = {};
    static int sms[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    const MvsLayout L(k);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!ready[dev]) {
            e = cudaFuncSetAttribute(mv_q6k_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MVS_SMEM_MAX);
            if (e != cudaSuccess) return e;
            e = cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return e;
            ready[dev] = true;
        }
    }
    const int n_chunks = n_out / MVS_ROWS;
    if (n_chunks == 0) return cudaSuccess;
    const int grid = n_chunks < sms[dev] ? n_chunks : sms[dev];
    mv_q6k_stream_kernel<<<grid, MVS_THREADS, L.total, s>>>(w, x, out, k, n_chunks);
    return cudaGetLastError();
}
