// Plain Q6_K mat-vec for one activation row at a time, streamed: out[o] = W[o, :] . x.
// Reference: `ops::mul_mv`, src/ops/mv_id.rs:54-56 (kernel_mul_mv_q6_K_f32, src/ops/mv.metal), which the model
// calls once per decoded token for the vocabulary projection (src/model.rs:388-403): Q6_K [100352 x 3072],
// 253 MB that must all cross HBM, so the kernel is a pure bandwidth problem.
//
//   * One persistent CTA per SM.  A producer thread moves chunks of 16 weight rows (one MMA row tile,
//     16 * row_bytes contiguous bytes, always a multiple of 16) into a shared-memory ring with one bulk copy
//     each, completion counted on an mbarrier; as many stages as fit (five at k = 3072: 200 KB in flight per SM).
//   * Three groups of four consumer warps take the chunks of the ring in turn; inside a group the four warps
//     split the super-blocks of the chunk (the K dimension) and meet in a small shared array behind a named
//     barrier of their own, so a group never waits for another group.
//   * The six-bit values go to the integer tensor-core path as in the fused decode kernel: the activation row is
//     quantized once per CTA under the largest magnitude of each 256-wide block and carried as three signed
//     base-128 digits (21 bits), so the integer sums are exact; the "-32" offset is one f16 MMA per super-block
//     against the 16-wide activation sums.  With one token only three MMA columns would be in use, so two
//     16-wide sub-blocks share one k = 32 MMA: columns 0-2 carry the digits of the first (zeros in the k slots
//     of the second), columns 3-5 those of the second.  That halves the MMAs and the integer scale multiplies.
//     The digits of a warp's super-blocks never change, so they stay in registers for the whole launch.
//   * Lane group g works on rows 2g and 2g+1 of the chunk: with 2520-byte rows the eight rows of one load then
//     sit in disjoint shared-memory banks.
//   * Every wait is bounded.  A wait that gives up marks the CTA (a shared-memory word) and the rows it still
//     writes become NaN, so a launch that went wrong cannot pass for a result.
#include "stream_math.cuh"

namespace {

constexpr int MVS_ROWS = 16;
constexpr int MVS_NG = 3;                       // warp groups, each on its own chunk
constexpr int MVS_NCW = 4;                      // warps of a group: the K split of a chunk
constexpr int MVS_BPW = 3;                      // super-blocks per warp (their digits live in registers)
constexpr int MVS_MAX_NB = MVS_NCW * MVS_BPW;   // k <= 3072
constexpr int MVS_CONS = 32 * MVS_NCW * MVS_NG;
constexpr int MVS_THREADS = MVS_CONS + 32;
constexpr int MVS_NDIG = 3;
constexpr int MVS_MAX_STAGES = 8;
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
        o_red = o; o += 2 * MVS_NG * MVS_NCW * MVS_ROWS * 4;
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
    for (int b = warp; b < nb; b += MVS_NCW * MVS_NG) {
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

// k = 32 form: the two 16-wide sub-blocks c = 0 / 1 of a 32-value run share one MMA; columns 0-2 carry the
// digits of c = 0 (zeros in the k slots of c = 1), columns 3-5 those of c = 1.
template <int MIS>
__device__ __forceinline__ void q6k_block_k32(const uint8_t *bg, const uint8_t *bG, int t, const uint32_t (&xb0)[8],
                                              const uint32_t (&xb1)[8], uint32_t s0, uint32_t s1, float2 cs, float r0,
                                              float r1, const uint32_t (&sel)[4], float (&acc)[4]) {
    constexpr uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x30303030u;
    const int8_t *scg = reinterpret_cast<const int8_t *>(bg + 192);
    const int8_t *scG = reinterpret_cast<const int8_t *>(bG + 192);
    const float dg = lmoe_h2f(*reinterpret_cast<const uint16_t *>(bg + 208));
    const float dG = lmoe_h2f(*reinterpret_cast<const uint16_t *>(bG + 208));
    // the 16 sub-block scales of each row: four words, used twice (f16 for the offset MMA, bytes for the IMADs)
    uint32_t swg[4], swG[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        swg[q] = lds32<MIS>(bg, 192 + 4 * q);
        swG[q] = lds32<MIS>(bG, 192 + 4 * q);
    }
    float co[4];
    mma16816_z(co, sc_pair_half2(scg + 2 * t), sc_pair_half2(scG + 2 * t), sc_pair_half2(scg + 2 * t + 8),
               sc_pair_half2(scG + 2 * t + 8), s0, s1);
    int al[4] = {0, 0, 0, 0};
#pragma unroll
    for (int n = 0; n < 2; n++) {
        const uint32_t swg0 = swg[2 * n], swg1 = swg[2 * n + 1], swG0 = swG[2 * n], swG1 = swG[2 * n + 1];
        uint32_t qa_g[2], qb_g[2], qh_g[2], qa_G[2], qb_G[2], qh_G[2];
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const int l0 = 16 * c + 4 * t;
            qa_g[c] = lds32<MIS>(bg, 64 * n + l0); qb_g[c] = lds32<MIS>(bg, 64 * n + 32 + l0);
            qh_g[c] = lds32<MIS>(bg, 128 + 32 * n + l0);
            qa_G[c] = lds32<MIS>(bG, 64 * n + l0); qb_G[c] = lds32<MIS>(bG, 64 * n + 32 + l0);
            qh_G[c] = lds32<MIS>(bG, 128 + 32 * n + l0);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t a[4];
#pragma unroll
            for (int c = 0; c < 2; c++) {
                const uint32_t qg = (i & 1) ? qb_g[c] : qa_g[c], qG = (i & 1) ? qb_G[c] : qa_G[c];
                const uint32_t lg = (i & 2) ? (qg >> 4) : qg, lG = (i & 2) ? (qG >> 4) : qG;
                const uint32_t hg = i == 0 ? (qh_g[c] << 4) : (i == 1 ? (qh_g[c] << 2) : (i == 2 ? qh_g[c] : (qh_g[c] >> 2)));
                const uint32_t hG = i == 0 ? (qh_G[c] << 4) : (i == 1 ? (qh_G[c] << 2) : (i == 2 ? qh_G[c] : (qh_G[c] >> 2)));
                a[2 * c] = (lg & M4) | (hg & M2);
                a[2 * c + 1] = (lG & M4) | (hG & M2);
            }
            int f[4];
            imma16832_z(f, a[0], a[1], a[2], a[3], xb0[n * 4 + i], xb1[n * 4 + i]);
            const uint32_t wg = i < 2 ? swg0 : swg1, wG = i < 2 ? swG0 : swG1;
            int sgA, sgB, sGA, sGB;
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(sgA) : "r"(wg), "r"(0u), "r"(sel[(i & 1) * 2]));
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(sgB) : "r"(wg), "r"(0u), "r"(sel[(i & 1) * 2 + 1]));
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(sGA) : "r"(wG), "r"(0u), "r"(sel[(i & 1) * 2]));
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(sGB) : "r"(wG), "r"(0u), "r"(sel[(i & 1) * 2 + 1]));
            al[0] += sgA * f[0]; al[1] += sgB * f[1]; al[2] += sGA * f[2]; al[3] += sGB * f[3];
        }
    }
    acc[0] += dg * (cs.x * ((float)al[0] - r0 * co[0]));
    acc[1] += dg * (cs.y * ((float)al[1] - r1 * co[1]));
    acc[2] += dG * (cs.x * ((float)al[2] - r0 * co[2]));
    acc[3] += dG * (cs.y * ((float)al[3] - r1 * co[3]));
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
    uint32_t *fail = reinterpret_cast<uint32_t *>(empty + MVS_MAX_STAGES);
    uint8_t *ring = smem + L.o_ring;
    const int tid = threadIdx.x, warp_all = tid >> 5, lane = tid & 31;
    const int gi = warp_all / MVS_NCW, warp = warp_all % MVS_NCW;
    if (tid == 0) {
        for (int s = 0; s < nstage; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, MVS_NCW);
        }
        fail[0] = fail[1] = fail[2] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp_all == MVS_NCW * MVS_NG) {
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
    // ---- consumers: group gi takes chunks gi, gi + NG, ... of the CTA's sequence
    mvs_stage_x(x, nb, xc, sh, sxs, L.xs, L.ss, warp_all, lane);
    bar_sync(1, MVS_CONS);
    const int g = lane >> 2, t = lane & 3;
    const int dcol = g % 3, ccol = g / 3; // this lane's B column: digit, sub-block half (columns 6, 7: nothing)
    const int8_t *xcol = xc + dcol * L.xs;
    const __half *scol = sh + (g < 2 ? g : 2) * L.ss;
    // the "-32" of a Q6_K value: the sums sit in columns 0 (high part) and 1 (low part) times 2^-9; against the
    // column scales sx * 128^2 and sx * 128 that is a factor 32 * 2^9 / 128^(2-d)
    const float r0 = t == 0 ? 1.0f : 0.f;
    const float r1 = t == 0 ? 128.f : 0.f;
    // byte selectors of the sub-block scale of this lane's two accumulator columns (2t: half t >= 2, 2t+1: half t >= 1)
    uint32_t sel[4];
    {
        const int cA = t >= 2, cB = t >= 1;
#pragma unroll
        for (int ii = 0; ii < 2; ii++) {
            const int ia = 2 * ii + cA, ib = 2 * ii + cB;
            sel[ii * 2] = (uint32_t)(ia | ((8 | ia) * 0x1110));
            sel[ii * 2 + 1] = (uint32_t)(ib | ((8 | ib) * 0x1110));
        }
    }
    uint32_t xb0[MVS_BPW][8], xb1[MVS_BPW][8], s0r[MVS_BPW], s1r[MVS_BPW];
    float2 csr[MVS_BPW];
#pragma unroll
    for (int j = 0; j < MVS_BPW; j++) {
        const int b = warp + j * MVS_NCW;
        s0r[j] = s1r[j] = 0u;
        csr[j] = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < 8; q++) xb0[j][q] = xb1[j][q] = 0u;
        if (b < nb) {
#pragma unroll
            for (int n = 0; n < 2; n++)
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t v = g < 6 ? *reinterpret_cast<const uint32_t *>(xcol + 256 * b + 128 * n + 16 * ccol + 4 * t + 32 * q) : 0u;
                    xb0[j][n * 4 + q] = ccol == 0 ? v : 0u;
                    xb1[j][n * 4 + q] = ccol == 1 ? v : 0u;
                }
            s0r[j] = *reinterpret_cast<const uint32_t *>(scol + 16 * b + 2 * t);
            s1r[j] = *reinterpret_cast<const uint32_t *>(scol + 16 * b + 2 * t + 8);
            // column scales of columns 2t, 2t+1: digit (col % 3) for col < 6
            const int c0 = 2 * t, c1 = 2 * t + 1;
            csr[j].x = c0 < 6 ? sxs[8 * b + c0 % 3] : 0.f;
            csr[j].y = c1 < 6 ? sxs[8 * b + c1 % 3] : 0.f;
        }
    }
    const bool interleave = (row_bytes & 2) == 0; // rows 2g / 2g+1: the eight rows of a load sit in disjoint banks
    const int rowA = interleave ? 2 * g : g, rowB = interleave ? 2 * g + 1 : g + 8;
    int i = gi;
    for (int c = blockIdx.x + gi * gridDim.x; c < n_chunks; c += MVS_NG * gridDim.x, i += MVS_NG) {
        const int s = i % nstage;
        mbar_wait(full + s, (uint32_t)((i / nstage) & 1), fail, 3u);
        const uint8_t *rg = ring + (size_t)s * L.stage_stride + rowA * row_bytes;
        const uint8_t *rG = ring + (size_t)s * L.stage_stride + rowB * row_bytes;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < MVS_BPW; j++) {
            const int b = warp + j * MVS_NCW;
            if (b < nb) {
                const uint8_t *bg = rg + b * Q6K_BYTES, *bG = rG + b * Q6K_BYTES;
                if (row_bytes & 2) q6k_block_k32<2>(bg, bG, t, xb0[j], xb1[j], s0r[j], s1r[j], csr[j], r0, r1, sel, acc);
                else if (b & 1) q6k_block_k32<1>(bg, bG, t, xb0[j], xb1[j], s0r[j], s1r[j], csr[j], r0, r1, sel, acc);
                else q6k_block_k32<0>(bg, bG, t, xb0[j], xb1[j], s0r[j], s1r[j], csr[j], r0, r1, sel, acc);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty + s);
        float v0 = acc[0] + acc[1], v1 = acc[2] + acc[3];
        v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
        v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
        v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
        float *rb = red + (gi * 2 + ((i / MVS_NG) & 1)) * MVS_NCW * MVS_ROWS;
        if (t == 0) {
            rb[warp * MVS_ROWS + rowA] = v0;
            rb[warp * MVS_ROWS + rowB] = v1;
        }
        // the buffer is written again two chunks of the group later, after the group's next barrier, which warp 0
        // reaches only when it has read this one
        bar_sync(2 + gi, 32 * MVS_NCW);
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

// True when the streamed kernel serves this shape: at most 12 super-blocks per row (their digits fit the
// registers of a group) and a ring at least three chunks deep.
bool mv_q6k_stream_available(int64_t n_out, int64_t k) {
    if (k <= 0 || k % QK_K != 0 || n_out < MVS_ROWS) return false;
    if (k / QK_K > MVS_MAX_NB) return false;
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
