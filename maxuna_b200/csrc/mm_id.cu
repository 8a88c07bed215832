// Grouped (indexed) quantized GEMM on the 5th-generation tensor cores: for every
// expert e, the rows routed to e times W[e]^T, scattered back to [t, top_k, n_out].
//
// Reference: `ops::mul_mm_id{,_shared}`, src/ops/mm_id.rs:16-39 ->
// kernel_mul_mm_id_q{4,6}_K_f32_t, src/ops/mm_id.metal:492-647 (f16 operand
// tiles, f32 accumulation); per-expert lists from map0, src/ops/mm_id.metal:207-269.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0        raw loader : cp.async.bulk of the tile's quantized super-blocks
//   warps 1-8     dequant    : raw Q4_K/Q6_K -> f16 A tile (128 rows x 64 k) written in the
//                              tensor core's K-major 128-byte-swizzled layout
//   warp 9        B loader   : one bulk copy per stage of the routed rows' f16 activations
//                              (256 rows x 64 k), stored in global memory in tile order
//   warp 11       MMA        : one thread issues tcgen05.mma (M=128, N<=256, K=16),
//                              accumulators in TMEM (two buffers of 256 columns)
//   warps 12-15   epilogue   : tcgen05.ld, optional row scale, scatter to the output rows
// The weight tile is the A operand (M = 128 output features) and the routed
// rows are the N dimension, so ragged per-expert row counts cost only a
// rounding to 16.  Every wait is bounded; a wait that runs out records a flag
// and the kernel drains and exits.
#include <cuda.h> // CUtensorMap (types only; the encoder is fetched through the runtime)

#include "fused.cuh"
#include "kquant.cuh"

namespace {

constexpr int MM_M = 128;      // weight rows per tile
constexpr int MM_N = LMOE_MM_N; // routed rows per tile (192)
constexpr int MM_K = 64;       // k per pipeline stage (one 128-byte swizzle row of f16)
constexpr int MM_THREADS = 16 * 32;
constexpr int A_STAGE_BYTES = MM_M * MM_K * 2; // 16 KB
constexpr int B_STAGE_BYTES = MM_N * MM_K * 2; // 32 KB
constexpr uint32_t MM_SPIN = 1u << 24;

struct MmParams {
    const uint8_t *w;        // stack blocks
    int64_t expert_bytes;
    int dtype, n_expert, n_out, k;
    const uint8_t *xt;       // f16 activations, already in tile order (see gather_tiles_kernel)
    const uint32_t *tpe;     // [n_expert] rows per expert
    const int32_t *ids_map;  // [n_expert, map_stride] flat ids
    int map_stride;
    const int32_t *tiles;    // [n_tiles][8] = expert, first list index, valid rows, m0, row-tile slot
    const int32_t *n_tiles;  // device scalar
    const float *row_scale;  // per flat id, or NULL
    float *out;              // [t*top_k, n_out] f32
    uint32_t *flag;          // device flag words
    int n_stage, n_stage_b, raw_slots, raw_slot_bytes;
};

// ---- PTX helpers ---------------------------------------------------------------
__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint64_t *b, uint32_t c) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(c));
}
__device__ __forceinline__ void mb_arrive(uint64_t *b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ void mb_expect_tx(uint64_t *b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mb_try(uint64_t *b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and records the flag) when the limit runs out.
__device__ __forceinline__ bool mb_wait(uint64_t *b, uint32_t parity, uint32_t *flag, uint32_t where) {
    for (uint32_t i = 0; i < MM_SPIN; i++)
        if (mb_try(b, parity)) return true;
    if (atomicCAS(flag, 0u, (uint32_t)LMOE_FLAG_WAIT_TIMEOUT) == 0u) {
        flag[1] = 0x1000u + where;
        flag[2] = blockIdx.x;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(s32(dst)),
                 "l"(src), "r"(bytes), "r"(s32(bar)) : "memory");
}
// 2-D tiled TMA load global -> shared (x = byte offset inside the row, a multiple of 16; y = row).
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     s32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(s32(bar))
                 : "memory");
}
// Ask L2 to fetch a contiguous global range (16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes) {
    if ((reinterpret_cast<uintptr_t>(src) & 15u) != 0 || bytes == 0) return; // a hint only: skipped when not aligned
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc),
        "r"(accum) : "memory");
}
// The same with the A operand in tensor memory: 128 lanes (weight rows) x 8 columns (K = 16 as f16 pairs).
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc),
        "r"(accum) : "memory");
}
// 32 registers of every lane -> 32 columns of the warp's 32 tensor-memory lanes, then wait for the store.
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
        "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major, 128-byte-swizzled operand tile: rows of 64 f16 (128 B); groups of 8 rows are
// 1024 B apart; the 16-byte chunk c of row r sits at chunk position c ^ (r % 8).
__device__ __forceinline__ uint32_t swz_off(int r, int chunk) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
}
// Shared-memory matrix descriptor of such a tile (start address advanced by 32 B per K=16 step).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    const uint64_t lo = (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16);           // LBO (unused) = 16 B
    const uint64_t hi = (uint64_t)(1024 >> 4) | ((uint64_t)1 << 14) | ((uint64_t)2 << 29);   // SBO 1024 B, version 1, SWIZZLE_128B
    return lo | (hi << 32);
}

// ---- dequantisation into the swizzled A tile ------------------------------------
// (1024 + a | 1024 + b) - off, times scale, minus bias: exact integers in f16, one rounding in the fma
__device__ __forceinline__ uint32_t h2_sub_fma(uint32_t v, uint32_t off, __half2 s, __half2 m) {
    const __half2 q = __hsub2(*reinterpret_cast<const __half2 *>(&v), *reinterpret_cast<const __half2 *>(&off));
    const __half2 r = __hfma2(q, s, m);
    return *reinterpret_cast<const uint32_t *>(&r);
}

// Half a row-stage: the 32 weights of one Q4_K sub-block (sub-block 2j + half) -> 4 chunks of 8 halfs.
// Within a chunk the order is [0 2 1 3 4 6 5 7]; the activation rows use the same order.
__device__ __forceinline__ void dequant_q4k_row32(const uint8_t *blk, int j, int half, uint8_t *a_stage, int r) {
    const uint32_t dm = *reinterpret_cast<const uint32_t *>(blk);
    const float d = lmoe_h2f((uint16_t)(dm & 0xffff)), dmin = lmoe_h2f((uint16_t)(dm >> 16));
    int sc, mn;
    q4k_scale_min(blk + 4, 2 * j + half, sc, mn);
    const __half2 s = __float2half2_rn(d * (float)sc), m = __float2half2_rn(-dmin * (float)mn);
    const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * j);
    const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * j);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    // low nibble -> 1024 + q (magic 0x6400); high nibble in place -> 64 + q (magic 0x5400)
    const uint32_t mask = half ? 0x00F000F0u : 0x000F000Fu, magic = half ? 0x54005400u : 0x64006400u;
#pragma unroll
    for (int c = 0; c < 4; c++) {
        uint32_t o[4];
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t v = w[2 * c + h];
            o[2 * h] = h2_sub_fma((v & mask) | magic, magic, s, m);
            o[2 * h + 1] = h2_sub_fma(((v >> 8) & mask) | magic, magic, s, m);
        }
        *reinterpret_cast<uint4 *>(a_stage + swz_off(r, c + 4 * half)) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

__device__ __forceinline__ uint32_t ld32_a2(const uint8_t *p) {
    const uint16_t *q = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)q[0] | ((uint32_t)q[1] << 16);
}

// Half a row-stage of a Q6_K super-block: quarter js (k = 64*js .. 64*js+63) holds the groups
// i = 2*(js&1) + gi, gi = 0, 1, of half n = js>>1 (group i: 4 bits from ql, 2 bits (2i, 2i+1) from qh).
__device__ __forceinline__ void dequant_q6k_row32(const uint8_t *blk, int js, int gi, uint8_t *a_stage, int r) {
    const int n = js >> 1, hi_nib = js & 1; // groups 0,1 use the low nibbles of ql, groups 2,3 the high nibbles
    const float d = lmoe_h2f(*reinterpret_cast<const uint16_t *>(blk + 208));
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192) + 8 * n + 4 * hi_nib;
    const uint8_t *ql = blk + 64 * n, *qh = blk + 128 + 32 * n;
    // low nibble: 6-bit q lands in mantissa bits 0-5 (1024 + q); high nibble: bits 4-9 (1024 + 16 q)
    const uint32_t ml = hi_nib ? 0x00F000F0u : 0x000F000Fu, mh = hi_nib ? 0x03000300u : 0x00300030u;
    const uint32_t off = hi_nib ? 0x66006600u : 0x64206420u; // 1024 + 16*32 | 1024 + 32
    const float pw = hi_nib ? 0.0625f : 1.0f;
    const __half2 zero = __float2half2_rn(0.f);
    {
#pragma unroll
        for (int c = 0; c < 4; c++) { // 8 l-values per chunk
            const __half2 s = __float2half2_rn(d * (float)sc[2 * gi + (c >> 1)] * pw);
            uint32_t o[4];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int l = 8 * c + 4 * h;
                const uint32_t q = ld32_a2(ql + 32 * gi + l), hh = ld32_a2(qh + l);
                const uint32_t h02 = gi ? (hh << 2) : (hh << 4); // bytes 0, 2 of the word
                const uint32_t h13 = gi ? (hh >> 6) : (hh >> 4); // bytes 1, 3
                const uint32_t v02 = (q & ml) | (h02 & mh) | 0x64006400u;
                const uint32_t v13 = ((q >> 8) & ml) | (h13 & mh) | 0x64006400u;
                o[2 * h] = h2_sub_fma(v02, off, s, zero);
                o[2 * h + 1] = h2_sub_fma(v13, off, s, zero);
            }
            *reinterpret_cast<uint4 *>(a_stage + swz_off(r, 4 * gi + c)) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// ---- tile list -----------------------------------------------------------------------
// tiles[i] = {expert, first list index, valid rows, first weight row, row-tile slot, first sorted row};
// m tiles vary fastest so
// CTAs running side by side share the same activation rows in L2.
__global__ void __launch_bounds__(512) build_tiles_kernel(const uint32_t *__restrict__ tpe, int n_expert, int n_out,
                                                          int32_t *__restrict__ tiles, int32_t *__restrict__ n_tiles,
                                                          int max_tiles, int m_step) {
    __shared__ int pre[513], rpre[513];
    const int m_tiles = (n_out + m_step - 1) / m_step;
    const int e = threadIdx.x;
    const int cnt = e < n_expert ? (int)((tpe[e] + MM_N - 1) / MM_N) * m_tiles : 0;
    pre[e + 1] = cnt;
    rpre[e + 1] = e < n_expert ? (int)tpe[e] : 0;
    if (e == 0) pre[0] = rpre[0] = 0;
    __syncthreads();
    if (e == 0)
        for (int i = 1; i <= 512; i++) pre[i] += pre[i - 1];
    if (e == 32)
        for (int i = 1; i <= 512; i++) rpre[i] += rpre[i - 1];
    __syncthreads();
    // every thread takes tiles idx, idx + 512, ...; the expert of a tile is found in the prefix table
    const int total = min(pre[512], max_tiles);
    for (int o = threadIdx.x; o < total; o += 512) {
        int lo = 0, hi = n_expert - 1;
        while (lo < hi) { // last expert whose first tile is <= o
            const int mid = (lo + hi + 1) >> 1;
            if (pre[mid] <= o) lo = mid; else hi = mid - 1;
        }
        const int ex = lo, rel = o - pre[ex];
        const int nt = rel / m_tiles, m = rel - nt * m_tiles, n0 = nt * MM_N;
        const int rows = (int)tpe[ex];
        tiles[8 * o + 0] = ex;
        tiles[8 * o + 1] = n0;
        tiles[8 * o + 2] = min(MM_N, rows - n0);
        tiles[8 * o + 3] = m * m_step;
        tiles[8 * o + 4] = pre[ex] / m_tiles + nt;
        tiles[8 * o + 5] = rpre[ex] + n0; // first row of the tile in expert-sorted row order
    }
    if (e == 0) *n_tiles = min(pre[512], max_tiles);
}

// Routed rows -> the f16 B operand in TILE ORDER.  Row tile `slot` (MM_N routed rows of one expert)
// and k-stage ks (64 values) form one contiguous 24 KB block that is the exact shared-memory image
// of a B stage: row rr at rr*128 B, its 16-byte chunk c at position c ^ (rr & 7) (the 128-byte
// swizzle of the tensor core's K-major layout), 8 values per chunk in the order [0 2 1 3 4 6 5 7]
// (the order in which the dequantiser emits a chunk of weights).  A B stage is then ONE bulk copy.
// pos[flat id] = slot*MM_N + rr lets later kernels (SwiGLU) write rows in the same order.
__device__ __forceinline__ size_t tiled_off(int slot, int k_stages, int ks, int rr, int c) {
    return (((size_t)slot * k_stages + ks) * MM_N + rr) * 128 + ((size_t)(c ^ (rr & 7)) << 4);
}

template <bool XF16>
__global__ void __launch_bounds__(256) gather_tiles_kernel(const void *__restrict__ xv, int x_per_row, int top_k, int k,
                                                           const uint32_t *__restrict__ tpe, const int32_t *__restrict__ ids_map,
                                                           int map_stride, int n_expert, uint8_t *__restrict__ xt,
                                                           int32_t *__restrict__ pos, int32_t *__restrict__ spos,
                                                           int32_t *__restrict__ sfid) {
    __shared__ int warp_sum[8], warp_rows[8];
    __shared__ int slot0_s, row0_s;
    const int e = blockIdx.x;
    // slot of this expert's first row tile = number of row tiles of all earlier experts; likewise its
    // first row in expert-sorted order = number of rows of all earlier experts
    int part = 0, rpart = 0;
    for (int i = threadIdx.x; i < e; i += 256) {
        part += (int)((tpe[i] + MM_N - 1) / MM_N);
        rpart += (int)tpe[i];
    }
    for (int o = 16; o; o >>= 1) {
        part += __shfl_xor_sync(0xffffffffu, part, o);
        rpart += __shfl_xor_sync(0xffffffffu, rpart, o);
    }
    if ((threadIdx.x & 31) == 0) { warp_sum[threadIdx.x >> 5] = part; warp_rows[threadIdx.x >> 5] = rpart; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0, r = 0;
        for (int i = 0; i < 8; i++) { t += warp_sum[i]; r += warp_rows[i]; }
        slot0_s = t;
        row0_s = r;
    }
    __syncthreads();
    const int slot0 = slot0_s, srow0 = row0_s, rows = (int)tpe[e], k_stages = k / MM_K, chunks = k / 8;
    // one warp per routed row, eight rows of the expert in flight per block
    const int lane = threadIdx.x & 31;
    for (int i = blockIdx.y * 8 + (threadIdx.x >> 5); i < rows; i += gridDim.y * 8) {
        const int fid = ids_map[(size_t)e * map_stride + i];
        const size_t srow = (size_t)(x_per_row == 1 ? fid / top_k : fid) * k;
        const int slot = slot0 + i / MM_N, rr = i % MM_N;
        if (lane == 0) {
            if (pos) pos[fid] = slot * MM_N + rr;
            if (spos) spos[fid] = srow0 + i;
            if (sfid) sfid[srow0 + i] = fid;
        }
#pragma unroll 4
        for (int ci = lane; ci < chunks; ci += 32) {
            uint4 o;
            if (XF16) {
                // rows already in f16 (the expert-parallel wire format): only the order inside the chunk changes
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(static_cast<const __half *>(xv) + srow) + ci);
                o = make_uint4(__byte_perm(v.x, v.y, 0x5410), __byte_perm(v.x, v.y, 0x7632), __byte_perm(v.z, v.w, 0x5410),
                               __byte_perm(v.z, v.w, 0x7632));
            } else {
                const float *src = static_cast<const float *>(xv) + srow;
                const float4 a = __ldg(reinterpret_cast<const float4 *>(src) + 2 * ci);
                const float4 b = __ldg(reinterpret_cast<const float4 *>(src) + 2 * ci + 1);
                __align__(16) __half2 h[4] = {__floats2half2_rn(a.x, a.z), __floats2half2_rn(a.y, a.w),
                                              __floats2half2_rn(b.x, b.z), __floats2half2_rn(b.y, b.w)};
                o = *reinterpret_cast<const uint4 *>(h);
            }
            *reinterpret_cast<uint4 *>(xt + tiled_off(slot, k_stages, ci >> 3, rr, ci & 7)) = o;
        }
    }
}

struct MmSmem {
    int o_raw, o_a, o_b, o_bar, o_tmem, total;
    __host__ __device__ MmSmem(int n_stage, int n_stage_b, int raw_slots, int raw_slot_bytes) {
        int o = 0;
        o_a = o; o += n_stage * A_STAGE_BYTES;
        o_b = o; o += n_stage_b * B_STAGE_BYTES;
        o_raw = o; o += raw_slots * ((raw_slot_bytes + 127) / 128 * 128);
        o_bar = o; o += 8 * (4 * 8 + 2 * 4 + 4);
        o_tmem = o; o += 16;
        total = o + 1024; // slack to align the base to 1024 B
    }
};


// ---- the grouped GEMM kernel -------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(MM_THREADS, 1) mm_id_kernel(const __grid_constant__ MmParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const MmSmem L(P.n_stage, P.n_stage_b, P.raw_slots, P.raw_slot_bytes);
    uint8_t *a_st = smem + L.o_a, *b_st = smem + L.o_b, *raw = smem + L.o_raw;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.o_bar);
    uint64_t *a_full = bars, *b_full = bars + 8, *ab_empty = bars + 16, *raw_full = bars + 24, *raw_empty = bars + 28;
    uint64_t *acc_full = bars + 32, *acc_empty = bars + 34, *b_empty = bars + 36;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L.o_tmem);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int NS = P.n_stage, NSB = P.n_stage_b;
    const int n_tiles = *P.n_tiles;
    const int k_stages = P.k / MM_K;
    const int ts = DT == LMOE_Q4_K ? Q4K_BYTES : Q6K_BYTES;
    const int row_bytes = P.k / QK_K * ts;
    const int raw_slot_stride = (P.raw_slot_bytes + 127) / 128 * 128;

    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            mb_init(&a_full[s], 8);
            mb_init(&ab_empty[s], 1);
        }
        for (int s = 0; s < NSB; s++) {
            mb_init(&b_full[s], 1);
            mb_init(&b_empty[s], 1);
        }
        for (int s = 0; s < P.raw_slots; s++) {
            mb_init(&raw_full[s], 1);
            mb_init(&raw_empty[s], 8);
        }
        for (int s = 0; s < 2; s++) {
            mb_init(&acc_full[s], 1);
            mb_init(&acc_empty[s], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 11) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ================= raw loader =================
        uint32_t rg = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int e = P.tiles[8 * tile], m0 = P.tiles[8 * tile + 3];
            const int vrows = min(MM_M, P.n_out - m0);
            const uint8_t *wt = P.w + (size_t)e * P.expert_bytes + (size_t)m0 * row_bytes;
            if (DT == LMOE_Q4_K) {
                for (int sb = 0; sb < P.k / QK_K && ok; sb++, rg++) {
                    const int slot = rg % P.raw_slots;
                    ok = mb_wait(&raw_empty[slot], ((rg / P.raw_slots) & 1) ^ 1, P.flag, 1);
                    if (lane == 0) mb_expect_tx(&raw_full[slot], (uint32_t)vrows * Q4K_BYTES);
                    __syncwarp();
                    uint8_t *dst = raw + (size_t)slot * raw_slot_stride;
                    for (int r = lane; r < vrows; r += 32)
                        bulk_g2s(dst + r * Q4K_BYTES, wt + (size_t)r * row_bytes + (size_t)sb * Q4K_BYTES, Q4K_BYTES,
                                 &raw_full[slot]);
                }
            } else {
                const int slot = rg % P.raw_slots;
                ok = mb_wait(&raw_empty[slot], ((rg / P.raw_slots) & 1) ^ 1, P.flag, 1);
                if (lane == 0) {
                    const uint32_t bytes = (uint32_t)vrows * row_bytes;
                    mb_expect_tx(&raw_full[slot], bytes);
                    bulk_g2s(raw + (size_t)slot * raw_slot_stride, wt, bytes, &raw_full[slot]);
                }
                __syncwarp();
                rg++;
            }
        }
    } else if (warp <= 8) {
        // ================= dequant: thread = (weight row, half of the 64-wide stage) =================
        const int r = ((warp - 1) * 32 + lane) & 127, half = (warp - 1) >> 2;
        uint32_t g = 0, rg = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int m0 = P.tiles[8 * tile + 3];
            const bool rvalid = m0 + r < P.n_out;
            for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                const int s = g % NS;
                const int slot = rg % P.raw_slots;
                const bool first = DT == LMOE_Q4_K ? (ks & 3) == 0 : ks == 0;
                const bool last = DT == LMOE_Q4_K ? (ks & 3) == 3 : ks == k_stages - 1;
                if (first) ok = mb_wait(&raw_full[slot], (rg / P.raw_slots) & 1, P.flag, 2);
                ok = ok && mb_wait(&ab_empty[s], ((g / NS) & 1) ^ 1, P.flag, 3);
                uint8_t *ast = a_st + (size_t)s * A_STAGE_BYTES;
                const uint8_t *rs = raw + (size_t)slot * raw_slot_stride;
                if (rvalid) {
                    if (DT == LMOE_Q4_K) dequant_q4k_row32(rs + r * Q4K_BYTES, ks & 3, half, ast, r);
                    else dequant_q6k_row32(rs + (size_t)r * row_bytes + (ks >> 2) * Q6K_BYTES, ks & 3, half, ast, r);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        *reinterpret_cast<uint4 *>(ast + swz_off(r, c + 4 * half)) = make_uint4(0u, 0u, 0u, 0u);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mb_arrive(&a_full[s]);
                    if (last) mb_arrive(&raw_empty[slot]);
                }
                if (last) rg++;
            }
        }
    } else if (warp <= 10) {
        // ================= B loader: one bulk copy per stage (the operand is stored in tile order) =======
        if (warp == 9 && lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int nv = P.tiles[8 * tile + 2], slot = P.tiles[8 * tile + 4];
                const uint8_t *src = P.xt + (size_t)slot * k_stages * B_STAGE_BYTES;
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    const int s = g % NSB;
                    ok = mb_wait(&b_empty[s], ((g / NSB) & 1) ^ 1, P.flag, 4);
                    mb_expect_tx(&b_full[s], (uint32_t)nv * 128u);
                    bulk_g2s(b_st + (size_t)s * B_STAGE_BYTES, src + (size_t)ks * B_STAGE_BYTES, (uint32_t)nv * 128u, &b_full[s]);
                }
            }
        }
    } else if (warp == 11) {
        // ================= MMA issuer =================
        if (lane == 0) {
            uint32_t g = 0, it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
                const int nv = P.tiles[8 * tile + 2];
                const int npad = (nv + 15) & ~15;
                const uint32_t idesc = (1u << 4) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(MM_M >> 4) << 24);
                const uint32_t buf = it & 1;
                ok = mb_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, P.flag, 5);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256;
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    const int s = g % NS, sb = g % NSB;
                    ok = mb_wait(&a_full[s], (g / NS) & 1, P.flag, 6);
                    ok = ok && mb_wait(&b_full[sb], (g / NSB) & 1, P.flag, 7);
                    tc_fence_after();
                    const uint64_t ad = umma_desc(s32(a_st + (size_t)s * A_STAGE_BYTES));
                    const uint64_t bd = umma_desc(s32(b_st + (size_t)sb * B_STAGE_BYTES));
#pragma unroll
                    for (int kk = 0; kk < MM_K / 16; kk++)
                        tc_mma_f16(d_tmem, ad + 2 * kk, bd + 2 * kk, idesc, (ks | kk) != 0 ? 1u : 0u);
                    tc_commit(&ab_empty[s]); // frees both stages when these MMAs have read them
                    tc_commit(&b_empty[sb]);
                }
                tc_commit(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else {
        // ================= epilogue: TMEM -> registers -> scattered rows =================
        const int q = warp & 3; // TMEM lane quadrant this warp may read
        const int m = 32 * q + lane;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
            const int e = P.tiles[8 * tile], l0 = P.tiles[8 * tile + 1], nv = P.tiles[8 * tile + 2], m0 = P.tiles[8 * tile + 3];
            const int32_t *list = P.ids_map + (size_t)e * P.map_stride + l0;
            const uint32_t buf = it & 1;
            // destination rows and their scales are fetched while the tile is still being multiplied
            int fids[MM_N / 32];
            float scs[MM_N / 32];
#pragma unroll
            for (int c = 0; c < MM_N / 32; c++) {
                const int my = 32 * c + lane;
                fids[c] = my < nv ? list[my] : 0;
            }
#pragma unroll
            for (int c = 0; c < MM_N / 32; c++) scs[c] = (P.row_scale && 32 * c + lane < nv) ? P.row_scale[fids[c]] : 1.0f;
            ok = mb_wait(&acc_full[buf], (it >> 1) & 1, P.flag, 8);
            tc_fence_after();
            const bool mvalid = m0 + m < P.n_out;
#pragma unroll
            for (int c = 0; c < MM_N / 32; c++) {
                const int cb = 32 * c;
                if (cb >= nv) break;
                uint32_t v[32];
                tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + buf * 256 + cb, v);
                const int myfid = fids[c];
                const float mysc = scs[c];
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int fid = __shfl_sync(0xffffffffu, myfid, j);
                    const float sc = __shfl_sync(0xffffffffu, mysc, j);
                    if (cb + j < nv && mvalid) P.out[(size_t)fid * P.n_out + m0 + m] = __uint_as_float(v[j]) * sc;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mb_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 11) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}



// ================= gate + up in one pass, SwiGLU in the epilogue =========================
// Same tile list as above, but a CTA multiplies one block of routed rows by 128 gate rows AND the
// matching 128 up rows (two accumulators of MM_N tensor-memory columns), so every activation stage is
// loaded once for both projections.  The quantized rows are staged by TMA tile loads; the dequantising
// threads (one per weight row and projection) write their f16 values straight into TENSOR MEMORY
// (tcgen05.st: lane = weight row, 32 columns = the 64 values of a k-stage) and the tensor core takes its
// A operand from there, so the dequantised tile never passes through shared memory: per k-stage that
// removes a 32 KB write and a 32 KB read from the shared-memory traffic that bounded the loop.
// Tensor-memory columns: [0, MM_N) gate accumulator, [MM_N, 2 MM_N) up accumulator,
// [2 MM_N, 2 MM_N + 128) the A operand: 2 stages x 2 projections x 32 columns.
// Epilogue: act = silu(gate) * up, f32, one row per routed row.
//   warps 0-7   dequant (thread = (projection, weight row))     warp 8   B loader (bulk copy)
//   warp 9      MMA issuer     warps 10-13  epilogue     warp 14  loader of the quantized columns
constexpr int GU_THREADS = 15 * 32;
constexpr int GU_NS = 2;
constexpr int GU_RAW_SLOT = MM_M * Q4K_BYTES; // one super-block column of 128 rows of one projection
constexpr int GU_RAW_SLOTS = 4;               // (column parity, projection)
constexpr int GU_ACC_UP = MM_N;               // first tensor-memory column of the up accumulator
constexpr int GU_A_COL0 = 2 * MM_N;           // first column of the A operand stages
static_assert(GU_A_COL0 + GU_NS * 2 * 32 <= 512, "tensor memory: two accumulators and the operand stages must fit 512 columns");

struct GuParams {
    // 2-D views of the gate / up stacks as bytes: [n_expert * n_out rows][row_bytes], box = 144 bytes x 128 rows
    CUtensorMap map_g, map_u;
    const uint8_t *wg, *wu; // gate / up stacks (Q4_K)
    int64_t expert_bytes;
    int n_out, k;
    const uint8_t *xt;
    const int32_t *ids_map;
    int map_stride;
    const int32_t *tiles, *n_tiles;
    float *act; // [rows, n_out] f32
    int sorted; // rows of `act` in expert-sorted order (tile table entry 5) instead of by flat id
    uint32_t *flag;
};

// 64 weights (sub-block pair j) of one Q4_K row -> the 32 words of the row's k-stage, in the order the
// activation rows are stored (8-value chunks as [0 2 1 3 4 6 5 7]): word 4c + i = chunk c, pair i.
__device__ __forceinline__ void dequant_q4k_regs(const uint4 hdr, const uint4 qa, const uint4 qb, int j, uint32_t (&o)[32]) {
    const float d = lmoe_h2f((uint16_t)(hdr.x & 0xffff)), dmin = lmoe_h2f((uint16_t)(hdr.x >> 16));
    uint32_t sc[2], mn[2];
    q4k_unpack_scales(hdr.y, hdr.z, hdr.w, sc[0], sc[1], mn[0], mn[1]);
    const uint32_t scw = sc[j >> 1] >> (16 * (j & 1)), mnw = mn[j >> 1] >> (16 * (j & 1));
    const __half2 s_lo = __float2half2_rn(d * (float)(scw & 0xff)), m_lo = __float2half2_rn(-dmin * (float)(mnw & 0xff));
    const __half2 s_hi = __float2half2_rn(d * (float)((scw >> 8) & 0xff)), m_hi = __float2half2_rn(-dmin * (float)((mnw >> 8) & 0xff));
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
    for (int c = 0; c < 4; c++) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t v = w[2 * c + h], v8 = v >> 8;
            // low nibbles (sub-block 2j): chunks 0-3; high nibbles (sub-block 2j+1): chunks 4-7
            o[4 * c + 2 * h] = h2_sub_fma((v & 0x000F000Fu) | 0x64006400u, 0x64006400u, s_lo, m_lo);
            o[4 * c + 2 * h + 1] = h2_sub_fma((v8 & 0x000F000Fu) | 0x64006400u, 0x64006400u, s_lo, m_lo);
            o[16 + 4 * c + 2 * h] = h2_sub_fma((v & 0x00F000F0u) | 0x54005400u, 0x54005400u, s_hi, m_hi);
            o[16 + 4 * c + 2 * h + 1] = h2_sub_fma((v8 & 0x00F000F0u) | 0x54005400u, 0x54005400u, s_hi, m_hi);
        }
    }
}

// Epilogue of the 32-column chunks [c0, c1) of a gate/up tile for the 32 weight rows of tensor-memory quadrant q:
// act = silu(gate) * up, one routed row per tile column.
__device__ __forceinline__ void gu_epilogue_chunks(const GuParams &P, uint32_t tmem_base, int tile, int q, int lane, int c0, int c1) {
    const int e = P.tiles[8 * tile], l0 = P.tiles[8 * tile + 1], nv = P.tiles[8 * tile + 2], m0 = P.tiles[8 * tile + 3];
    const int m = 32 * q + lane;
    const bool mvalid = m0 + m < P.n_out;
    for (int c = c0; c < c1; c++) {
        const int cb = 32 * c;
        if (cb >= nv) break;
        uint32_t vg[32], vu[32];
        tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + cb, vg);
        tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + GU_ACC_UP + cb, vu);
        if (P.sorted) {
            // rows in expert-sorted order: consecutive tile columns are consecutive rows
            float *dst = P.act + (size_t)(P.tiles[8 * tile + 5] + cb) * P.n_out + m0 + m;
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float gv = __uint_as_float(vg[j]), uv = __uint_as_float(vu[j]);
                const float a = __fdividef(gv, 1.0f + __expf(-gv)) * uv;
                if (cb + j < nv && mvalid) dst[(size_t)j * P.n_out] = a;
            }
        } else {
            const int32_t *list = P.ids_map + (size_t)e * P.map_stride + l0;
            const int myfid = cb + lane < nv ? list[cb + lane] : 0;
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int fid = __shfl_sync(0xffffffffu, myfid, j);
                const float gv = __uint_as_float(vg[j]), uv = __uint_as_float(vu[j]);
                const float a = __fdividef(gv, 1.0f + __expf(-gv)) * uv;
                if (cb + j < nv && mvalid) P.act[(size_t)fid * P.n_out + m0 + m] = a;
            }
        }
    }
}

// Chunks of a tile's epilogue by warp: the four epilogue warps take the first GU_EPI_OWN chunks, the dequantising
// warps of the gate projection the next two, those of the up projection the last two.  An epilogue of 192 columns
// by four warps alone takes as long as a fifth of the tile's multiplies, and nothing can be multiplied meanwhile
// (there is one accumulator set); the dequantising warps have nothing to do at that moment.
constexpr int GU_EPI_OWN = 2;
static_assert(MM_N == 32 * (GU_EPI_OWN + 4), "the epilogue split covers six 32-column chunks");

__global__ void __launch_bounds__(GU_THREADS, 1) mm_gateup_kernel(const __grid_constant__ GuParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *b_st = smem;
    uint8_t *raw = b_st + GU_NS * B_STAGE_BYTES; // quantized super-block columns, TMA-staged
    uint64_t *bars = reinterpret_cast<uint64_t *>(raw + GU_RAW_SLOTS * GU_RAW_SLOT);
    // full[s]: eight dequant warps + the B loader's expect_tx arrival; empty[s]: one tcgen05.commit;
    // raw_full[i]: the TMA load's bytes; raw_empty[i]: the four dequant warps of the slot's projection
    uint64_t *full = bars, *empty = bars + 4, *raw_full = bars + 8, *raw_empty = bars + 12, *acc_full = bars + 16, *acc_empty = bars + 17;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 18);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = *P.n_tiles;
    const int k_stages = P.k / MM_K;
    const int row_bytes = P.k / QK_K * Q4K_BYTES;

    if (tid == 0) {
        for (int s = 0; s < GU_NS; s++) {
            mb_init(&full[s], 9);
            mb_init(&empty[s], 1);
        }
        for (int i = 0; i < GU_RAW_SLOTS; i++) {
            mb_init(&raw_full[i], 1);
            mb_init(&raw_empty[i], 4);
        }
        mb_init(acc_full, 1);
        mb_init(acc_empty, 12); // the four epilogue warps and the eight dequantising warps that share the epilogue
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // ---------------- dequant: thread = (projection, weight row) ----------------
        // The row's 144-byte super-block sits in the TMA-staged column of its projection (pitch 144 bytes:
        // eight consecutive rows cover all banks for 16-byte reads).
        const int sub = warp >> 2, r = tid & 127;
        const int n_blk = P.k / QK_K;
        uint32_t g = 0, col = 0, it_e = 0; // k-stage counter, super-block column counter of this projection, tiles done
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int m0 = P.tiles[8 * tile + 3];
            const bool rvalid = m0 + r < P.n_out;
            for (int b = 0; b < n_blk && ok; b++, col++) {
                const int slot = sub + 2 * (col & 1);
                ok = mb_wait(&raw_full[slot], (col >> 1) & 1, P.flag, 2);
                const uint4 *blk = reinterpret_cast<const uint4 *>(raw + (size_t)slot * GU_RAW_SLOT + r * Q4K_BYTES);
                const uint4 hdr = blk[0];
#pragma unroll
                for (int j = 0; j < 4; j++, g++) {
                    const int s = g % GU_NS;
                    ok = ok && mb_wait(&empty[s], ((g / GU_NS) & 1) ^ 1, P.flag, 3);
                    uint32_t o[32];
                    if (rvalid) {
                        dequant_q4k_regs(hdr, blk[1 + 2 * j], blk[2 + 2 * j], j, o);
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; c++) o[c] = 0u;
                    }
                    // lane = weight row of this warp's quadrant; the stage's 32 columns of this projection
                    tc_fence_after();
                    tc_st32(tmem_base + ((uint32_t)(32 * (warp & 3)) << 16) + GU_A_COL0 + (uint32_t)(s * 2 + sub) * 32u, o);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mb_arrive(&full[s]);
                }
                // the column is consumed: hand its slot back to the loader
                __syncwarp();
                if (lane == 0) mb_arrive(&raw_empty[slot]);
            }
            // this warp's share of the tile's epilogue (columns beyond the first 64, if the tile has them)
            if (P.tiles[8 * tile + 2] > 32 * (GU_EPI_OWN + 2 * sub) && ok) {
                ok = mb_wait(acc_full, it_e & 1, P.flag, 10);
                tc_fence_after();
                gu_epilogue_chunks(P, tmem_base, tile, warp & 3, lane, GU_EPI_OWN + 2 * sub, GU_EPI_OWN + 2 * sub + 2);
                tc_fence_before();
            }
            __syncwarp();
            if (lane == 0) mb_arrive(acc_empty);
            it_e++;
        }
    } else if (warp == 14) {
        // ---------------- raw loader: one TMA tile load per (super-block column, projection) ----------------
        if (lane == 0) {
            const int n_blk = P.k / QK_K;
            uint32_t col = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int e = P.tiles[8 * tile], m0 = P.tiles[8 * tile + 3];
                const int y = e * P.n_out + m0;
                for (int b = 0; b < n_blk && ok; b++, col++) {
#pragma unroll
                    for (int sub = 0; sub < 2; sub++) {
                        const int slot = sub + 2 * (col & 1);
                        ok = ok && mb_wait(&raw_empty[slot], ((col >> 1) & 1) ^ 1, P.flag, 1);
                        mb_expect_tx(&raw_full[slot], (uint32_t)GU_RAW_SLOT);
                        tma_load_2d(raw + (size_t)slot * GU_RAW_SLOT, sub ? &P.map_u : &P.map_g, b * Q4K_BYTES, y, &raw_full[slot]);
                    }
                }
            }
        }
    } else if (warp == 8) {
        // ---------------- B loader ----------------
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int nv = P.tiles[8 * tile + 2], slot = P.tiles[8 * tile + 4];
                const uint8_t *src = P.xt + (size_t)slot * k_stages * B_STAGE_BYTES;
                {
                    // the quantized rows of this CTA's next tile are two contiguous ranges: have L2 fetch them now
                    const int nt = tile + gridDim.x;
                    if (nt < n_tiles) {
                        const int ne = P.tiles[8 * nt], nm0 = P.tiles[8 * nt + 3];
                        const int nrows = min(MM_M, P.n_out - nm0);
                        const size_t off = (size_t)ne * P.expert_bytes + (size_t)nm0 * row_bytes;
                        bulk_prefetch_l2(P.wg + off, (uint32_t)(nrows * row_bytes) & ~15u);
                        bulk_prefetch_l2(P.wu + off, (uint32_t)(nrows * row_bytes) & ~15u);
                    }
                }
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    const int s = g % GU_NS;
                    ok = mb_wait(&empty[s], ((g / GU_NS) & 1) ^ 1, P.flag, 4);
                    mb_expect_tx(&full[s], (uint32_t)nv * 128u);
                    bulk_g2s(b_st + (size_t)s * B_STAGE_BYTES, src + (size_t)ks * B_STAGE_BYTES, (uint32_t)nv * 128u, &full[s]);
                }
            }
        }
    } else if (warp == 9) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // The issuing thread runs a dependent chain of scalar instructions, so everything it can
            // know ahead is precomputed: operand descriptors per ring slot, slot and phase as counters.
            uint64_t bd[GU_NS];
#pragma unroll
            for (int s = 0; s < GU_NS; s++) bd[s] = umma_desc(s32(b_st + (size_t)s * B_STAGE_BYTES));
            uint32_t it = 0, ph = 0;
            int s = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
                const int nv = P.tiles[8 * tile + 2];
                const int npad = (nv + 15) & ~15;
                const uint32_t idesc = (1u << 4) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(MM_M >> 4) << 24);
                ok = mb_wait(acc_empty, (it & 1) ^ 1, P.flag, 5);
                tc_fence_after();
                for (int ks = 0; ks < k_stages && ok; ks++) {
                    ok = mb_wait(&full[s], ph, P.flag, 6);
                    tc_fence_after();
                    // slot-indexed descriptors without dynamic register indexing
                    const uint64_t b0 = s == 0 ? bd[0] : bd[GU_NS - 1];
                    // A operand: 8 tensor-memory columns per K = 16 step of the stage's gate / up block
                    const uint32_t a0 = tmem_base + GU_A_COL0 + (uint32_t)s * 64u, a1 = a0 + 32u;
#pragma unroll
                    for (int kk = 0; kk < MM_K / 16; kk++) {
                        tc_mma_f16_ts(tmem_base, a0 + 8 * kk, b0 + 2 * kk, idesc, (ks | kk) != 0 ? 1u : 0u);
                        tc_mma_f16_ts(tmem_base + GU_ACC_UP, a1 + 8 * kk, b0 + 2 * kk, idesc, (ks | kk) != 0 ? 1u : 0u);
                    }
                    tc_commit(&empty[s]);
                    if (++s == GU_NS) { s = 0; ph ^= 1; }
                }
                tc_commit(acc_full);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: act = silu(gate) * up (the first chunks; see GU_EPI_OWN) ----------------
        const int q = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
            ok = mb_wait(acc_full, it & 1, P.flag, 8);
            tc_fence_after();
            gu_epilogue_chunks(P, tmem_base, tile, q, lane, 0, GU_EPI_OWN);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mb_arrive(acc_empty);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}


// ================= down projection (Q6_K), 128 weight rows per CTA tile ===========================
// A tile's quantized rows are four contiguous runs of 32 rows (one per tensor-memory lane quadrant); each run
// is ONE bulk copy into a ring of shared-memory slots, so no load/store unit moves weight bytes.  Sixteen
// dequantising warps (quadrant x 16-wide l range x nibble half) read their row's block out of shared memory
// - at whatever 2-byte alignment the 210-byte blocks fall, re-aligned with funnel shifts - convert 32 weights
// each with one scale per 16 and store them straight into TENSOR MEMORY (tcgen05.st), from where the tensor
// core takes its A operand (TS-form tcgen05.mma).  Two accumulator buffers let the epilogue of a tile overlap
// the multiplies of the next.
// Tensor-memory columns: [0, MM_N) and [MM_N, 2 MM_N) accumulator buffers, [2 MM_N, 2 MM_N + 128) four A stages.
//   warps 0-15 dequant (quadrant = warp & 3, l half = (warp >> 2) & 1, nibble half = warp >> 3)
//   warp 16 loader of the quantized runs    warp 17 B loader    warp 18 MMA issuer    warps 19-22 epilogue
//   warp 23 forwarder: a B stage has landed -> the A stage's barrier (the issuer waits once per k-stage)
constexpr int DN_DQ_WARPS = 16;
constexpr int DN_THREADS = (DN_DQ_WARPS + 8) * 32;
constexpr int DN_NSA = 4, DN_NSB = 2;
constexpr int DN_RUN_ROWS = 32;                 // rows of one bulk-copied run (= one lane quadrant)
constexpr int DN_RAW_SLOTS = 6;                 // ring of runs: the four of the current tile and two ahead
constexpr int DN_MAX_NB = 4;                    // super-blocks per row this kernel stages (k <= 1024)
constexpr int DN_A_COL0 = 2 * MM_N;
static_assert(DN_A_COL0 + DN_NSA * 32 <= 512, "tensor memory: two accumulators and four operand stages must fit 512 columns");

struct DnParams {
    const uint8_t *w; // down stack (Q6_K)
    int64_t expert_bytes;
    int n_out, k;
    const uint8_t *xt;
    const int32_t *ids_map;
    int map_stride;
    const int32_t *tiles, *n_tiles;
    const float *row_scale;
    float *out; // [rows, n_out]
    int sorted; // rows of `out` in expert-sorted order, unscaled, instead of scaled rows by flat id
    uint32_t *flag;
    int raw_slot_bytes; // 32 rows of quantized blocks + slack for re-aligning reads
};

// 16 bytes at byte offset `o` (even) from a 4-byte aligned base, as four words
__device__ __forceinline__ void dn_read16(const uint8_t *base4, int o, uint32_t (&out)[4]) {
    const uint32_t *w = reinterpret_cast<const uint32_t *>(base4) + (o >> 2);
    const uint32_t sh = (uint32_t)(o & 3) * 8u;
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3], w4 = w[4];
    out[0] = __funnelshift_r(w0, w1, sh);
    out[1] = __funnelshift_r(w1, w2, sh);
    out[2] = __funnelshift_r(w2, w3, sh);
    out[3] = __funnelshift_r(w3, w4, sh);
}

// The fields of (row, half n, l range lh) of the Q6_K block that starts `sh` bytes (even) after the 4-byte
// aligned address base4: 16 bytes of ql for groups {0,2} and for groups {1,3}, 16 bytes of qh, the eight
// scales of the half, d.
struct DnFields {
    uint32_t qa[4], qb[4], qh[4], s0, s1;
    float d;
};
__device__ __forceinline__ void dn_fields(const uint8_t *base4, int sh, int n, int lh, DnFields &F) {
    dn_read16(base4, sh + 64 * n + 16 * lh, F.qa);
    dn_read16(base4, sh + 64 * n + 32 + 16 * lh, F.qb);
    dn_read16(base4, sh + 128 + 32 * n + 16 * lh, F.qh);
    {
        const int o = sh + 192 + 8 * n;
        const uint32_t *w = reinterpret_cast<const uint32_t *>(base4) + (o >> 2);
        const uint32_t s = (uint32_t)(o & 3) * 8u;
        const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
        F.s0 = __funnelshift_r(w0, w1, s);
        F.s1 = __funnelshift_r(w1, w2, s);
    }
    {
        const int o = sh + 208;
        const uint32_t w = reinterpret_cast<const uint32_t *>(base4)[o >> 2];
        F.d = lmoe_h2f((uint16_t)((w >> ((o & 2) * 8)) & 0xffffu));
    }
}

// Groups 2*hn and 2*hn+1 (low nibbles: hn = 0, the even k-stage of the half; high nibbles: hn = 1, the odd
// one) of one (row, l range): 32 weights -> o[0..7] = the 16 values of group 2*hn (stage chunks 2*lh,
// 2*lh + 1), o[8..15] = the 16 of group 2*hn + 1 (chunks 4 + 2*lh, 5 + 2*lh); 8-value chunks as [0 2 1 3 4 6 5 7].
__device__ __forceinline__ void dn_dequant32(const DnFields &F, int hn, int lh, uint32_t (&o)[16]) {
    const uint32_t ml = hn ? 0x00F000F0u : 0x000F000Fu, mh = hn ? 0x03000300u : 0x00300030u;
    const uint32_t off = hn ? 0x66006600u : 0x64206420u; // 1024 + 16*32 | 1024 + 32
    const uint32_t scw = hn ? F.s1 : F.s0;
#pragma unroll
    for (int g1 = 0; g1 < 2; g1++) { // group 2*hn + g1
        // scale 2*(2*hn + g1) + lh of this half: byte 2*g1 + lh of the word
        const int sb = (int)(int8_t)((scw >> (8 * (2 * g1 + lh))) & 0xff);
        const __half2 sc = __float2half2_rn(F.d * (float)sb * (hn ? 0.0625f : 1.0f));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t q = g1 ? F.qb[j] : F.qa[j], hh = F.qh[j];
            // the two qh bits of group 2*hn + g1 sit four positions higher for hn = 1, and so does the place they go
            // to (next to a nibble that stays in the high half of its byte): the shifts are the same, the mask differs
            const uint32_t h02 = g1 ? (hh << 2) : (hh << 4), h13 = g1 ? (hh >> 6) : (hh >> 4);
            const uint32_t v02 = (q & ml) | (h02 & mh) | 0x64006400u;
            const uint32_t v13 = ((q >> 8) & ml) | (h13 & mh) | 0x64006400u;
            const __half2 d02 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&v02), *reinterpret_cast<const __half2 *>(&off)), sc);
            const __half2 d13 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&v13), *reinterpret_cast<const __half2 *>(&off)), sc);
            o[8 * g1 + 2 * j] = *reinterpret_cast<const uint32_t *>(&d02);
            o[8 * g1 + 2 * j + 1] = *reinterpret_cast<const uint32_t *>(&d13);
        }
    }
}

// 8 registers of every lane -> 8 columns of the warp's 32 tensor-memory lanes
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__global__ void __launch_bounds__(DN_THREADS, 1) mm_down_kernel(const __grid_constant__ DnParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *b_st = smem;
    uint8_t *raw = b_st + DN_NSB * B_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(raw + DN_RAW_SLOTS * P.raw_slot_bytes);
    uint64_t *a_full = bars, *a_empty = bars + 4, *b_full = bars + 8, *raw_full = bars + 12,
             *raw_empty = bars + 18, *acc_full = bars + 24, *acc_empty = bars + 26;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 28);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = *P.n_tiles;
    const int k_stages = P.k / MM_K, n_blk = P.k / QK_K;
    const int row_bytes = n_blk * Q6K_BYTES;

    if (tid == 0) {
        // The thread that issues the multiplies pays 100-300 cycles for every synchronising instruction, and its chain
        // per k-stage was the kernel's period: it waits on ONE barrier per stage (a_full: the eight warps of the
        // stage's nibble half + the forwarder's word that the B stage has landed) and commits to ONE (a_empty:
        // the stage's multiplies are done), which the dequantising warps (stage g - 4), the B loader (stage g - 2)
        // and the forwarder (stage g - 4) all wait on.
        for (int s = 0; s < DN_NSA; s++) {
            mb_init(&a_full[s], DN_DQ_WARPS / 2 + 1);
            mb_init(&a_empty[s], 1);
        }
        for (int s = 0; s < DN_NSB; s++) mb_init(&b_full[s], 1);
        for (int s = 0; s < DN_RAW_SLOTS; s++) {
            mb_init(&raw_full[s], 1);
            mb_init(&raw_empty[s], 4); // the four dequant warps of the run's quadrant
        }
        for (int s = 0; s < 2; s++) {
            mb_init(&acc_full[s], 1);
            mb_init(&acc_empty[s], 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == DN_DQ_WARPS + 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DN_DQ_WARPS) {
        // ---------------- dequant: thread = (weight row, 16-wide l range, nibble half) ----------------
        const int q = warp & 3, lh = (warp >> 2) & 1, hn = warp >> 3;
        const int r = 32 * q + lane; // row of the tile = tensor-memory lane
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
            const int m0 = P.tiles[8 * tile + 3];
            const bool rvalid = m0 + r < P.n_out;
            const uint32_t c = it * 4u + (uint32_t)q; // sequence number of this quadrant's run
            const int slot = (int)(c % DN_RAW_SLOTS);
            ok = mb_wait(&raw_full[slot], (c / DN_RAW_SLOTS) & 1, P.flag, 2);
            // the row's blocks: 4-byte aligned address below the block start, plus the offset inside it
            const uint8_t *rowp = raw + (size_t)slot * P.raw_slot_bytes + (size_t)lane * row_bytes;
            const uint32_t g0 = it * (uint32_t)k_stages; // first k-stage of the tile in the kernel-wide count
            for (int b = 0; b < n_blk && ok; b++) {
                const uint8_t *blk = rowp + b * Q6K_BYTES;
                const uint8_t *base4 = reinterpret_cast<const uint8_t *>(reinterpret_cast<uintptr_t>(blk) & ~(uintptr_t)3);
                const int sh = (int)(reinterpret_cast<uintptr_t>(blk) & 3u);
#pragma unroll 1
                for (int n = 0; n < 2; n++) {
                    uint32_t o[16];
                    if (rvalid) {
                        DnFields F;
                        dn_fields(base4, sh, n, lh, F);
                        dn_dequant32(F, hn, lh, o);
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) o[i] = 0u;
                    }
                    const uint32_t g = g0 + (uint32_t)(4 * b + 2 * n + hn); // this thread's k-stage of the pair
                    const int sa = (int)(g % DN_NSA);
                    ok = ok && mb_wait(&a_empty[sa], ((g / DN_NSA) & 1) ^ 1, P.flag, 3);
                    tc_fence_after();
                    const uint32_t ta = tmem_base + ((uint32_t)(32 * q) << 16) + DN_A_COL0 + (uint32_t)sa * 32u;
                    tc_st8(ta + 8u * lh, o);            // group 2*hn: chunks 2*lh, 2*lh + 1
                    tc_st8(ta + 16u + 8u * lh, o + 8);  // group 2*hn + 1: chunks 4 + 2*lh, 5 + 2*lh
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mb_arrive(&a_full[sa]);
                }
            }
            // the run is consumed: hand its slot back to the loader
            __syncwarp();
            if (lane == 0) mb_arrive(&raw_empty[slot]);
        }
    } else if (warp == DN_DQ_WARPS) {
        // ---------------- loader of the quantized runs: one bulk copy per (tile, quadrant) ----------------
        if (lane == 0) {
            uint32_t c = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int e = P.tiles[8 * tile], m0 = P.tiles[8 * tile + 3];
                const uint8_t *tw = P.w + (size_t)e * P.expert_bytes + (size_t)m0 * row_bytes;
                for (int q = 0; q < 4 && ok; q++, c++) {
                    const int slot = (int)(c % DN_RAW_SLOTS);
                    ok = mb_wait(&raw_empty[slot], ((c / DN_RAW_SLOTS) & 1) ^ 1, P.flag, 1);
                    int rows = P.n_out - m0 - DN_RUN_ROWS * q;
                    rows = rows < 0 ? 0 : (rows > DN_RUN_ROWS ? DN_RUN_ROWS : rows);
                    const uint32_t bytes = (uint32_t)(rows * row_bytes); // even row count: a multiple of 16 bytes
                    if (bytes) {
                        mb_expect_tx(&raw_full[slot], bytes);
                        bulk_g2s(raw + (size_t)slot * P.raw_slot_bytes, tw + (size_t)q * DN_RUN_ROWS * row_bytes, bytes, &raw_full[slot]);
                    } else {
                        mb_arrive(&raw_full[slot]);
                    }
                }
            }
        }
    } else if (warp == DN_DQ_WARPS + 1) {
        // ---------------- B loader ----------------
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int nv = P.tiles[8 * tile + 2], slot = P.tiles[8 * tile + 4];
                const uint8_t *src = P.xt + (size_t)slot * k_stages * B_STAGE_BYTES;
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    const int s = g % DN_NSB;
                    // the B stage is free when the multiplies of stage g - DN_NSB are done
                    if (g >= DN_NSB) ok = mb_wait(&a_empty[(g - DN_NSB) % DN_NSA], ((g - DN_NSB) / DN_NSA) & 1, P.flag, 4);
                    mb_expect_tx(&b_full[s], (uint32_t)nv * 128u);
                    bulk_g2s(b_st + (size_t)s * B_STAGE_BYTES, src + (size_t)ks * B_STAGE_BYTES, (uint32_t)nv * 128u, &b_full[s]);
                }
            }
        }
    } else if (warp == DN_DQ_WARPS + 7) {
        // ---------------- forwarder ----------------
        // Its word for stage g must fall into phase g / DN_NSA of a_full[g % DN_NSA]: it is given once the multiplies
        // of stage g - DN_NSA are done (the dequantising warps wait for the same event before they store).
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                for (int ks = 0; ks < k_stages && ok; ks++, g++) {
                    ok = mb_wait(&b_full[g % DN_NSB], (g / DN_NSB) & 1, P.flag, 7);
                    if (g >= DN_NSA) ok = ok && mb_wait(&a_empty[g % DN_NSA], ((g - DN_NSA) / DN_NSA) & 1, P.flag, 9);
                    mb_arrive(&a_full[g % DN_NSA]);
                }
            }
        }
    } else if (warp == DN_DQ_WARPS + 2) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t g = 0, it = 0;
            bool ok = true;
            const uint64_t bd0 = umma_desc(s32(b_st)); // B stage i: this plus i stages in the 16-byte address field
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
                const int nv = P.tiles[8 * tile + 2];
                const int npad = (nv + 15) & ~15;
                const uint32_t idesc = (1u << 4) | ((uint32_t)(npad >> 3) << 17) | ((uint32_t)(MM_M >> 4) << 24);
                const uint32_t buf = it & 1;
                ok = mb_wait(&acc_empty[buf], ((it >> 1) & 1) ^ 1, P.flag, 5);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * MM_N;
                // a tile has a multiple of four k-stages (k is a multiple of 256): the ring slots of a stage follow from
                // its index in the tile, and the loop is unrolled over them
                for (int k4 = 0; k4 < k_stages / 4 && ok; k4++, g += 4) {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        ok = ok && mb_wait(&a_full[u], (g / DN_NSA) & 1, P.flag, 6);
                        tc_fence_after();
                        const uint32_t a_tmem = tmem_base + DN_A_COL0 + (uint32_t)u * 32u;
                        const uint64_t bd = bd0 + (uint64_t)((u % DN_NSB) * (B_STAGE_BYTES >> 4));
#pragma unroll
                        for (int kk = 0; kk < MM_K / 16; kk++)
                            tc_mma_f16_ts(d_tmem, a_tmem + 8 * kk, bd + 2 * kk, idesc, (k4 | u | kk) != 0 ? 1u : 0u);
                        tc_commit(&a_empty[u]); // the stage's multiplies are done: its A and B stages are free
                    }
                }
                tc_commit(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: rows of one accumulator buffer ----------------
        const int q = warp & 3; // tensor-memory lane quadrant this warp may read
        const int m = 32 * q + lane;
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, it++) {
            const int e = P.tiles[8 * tile], l0 = P.tiles[8 * tile + 1], nv = P.tiles[8 * tile + 2], m0 = P.tiles[8 * tile + 3];
            const int32_t *list = P.ids_map + (size_t)e * P.map_stride + l0;
            const uint32_t buf = it & 1;
            const int mrow = m0 + m;
            const bool mvalid = mrow < P.n_out;
            ok = mb_wait(&acc_full[buf], (it >> 1) & 1, P.flag, 8);
            tc_fence_after();
            for (int cb = 0; cb < nv; cb += 32) {
                uint32_t v[32];
                tc_ld32(tmem_base + ((uint32_t)(32 * q) << 16) + buf * MM_N + cb, v);
                if (P.sorted) {
                    // rows in expert-sorted order, unscaled: consecutive tile columns are consecutive rows
                    float *dst = P.out + (size_t)(P.tiles[8 * tile + 5] + cb) * P.n_out + mrow;
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (cb + j < nv && mvalid) dst[(size_t)j * P.n_out] = __uint_as_float(v[j]);
                } else {
                    const int my = cb + lane;
                    const int myfid = my < nv ? list[my] : 0;
                    const float mysc = (P.row_scale && my < nv) ? P.row_scale[myfid] : 1.0f;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int fid = __shfl_sync(0xffffffffu, myfid, j);
                        const float sc = __shfl_sync(0xffffffffu, mysc, j);
                        if (cb + j < nv && mvalid) P.out[(size_t)fid * P.n_out + mrow] = __uint_as_float(v[j]) * sc;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mb_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == DN_DQ_WARPS + 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
}

} // namespace

// ---- host side ---------------------------------------------------------------------------
static int mm_m_tiles(int64_t n_out) { return (int)((n_out + MM_M - 1) / MM_M); }

int64_t mm_max_tiles(int64_t rows, int64_t n_expert, int64_t n_out) {
    return ((rows + MM_N - 1) / MM_N + n_expert) * mm_m_tiles(n_out);
}

// Pipeline shape for a stack; false when the tile does not fit in shared memory.
static bool mm_shape(int dtype, int64_t k, int &n_stage, int &n_stage_b, int &raw_slots, int &raw_slot_bytes) {
    if (dtype == LMOE_Q4_K) {
        n_stage = 3; n_stage_b = 4; raw_slots = 2; raw_slot_bytes = MM_M * Q4K_BYTES;
    } else {
        n_stage = 2; n_stage_b = 2; raw_slots = 1; raw_slot_bytes = (int)(MM_M * (k / QK_K) * Q6K_BYTES);
    }
    return MmSmem(n_stage, n_stage_b, raw_slots, raw_slot_bytes).total <= 227 * 1024;
}

bool mm_id_kernel_available(int dtype, int64_t n_out, int64_t k) {
    int a, b, c, d;
    if (dtype != LMOE_Q4_K && dtype != LMOE_Q6_K) return false;
    if (k <= 0 || k % QK_K) return false;
    if (dtype == LMOE_Q6_K && (n_out & 1)) return false; // whole-tile bulk copies need 16-byte multiples
    return mm_shape(dtype, k, a, b, c, d);
}

size_t mm_tiles_bytes(int64_t rows, int64_t n_expert, int64_t n_out) {
    return lmoe_align_up((size_t)mm_max_tiles(rows, n_expert, n_out) * 32 + 256, 256);
}

// Bytes of the tile-ordered f16 operand for `rows` routed rows of width k.
size_t mm_tiled_bytes(int64_t rows, int64_t n_expert, int64_t k) {
    return lmoe_align_up((size_t)((rows + MM_N - 1) / MM_N + n_expert) * (size_t)(k / MM_K) * B_STAGE_BYTES, 256);
}

cudaError_t launch_gather_tiles(const void *x, int x_f16, int x_per_row, int top_k, int k, const uint32_t *tpe,
                                const int32_t *ids_map, int map_stride, int n_expert, void *xt, int32_t *pos,
                                int32_t *spos, int32_t *sfid, cudaStream_t s) {
    // enough blocks per expert to cover the device even when one expert holds all the rows
    const int gy = n_expert >= 64 ? 16 : (n_expert >= 8 ? 128 : 1024);
    if (x_f16)
        gather_tiles_kernel<true><<<dim3(n_expert, gy), 256, 0, s>>>(x, x_per_row, top_k, k, tpe, ids_map, map_stride, n_expert,
                                                                     static_cast<uint8_t *>(xt), pos, spos, sfid);
    else
        gather_tiles_kernel<false><<<dim3(n_expert, gy), 256, 0, s>>>(x, x_per_row, top_k, k, tpe, ids_map, map_stride, n_expert,
                                                                      static_cast<uint8_t *>(xt), pos, spos, sfid);
    return cudaGetLastError();
}

// A 2-D TMA view of an expert stack as bytes: [rows][row_bytes], boxes of box_bytes x box_rows.  The encoder
// is a driver entry point, fetched through the runtime (no link against the driver library).
static lmoe_status make_rows_map(CUtensorMap *map, const void *base, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes,
                                 uint32_t box_rows) {
    typedef CUresult (*encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static encode_fn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
            q != cudaDriverEntryPointSuccess)
            return lmoe_fail(LMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        encode = reinterpret_cast<encode_fn>(fn);
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || row_bytes % 16 || box_bytes % 16 || box_bytes > 256 || box_rows > 256)
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "expert stack layout does not fit a TMA tile (16-byte alignment of base, row and box)");
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return lmoe_fail(LMOE_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)rc);
    return LMOE_OK;
}

// One grouped projection. `xt`: the f16 operand in tile order; `tiles_ws`: mm_tiles_bytes() scratch
// whose last 256 bytes hold the tile count; `flag`: 4 device words (zero = clean).
lmoe_status launch_mm_id(const lmoe_expert_stack *st, const void *xt, const uint32_t *tpe, const int32_t *ids_map, int64_t map_stride, int64_t list_rows,
                         const float *row_scale, float *out, void *tiles_ws, uint32_t *flag, cudaStream_t stream) {
    MmParams P;
    if (!mm_shape(st->dtype, st->k, P.n_stage, P.n_stage_b, P.raw_slots, P.raw_slot_bytes))
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "grouped GEMM tile for k=%lld does not fit in shared memory", (long long)st->k);
    if (st->n_expert > 512) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "grouped GEMM supports at most 512 experts");
    const int64_t max_tiles = mm_max_tiles(list_rows, st->n_expert, st->n_out);
    int32_t *tiles = static_cast<int32_t *>(tiles_ws);
    int32_t *n_tiles = reinterpret_cast<int32_t *>(static_cast<uint8_t *>(tiles_ws) + lmoe_align_up((size_t)max_tiles * 32, 256));
    build_tiles_kernel<<<1, 512, 0, stream>>>(tpe, (int)st->n_expert, (int)st->n_out, tiles, n_tiles, (int)max_tiles, MM_M);
    LMOE_LAUNCH_CHECK("build_tiles_kernel");
    P.w = st->blocks(); P.expert_bytes = st->expert_bytes();
    P.dtype = st->dtype; P.n_expert = (int)st->n_expert; P.n_out = (int)st->n_out; P.k = (int)st->k;
    P.xt = static_cast<const uint8_t *>(xt);
    P.tpe = tpe; P.ids_map = ids_map; P.map_stride = (int)map_stride;
    P.tiles = tiles; P.n_tiles = n_tiles; P.row_scale = row_scale; P.out = out; P.flag = flag;
    const MmSmem L(P.n_stage, P.n_stage_b, P.raw_slots, P.raw_slot_bytes);
    static thread_local int c_dev = -1, c_sms = 0;
    int dev = 0;
    LMOE_CUDA(cudaGetDevice(&dev));
    if (dev != c_dev) {
        LMOE_CUDA(cudaDeviceGetAttribute(&c_sms, cudaDevAttrMultiProcessorCount, dev));
        LMOE_CUDA(cudaFuncSetAttribute(mm_id_kernel<LMOE_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        LMOE_CUDA(cudaFuncSetAttribute(mm_id_kernel<LMOE_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        c_dev = dev;
    }
    if (st->dtype == LMOE_Q4_K) mm_id_kernel<LMOE_Q4_K><<<c_sms, MM_THREADS, L.total, stream>>>(P);
    else mm_id_kernel<LMOE_Q6_K><<<c_sms, MM_THREADS, L.total, stream>>>(P);
    LMOE_LAUNCH_CHECK("mm_id_kernel");
    return LMOE_OK;
}

// gate and up of one expert block in one kernel, SwiGLU applied: act[rows, ff] (f32).
lmoe_status launch_mm_gateup(const lmoe_expert_stack *gate, const lmoe_expert_stack *up, const void *xt,
                             const uint32_t *tpe, const int32_t *ids_map, int64_t map_stride, int64_t list_rows,
                             float *act, int sorted, void *tiles_ws, uint32_t *flag, cudaStream_t stream) {
    if (gate->dtype != LMOE_Q4_K || up->dtype != LMOE_Q4_K)
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "the fused gate/up kernel is built for Q4_K stacks");
    if (gate->n_expert > 512) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "grouped GEMM supports at most 512 experts");
    const int64_t max_tiles = mm_max_tiles(list_rows, gate->n_expert, gate->n_out);
    int32_t *tiles = static_cast<int32_t *>(tiles_ws);
    int32_t *n_tiles = reinterpret_cast<int32_t *>(static_cast<uint8_t *>(tiles_ws) + lmoe_align_up((size_t)max_tiles * 32, 256));
    build_tiles_kernel<<<1, 512, 0, stream>>>(tpe, (int)gate->n_expert, (int)gate->n_out, tiles, n_tiles, (int)max_tiles, MM_M);
    LMOE_LAUNCH_CHECK("build_tiles_kernel");
    GuParams P;
    const uint64_t rb = (uint64_t)(gate->k / QK_K) * Q4K_BYTES, rows_all = (uint64_t)gate->n_expert * gate->n_out;
    lmoe_status mst = make_rows_map(&P.map_g, gate->blocks(), rb, rows_all, Q4K_BYTES, MM_M);
    if (mst) return mst;
    if ((mst = make_rows_map(&P.map_u, up->blocks(), rb, rows_all, Q4K_BYTES, MM_M))) return mst;
    P.wg = gate->blocks(); P.wu = up->blocks(); P.expert_bytes = gate->expert_bytes();
    P.n_out = (int)gate->n_out; P.k = (int)gate->k; P.xt = static_cast<const uint8_t *>(xt);
    P.ids_map = ids_map; P.map_stride = (int)map_stride; P.tiles = tiles; P.n_tiles = n_tiles; P.act = act; P.sorted = sorted; P.flag = flag;
    const int smem = GU_NS * B_STAGE_BYTES + GU_RAW_SLOTS * GU_RAW_SLOT + 256 + 1024;
    static thread_local int c_dev = -1, c_sms = 0;
    int dev = 0;
    LMOE_CUDA(cudaGetDevice(&dev));
    if (dev != c_dev) {
        LMOE_CUDA(cudaDeviceGetAttribute(&c_sms, cudaDevAttrMultiProcessorCount, dev));
        LMOE_CUDA(cudaFuncSetAttribute(mm_gateup_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        c_dev = dev;
    }
    mm_gateup_kernel<<<c_sms, GU_THREADS, smem, stream>>>(P);
    LMOE_LAUNCH_CHECK("mm_gateup_kernel");
    return LMOE_OK;
}

// The down projection: Q6_K stacks with at most DN_MAX_NB super-blocks per row and an even row count
// (run copies are multiples of 16 bytes); optional per-row scale in the epilogue.
bool mm_down_available(const lmoe_expert_stack *down) {
    return down->dtype == LMOE_Q6_K && down->k / QK_K <= DN_MAX_NB && (down->n_out & 1) == 0 && down->n_expert <= 512;
}

lmoe_status launch_mm_down(const lmoe_expert_stack *down, const void *xt, const uint32_t *tpe, const int32_t *ids_map,
                           int64_t map_stride, int64_t list_rows, const float *row_scale, float *out, int sorted,
                           void *tiles_ws, uint32_t *flag, cudaStream_t stream) {
    if (!mm_down_available(down))
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "the down kernel needs a Q6_K stack with k <= %d, even n_out and at most 512 experts",
                         DN_MAX_NB * QK_K);
    const int64_t max_tiles = mm_max_tiles(list_rows, down->n_expert, down->n_out);
    int32_t *tiles = static_cast<int32_t *>(tiles_ws);
    int32_t *n_tiles = reinterpret_cast<int32_t *>(static_cast<uint8_t *>(tiles_ws) + lmoe_align_up((size_t)max_tiles * 32, 256));
    build_tiles_kernel<<<1, 512, 0, stream>>>(tpe, (int)down->n_expert, (int)down->n_out, tiles, n_tiles, (int)max_tiles, MM_M);
    LMOE_LAUNCH_CHECK("build_tiles_kernel");
    DnParams P;
    P.w = down->blocks(); P.expert_bytes = down->expert_bytes(); P.n_out = (int)down->n_out; P.k = (int)down->k;
    P.xt = static_cast<const uint8_t *>(xt); P.ids_map = ids_map; P.map_stride = (int)map_stride;
    P.tiles = tiles; P.n_tiles = n_tiles; P.row_scale = row_scale; P.out = out; P.sorted = sorted; P.flag = flag;
    // a slot holds 32 rows; re-aligning reads may touch up to 20 bytes past the last block
    P.raw_slot_bytes = (int)lmoe_align_up((size_t)DN_RUN_ROWS * down->row_bytes() + 32, 128);
    const int smem = DN_NSB * B_STAGE_BYTES + DN_RAW_SLOTS * P.raw_slot_bytes + 512 + 1024;
    static thread_local int c_dev = -1, c_sms = 0, c_smem = 0;
    int dev = 0;
    LMOE_CUDA(cudaGetDevice(&dev));
    if (dev != c_dev || smem > c_smem) {
        LMOE_CUDA(cudaDeviceGetAttribute(&c_sms, cudaDevAttrMultiProcessorCount, dev));
        LMOE_CUDA(cudaFuncSetAttribute(mm_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        c_dev = dev;
        c_smem = smem;
    }
    mm_down_kernel<<<c_sms, DN_THREADS, smem, stream>>>(P);
    LMOE_LAUNCH_CHECK("mm_down_kernel");
    return LMOE_OK;
}
