// Fused MoE block for decode batches (t <= 64 tokens per launch): routing, the
// gate/up mat-vecs with SwiGLU, the down mat-vec, the weighted combine and the
// shared expert in ONE persistent kernel.
//
// Reference semantics: `MoeBlock::forward`, src/moe.rs:73-78, with the mv_id
// branch of `FusedExperts::forward`, src/moe.rs:221-323 (kernels
// kernel_mul_mv_id_q4_K/q6_K_f32_v, src/ops/mv.metal:181-290, 413-504),
// `silu_mul` (src/ops/silu_mul.metal:57-72), `combine`
// (src/ops/combine.metal:70-97) and `SharedExpert::forward`, src/moe.rs:342-344.
// With caller-supplied expert ids and weights the same kernel is the
// `ExpertFfn::forward` seam of src/moe.rs:19-21 (routing skipped).
//
// Structure (the path is HBM-bound: 70.5 MB per token at the production shape)
//   * grid = every SM x 2 CTAs, launched cooperatively so all CTAs are resident;
//     CTA = 4 consumer warps + 1 producer warp + 1 epilogue warp.  (The kernel is written for NG groups of
//     four consumer warps per CTA; geometries with two to four groups in one CTA per SM were measured and did
//     not beat one group in each of two CTAs up to 16 tokens, so only NG = 1 is instantiated.)
//   * The producer streams raw super-blocks global -> shared with 1-D bulk
//     copies (cp.async.bulk + mbarrier) through a 3-stage ring: each DISTINCT
//     selected expert (and the shared expert) is read from HBM exactly once per
//     call, however many tokens selected it.
//   * Consumers feed the 4/6-bit fields to the integer tensor-core path: a Q4_K nibble (after one mask)
//     or a Q6_K value (low nibble | two high bits) is one unsigned byte of the A operand of mma.sync
//     u8 x s8 -> s32 (m16n8k32 per 32-wide Q4_K sub-block, m16n8k16 per 16-wide Q6_K sub-block; 16 weight
//     rows per MMA).  The activations are B: each value is quantized under the largest magnitude of its
//     256-wide block and carried as signed base-128 digits in separate MMA columns, so the integer sums are
//     exact: three digits (21 bits) for two tokens per pass up to 8 tokens, two digits (15 bits) for three
//     tokens per pass beyond.  The integer sub-block scales multiply the sums (IMAD), and the float factors
//     (d of the row, digit scale of the column) come in once per super-block.  The Q4_K "min" term and the
//     Q6_K "-32" offset are one f16 MMA per super-block against per-sub-block activation sums, which are kept
//     as scaled integers so that they fit f16 whatever the magnitude of the input.
//   * Work units (8 gate+8 up rows, or 32 down rows, of one expert) are split
//     contiguously over CTAs; the K dimension of a unit is split over the four
//     consumer warps, whose partial sums go through mbarrier-guarded shared-memory
//     buffers to the epilogue warp: it adds them in a fixed order and writes the
//     SwiGLU activations / weighted partial rows, so the consumer warps never wait
//     for one another inside a phase.
//   * Phases are separated by bounded grid barriers (up to 16 tokens the one
//     between the two projections is replaced by per-pass completion counters);
//     the producer runs ahead of them (weights do not depend on them), which keeps
//     HBM busy across phases.  Once a wait has given up, every later wait of the launch
//     returns at once, and the producer leaves only when its last copies have landed.
//   * The down projection writes weighted partial rows; a last phase sums the
//     K+1 partials of every output element in slot order, so the result is
//     deterministic without float atomics.
#include "fused.cuh"
#include "kquant.cuh"
#include "route_math.cuh"
#include "stream_math.cuh"

namespace {

constexpr int CW = 4;             // consumer warps of a group: the K split of one unit
constexpr int DOWN_ROWS = 32;     // rows of a down-projection unit: two MMA row tiles
// Launch geometry by the number of groups NG (units a CTA works on at the same time): one group means two
// CTAs per SM with a 3-stage ring each; more groups share one CTA per SM, one activation cache and a longer ring.
template <int NG_>
struct Cfg {
    static constexpr int NG = NG_;
    static constexpr int NCW = CW * NG;                 // consumer warps
    static constexpr int THREADS = 32 * (NCW + 2);      // + producer warp + epilogue warp
    static constexpr int CONS = 32 * NCW;
    static constexpr int RING = 32 * (NCW + 1);         // consumers + producer
    static constexpr int EPI = 32 * (NCW + 1);          // consumers + epilogue warp
    static constexpr int NSTAGE = NG == 1 ? 3 : (NG == 2 ? 4 : 6);
    static constexpr int NRED = NG == 1 ? 3 : 2 * NG;   // K-split partial buffers between the consumers and the epilogue warp
    static constexpr int MIN_CTAS = NG == 1 ? 2 : 1;
};
constexpr int SYNC_PASS0 = 32;   // layer sync words: [0] grid barrier, [1] exit count, [32 + pass] phase-1 units done
constexpr int SYNC_WORDS = SYNC_PASS0 + 1024;
constexpr int DEC_MAX_T = 64;
constexpr int MAX_NTOK = 4;
#ifndef LMOE_DEC_PASS_FLAG_MAX_T
#define LMOE_DEC_PASS_FLAG_MAX_T 16 // up to this many tokens, phase 2 of a pass starts on the pass's own counter
#endif
#ifndef LMOE_DEC_V23_FROM_T
#define LMOE_DEC_V23_FROM_T 9       // from this many tokens: two digits per activation, three tokens per pass
#endif

struct DecodeParams {
    const float *x;
    float *out;
    uint32_t *ids_out;
    float *w_out;
    const float *router, *bias;
    const uint32_t *ext_ids; // caller-supplied routing decision [t, top_k] (ids >= n_expert: empty slot) or NULL
    const float *ext_w;
    const uint8_t *gate, *up, *down, *sh_gate, *sh_up, *sh_down;
    int t, hidden, ff, n_expert, top_k;
    float scale;
    int norm, has_shared;
    int sh_t0, sh_nt; // the shared expert serves tokens [sh_t0, sh_t0 + sh_nt) (all of them unless the caller narrows it)
    uint32_t *ctrl;   // workspace: [0..3] device flag (zeroed by the launch with first_launch set)
    uint32_t *sync;   // owned by the layer, zero between launches: [0] grid barrier, [1] exit count, [32..] per-pass counts
    int first_launch;
    float *logits;    // [t][n_expert]
    uint32_t *ids_ws; // [t][top_k] routing decision, written by the CTA that ranked the token
    float *w_ws;
    float *act_f;     // [t*(top_k+1)][ff] SwiGLU activations
    float *ypart;     // [t*(top_k+1)][hidden]
};

// Shared-memory layout (bytes), computed identically on host and device.
struct DecLayout {
    int stage_bytes, xs, ss;
    int o_ring, o_xc, o_s, o_sx, o_red, o_bar, o_ids, o_w, o_cnt, o_off, o_plist, o_act, o_ppre, total;
    __host__ __device__ DecLayout(int hidden, int ff, int n_expert, int t, int top_k, int ncol, int ncw, int nstage, int nred) {
        const int row4 = hidden / QK_K * Q4K_BYTES, row6 = ff / QK_K * Q6K_BYTES;
        int sb = 16 * row4 > DOWN_ROWS * row6 ? 16 * row4 : DOWN_ROWS * row6;
        stage_bytes = (sb + 127) / 128 * 128;
        const int kmax = hidden > ff ? hidden : ff;
        xs = kmax + 32; // bytes per column (+32 B: four columns of a half-warp's loads cover all 32 banks)
        int nsb = hidden / 32 > ff / 16 ? hidden / 32 : ff / 16;
        ss = (nsb + 15) / 16 * 16;
        const int tk = t * top_k;
        int o = 0;
        o_ring = o; o += nstage * stage_bytes;
        o_xc = o;
        int xc_bytes = ncol * xs;
        const int sel_bytes = 2 * n_expert * 4 + 2 * ncw * 32 * 4; // routing scratch aliases the activation cache
        if (sel_bytes > xc_bytes) xc_bytes = sel_bytes;
        o += (xc_bytes + 15) / 16 * 16;
        o_s = o; o += ncol * ss * 2;
        o_sx = o; o += (kmax / QK_K) * 8 * 4; // [256-block][8 columns] digit scales
        // the K-split partial buffers (phases 1-2) share their space with two routing tables that are
        // only alive while the token lists are built: expert counts and the id list
        int red_bytes = nred * CW * 16 * ncol * 4;
        if (red_bytes < (n_expert + tk) * 4) red_bytes = (n_expert + tk) * 4;
        o_red = o; o_cnt = o; o_ids = o + n_expert * 4;
        o += (red_bytes + 15) / 16 * 16;
        o_bar = o; o += ((2 * nstage + 2 * nred) * 8 + 127) / 128 * 128;
        o_w = o; o += tk * 4;
        o_off = o; o += (n_expert + 2) / 2 * 2 * 2;
        o_plist = o; o += (tk + 1) / 2 * 2 * 2;
        o_act = o; o += (tk + 2) / 2 * 2 * 2;
        o_ppre = o; o += (tk + 2) / 2 * 2 * 2;
        total = (o + 15) / 16 * 16;
    }
};

// Index guard for values read back from the routing tables, on the paths that run once per unit or less
// (the producer's source addresses, the list build): a value outside its range is recorded in the device
// flag (code, value, CTA) and the access it would have fed is skipped or redirected, never made.
__device__ __noinline__ void dec_bad_index(uint32_t *ctrl, uint32_t code, uint32_t val) {
    if (atomicCAS(ctrl, 0u, (uint32_t)LMOE_FLAG_BAD_INDEX) == 0u) {
        ctrl[1] = code;
        ctrl[2] = val;
        ctrl[3] = blockIdx.x;
    }
}
#define DEC_GUARD(cond, code, val) ((cond) ? true : (dec_bad_index(P.ctrl, (code), (uint32_t)(val)), false))

// Grid-wide barrier among the consumer threads of all CTAs (thread 0 of each
// CTA arrives).  `target` = arrivals expected so far in this launch.
__device__ __forceinline__ void grid_barrier(uint32_t *ctrl, uint32_t *sync, uint32_t target, int tid, int cons_threads,
                                             int first_id, int first_count) {
    // the CTA barrier orders every thread's stores before thread 0's fence, which is cumulative: one fence per CTA
    bar_sync(first_id, first_count); // phases 1/2: the epilogue warp arrives here once its stores are fenced
    if (tid == 0) {
        __threadfence();
        atomicAdd(&sync[0], 1u);
        uint32_t i = 0;
        while (ld_acquire(&sync[0]) < target) {
            if ((i & 1023u) == 1023u && *reinterpret_cast<volatile uint32_t *>(ctrl) != 0u) break;
            if (++i > SPIN_LIMIT) {
                if (atomicCAS(ctrl, 0u, (uint32_t)LMOE_FLAG_WAIT_TIMEOUT) == 0u) {
                    ctrl[1] = 0x100u + target;
                    ctrl[2] = blockIdx.x;
                }
                break;
            }
        }
    }
    bar_sync(1, cons_threads);
}

// One pass: up to NTOK tokens that share one expert's weights.
struct Pass {
    int n_tok;
    int tok[MAX_NTOK], pair[MAX_NTOK];
};

struct Tables {
    const uint16_t *off, *plist, *act, *ppre;
    int n_active, routed_passes, shared_passes;
};

__device__ __forceinline__ void unit_range(int n_units, int &u0, int &u1) {
    u0 = (int)((long long)blockIdx.x * n_units / gridDim.x);
    u1 = (int)((long long)(blockIdx.x + 1) * n_units / gridDim.x);
}

// Resolve routed pass index -> active index (the expert it belongs to).
__device__ __forceinline__ int find_active(const uint16_t *ppre, int n_active, int q) {
    int lo = 0, hi = n_active - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (ppre[mid] <= q) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// The tokens pass `q` serves (shared expert: tokens q*NTOK ...; routed: a slice of one expert's list).
template <int NTOK>
__device__ __forceinline__ void make_pass(Pass &U, int sh_t0, int sh_nt, int top_k, const Tables &T, int shared, int q) {
    if (shared) {
        U.n_tok = min(NTOK, sh_nt - q * NTOK);
#pragma unroll
        for (int i = 0; i < NTOK; i++) {
            U.tok[i] = sh_t0 + min(q * NTOK + i, sh_nt - 1);
            U.pair[i] = U.tok[i] * (top_k + 1) + top_k;
        }
    } else {
        const int a = find_active(T.ppre, T.n_active, q);
        const int e = T.act[a];
        const int r = q - T.ppre[a];
        const int o = T.off[e], n = T.off[e + 1] - o;
        U.n_tok = min(NTOK, n - r * NTOK);
#pragma unroll
        for (int i = 0; i < NTOK; i++) {
            const int p = T.plist[o + min(r * NTOK + i, n - 1)];
            U.tok[i] = p / top_k;
            U.pair[i] = U.tok[i] * (top_k + 1) + (p - U.tok[i] * top_k);
        }
    }
}

// ---- activation cache staging --------------------------------------------------
// Each value of a token's row becomes NDIG signed base-128 digits of X = round(v * QMAX / amax), amax
// taken per 256-wide block (QMAX = 2^19 - 1 for three digits, 16191 for two: the top digit stays inside a
// signed byte).  Digit d (most significant first) of token tk is int8 column NDIG*tk + d of the cache, in
// natural k order, and sxs[block][column] is the float that turns the column's integer dot product back
// into the row's scale.  sh: SUB-wide sums of the quantized values, as f16 hi/lo pairs in columns NDIG*tk and
// NDIG*tk + 1 (zero in a third), for the Q4_K min term and the Q6_K offset; they are stored as the INTEGER sums
// times 2^-9 (three digits) or 2^-4 (two), so they fit f16 for any input magnitude.  One warp per (token,
// block): a lane owns 8 consecutive values.
// FROM_X: phase 1, rows of x (global, read-only); else phase 2, SwiGLU activations written by other CTAs.
template <int NDIG, int NTOK, int SUB, bool FROM_X, int NCW>
__device__ __forceinline__ void stage_rows(const DecodeParams &P, const Pass &U, int8_t *xc, __half *sh, float *sxs,
                                           int xs, int ss, int warp, int lane) {
    constexpr float QMAX = NDIG == 3 ? 524287.f : 16191.f;
    const int k = FROM_X ? P.hidden : P.ff;
    const int nblk = k / QK_K;
    for (int it = warp; it < U.n_tok * nblk; it += NCW) {
        const int tk = it / nblk, b = it - tk * nblk;
        const float *src = (FROM_X ? P.x + (size_t)U.tok[tk] * P.hidden : P.act_f + (size_t)U.pair[tk] * P.ff) +
                           b * QK_K + lane * 8;
        float4 a, c;
        if (FROM_X) {
            a = __ldg(reinterpret_cast<const float4 *>(src));
            c = __ldg(reinterpret_cast<const float4 *>(src) + 1);
        } else {
            a = __ldcg(reinterpret_cast<const float4 *>(src));
            c = __ldcg(reinterpret_cast<const float4 *>(src) + 1);
        }
        const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) amax = fmaxf(amax, fabsf(v[j]));
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float inv = amax > 0.f ? QMAX / amax : 0.f;
        const float sx = amax * (1.0f / QMAX);
        int sum = 0;
        uint32_t dig[NDIG][2];
#pragma unroll
        for (int d = 0; d < NDIG; d++) dig[d][0] = dig[d][1] = 0u;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            int X = __float2int_rn(v[j] * inv);
            sum += X;
            // least significant digit first; the last digit takes what is left
#pragma unroll
            for (int d = NDIG - 1; d > 0; d--) {
                const int dd = ((X + 64) & 127) - 64;
                dig[d][j >> 2] |= (uint32_t)(dd & 255) << (8 * (j & 3));
                X = (X - dd) >> 7;
            }
            dig[0][j >> 2] |= (uint32_t)(X & 255) << (8 * (j & 3));
        }
#pragma unroll
        for (int d = 0; d < NDIG; d++)
            *reinterpret_cast<uint2 *>(xc + (NDIG * tk + d) * xs + b * QK_K + lane * 8) = make_uint2(dig[d][0], dig[d][1]);
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if (SUB == 32) sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((lane & (SUB / 8 - 1)) == 0) {
            // the integer sum, scaled into the f16 range whatever the magnitude of the row (|sum| <= 32 * QMAX);
            // the block's scale comes back in through the column scales (see sum_ratio)
            const float sf = (float)sum * (NDIG == 3 ? 0x1p-9f : 0x1p-4f);
            const __half h = __float2half_rn(sf);
            const int idx = b * (QK_K / SUB) + lane / (SUB / 8);
            sh[(NDIG * tk) * ss + idx] = h;
            sh[(NDIG * tk + 1) * ss + idx] = __float2half_rn(sf - __half2float(h));
            if (NDIG == 3) sh[(NDIG * tk + 2) * ss + idx] = __float2half_rn(0.f);
        }
        if (lane < NDIG) {
            // column scale: digit d (most significant first) weighs 128^(NDIG-1-d)
            float f = sx;
            for (int d = lane; d < NDIG - 1; d++) f *= 128.f;
            sxs[b * 8 + NDIG * tk + lane] = f;
        }
    }
}

// The sub-block sums sit in MMA columns NDIG*tk (high part) and NDIG*tk + 1 (low part) as integers times
// 2^-SHIFT; column c's digit scale is sx * 128^(NDIG-1-d), d = c mod NDIG.  sum_ratio(c) = 2^SHIFT / 128^(NDIG-1-d)
// turns the column scale into the factor of that column's sum term.
template <int NDIG>
__device__ __forceinline__ float sum_ratio(int c) {
    const int d = c % NDIG;
    if (NDIG == 3) return d == 0 ? 0x1p-5f : (d == 1 ? 4.0f : 512.0f);
    return d == 0 ? 0x1p-3f : 16.0f;
}

// ---- per-unit math ---------------------------------------------------------------
// One Q4_K super-block of rows g (bg) and g+8 (bG): 8 gate + 8 up rows.
// xb / sb / sxb: the activation digits, the 32-wide activation sums and the column scales of this
// super-block for this lane's MMA column.  acc: rows g / g+8, columns 2t, 2t+1.
// The nibbles of a 32-weight sub-block are the bytes of one k = 32 integer MMA (no unpacking beyond a mask);
// the six-bit sub-block scales multiply the exact integer sums, and the float factors (d of the row, digit
// scale of the column) come in once per super-block.
__device__ __forceinline__ void q4k_block(const uint8_t *bg, const uint8_t *bG, int t, const int8_t *xb,
                                          const __half *sb, const float *sxb, float r0, float r1, float (&acc)[4]) {
    constexpr uint32_t M4 = 0x0F0F0F0Fu;
    const uint4 hg = *reinterpret_cast<const uint4 *>(bg);
    const uint4 hG = *reinterpret_cast<const uint4 *>(bG);
    const float dg = lmoe_h2f((uint16_t)(hg.x & 0xffff));
    const float mg = lmoe_h2f((uint16_t)(hg.x >> 16)) * 16777216.f;
    const float dG = lmoe_h2f((uint16_t)(hG.x & 0xffff));
    const float mG = lmoe_h2f((uint16_t)(hG.x >> 16)) * 16777216.f;
    uint32_t scg[2], mng[2], scG[2], mnG[2]; // (scale, min) pairs, one per byte, per half
    q4k_unpack_scales(hg.y, hg.z, hg.w, scg[0], scg[1], mng[0], mng[1]);
    q4k_unpack_scales(hG.y, hG.z, hG.w, scG[0], scG[1], mnG[0], mnG[1]);
    // min term: one f16 MMA, A = the six-bit mins of each row (as f16 subnormals), B = 32-wide activation sums
    float cm[4];
    {
        const uint32_t sel = (t & 1) ? 0x4342u : 0x4140u;
        const uint32_t ma = __byte_perm(t < 2 ? mng[0] : mng[1], 0u, sel);
        const uint32_t mA = __byte_perm(t < 2 ? mnG[0] : mnG[1], 0u, sel);
        const uint32_t sv = *reinterpret_cast<const uint32_t *>(sb + 2 * t);
        mma16816_z(cm, ma, mA, 0u, 0u, sv, 0u);
    }
    int al[4] = {0, 0, 0, 0};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint32_t sg = h ? scg[1] : scg[0], sG = h ? scG[1] : scG[0];
#pragma unroll
        for (int jj = 0; jj < 2; jj++) {
            const int j = 2 * h + jj;
            // bytes 8t..8t+7 of the 32-byte chunk: low nibbles = sub-block 2j, high nibbles = sub-block 2j+1
            const uint2 wg = *reinterpret_cast<const uint2 *>(bg + 16 + 32 * j + 8 * t);
            const uint2 wG = *reinterpret_cast<const uint2 *>(bG + 16 + 32 * j + 8 * t);
            const uint2 xl = *reinterpret_cast<const uint2 *>(xb + 64 * j + 8 * t);
            const uint2 xh = *reinterpret_cast<const uint2 *>(xb + 64 * j + 32 + 8 * t);
            int fl[4], fh[4];
            imma16832_z(fl, wg.x & M4, wG.x & M4, wg.y & M4, wG.y & M4, xl.x, xl.y);
            imma16832_z(fh, (wg.x >> 4) & M4, (wG.x >> 4) & M4, (wg.y >> 4) & M4, (wG.y >> 4) & M4, xh.x, xh.y);
            const int s0g = ubyte(sg, 2 * jj), s1g = ubyte(sg, 2 * jj + 1);
            const int s0G = ubyte(sG, 2 * jj), s1G = ubyte(sG, 2 * jj + 1);
            al[0] += s0g * fl[0] + s1g * fh[0];
            al[1] += s0g * fl[1] + s1g * fh[1];
            al[2] += s0G * fl[2] + s1G * fh[2];
            al[3] += s0G * fl[3] + s1G * fh[3];
        }
    }
    const float2 cs = *reinterpret_cast<const float2 *>(sxb + 2 * t);
    // r0 / r1: sum_ratio of columns 2t / 2t+1
    acc[0] += cs.x * (dg * (float)al[0] - mg * (r0 * cm[0]));
    acc[1] += cs.y * (dg * (float)al[1] - mg * (r1 * cm[1]));
    acc[2] += cs.x * (dG * (float)al[2] - mG * (r0 * cm[2]));
    acc[3] += cs.y * (dG * (float)al[3] - mG * (r1 * cm[3]));}

// 16 Q4_K rows (8 gate + 8 up): warp wq of the group takes every CW-th super-block.
__device__ __forceinline__ void unit_q4k(const uint8_t *stage, int row_bytes, int nb, int wq, int g, int t,
                                         const int8_t *xcol, const __half *scol, const float *sxs, float r0, float r1,
                                         float (&acc)[4]) {
    const uint8_t *rg = stage + g * row_bytes;
    const uint8_t *rG = rg + 8 * row_bytes;
    for (int b = wq; b < nb; b += CW)
        q4k_block(rg + b * Q4K_BYTES, rG + b * Q4K_BYTES, t, xcol + 256 * b, scol + 8 * b, sxs + 8 * b, r0, r1, acc);
}

// 32 Q6_K rows: warp wq of the group takes row tile wq & 1 (16 rows) and every (CW/2)-th super-block of it.
// Super-blocks are 210 bytes long, so every other one starts 2 bytes off a word boundary.
__device__ __forceinline__ void unit_q6k(const uint8_t *stage, int row_bytes, int nb, int wq, int g, int t,
                                         const int8_t *xcol, const __half *scol, const float *sxs, float r0, float r1,
                                         float (&acc)[4]) {
    // lane group g works on rows 2g and 2g+1 of the tile: with 840-byte rows the eight rows of one load sit in
    // disjoint shared-memory banks (rows g and g+8 would share two)
    const uint8_t *rg = stage + ((wq & 1) * 16 + 2 * g) * row_bytes;
    const uint8_t *rG = rg + row_bytes;
    for (int b = wq >> 1; b < nb; b += CW / 2) {
        const uint8_t *bg = rg + b * Q6K_BYTES, *bG = rG + b * Q6K_BYTES;
        if (row_bytes & 2) q6k_block<2>(bg, bG, b, t, xcol, scol, sxs, r0, r1, acc); // odd block count: rows alternate too
        else if (b & 1) q6k_block<1>(bg, bG, b, t, xcol, scol, sxs, r0, r1, acc);
        else q6k_block<0>(bg, bG, b, t, xcol, scol, sxs, r0, r1, acc);
    }
}

// Per-pass hand-over between phases 1 and 2 (small batches).  Out of line on purpose: they run once per
// pass and must not disturb the register allocation of the unit loops.
__device__ __noinline__ void dec_publish_pass(uint32_t *cnt, uint32_t add) {
    __threadfence();
    atomicAdd(cnt, add);
}
__device__ __noinline__ void dec_wait_pass(const uint32_t *cnt, uint32_t need, uint32_t *ctrl, uint32_t where) {
    uint32_t i = 0;
    while (ld_acquire(cnt) < need) {
        if ((i & 1023u) == 1023u && *reinterpret_cast<volatile uint32_t *>(ctrl) != 0u) break;
        if (++i > SPIN_LIMIT) {
            if (atomicCAS(ctrl, 0u, (uint32_t)LMOE_FLAG_WAIT_TIMEOUT) == 0u) {
                ctrl[1] = where;
                ctrl[2] = blockIdx.x;
            }
            break;
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------
template <int NDIG, int NTOK, int NG>
__global__ void __launch_bounds__(Cfg<NG>::THREADS, Cfg<NG>::MIN_CTAS) moe_decode_kernel(const __grid_constant__ DecodeParams P) {
    using C = Cfg<NG>;
    constexpr int NCOL = NDIG * NTOK; // MMA columns in use: (token, digit)
    constexpr int NSTAGE = C::NSTAGE, NRED = C::NRED, NCW = C::NCW, CONS_THREADS = C::CONS;
    extern __shared__ __align__(128) uint8_t smem[];
    const DecLayout L(P.hidden, P.ff, P.n_expert, P.t, P.top_k, NCOL, NCW, NSTAGE, NRED);
    uint8_t *ring = smem + L.o_ring;
    int8_t *xc = reinterpret_cast<int8_t *>(smem + L.o_xc);
    __half *sh = reinterpret_cast<__half *>(smem + L.o_s);
    float *sxs = reinterpret_cast<float *>(smem + L.o_sx);
    float *red = reinterpret_cast<float *>(smem + L.o_red);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + L.o_bar);
    uint64_t *empty = full + NSTAGE;
    uint64_t *red_full = empty + NSTAGE, *red_free = red_full + NRED; // K-split partial buffers: consumers -> epilogue warp
    uint32_t *ids_s = reinterpret_cast<uint32_t *>(smem + L.o_ids);
    float *w_s = reinterpret_cast<float *>(smem + L.o_w);
    uint32_t *cnt_s = reinterpret_cast<uint32_t *>(smem + L.o_cnt);
    uint16_t *off_s = reinterpret_cast<uint16_t *>(smem + L.o_off);
    uint16_t *plist_s = reinterpret_cast<uint16_t *>(smem + L.o_plist);
    uint16_t *act_s = reinterpret_cast<uint16_t *>(smem + L.o_act);
    uint16_t *ppre_s = reinterpret_cast<uint16_t *>(smem + L.o_ppre);
    __shared__ int s_n_active, s_routed_passes;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x;
    const int K = P.top_k, E = P.n_expert;
    const int nb4 = P.hidden / QK_K, nb6 = P.ff / QK_K;
    const int row4 = nb4 * Q4K_BYTES, row6 = nb6 * Q6K_BYTES;
    const int tiles1 = P.ff / 8, tiles2 = P.hidden / DOWN_ROWS;
    const int shared_passes = P.has_shared ? (P.sh_nt + NTOK - 1) / NTOK : 0;
    const size_t gexp = (size_t)P.ff * row4, dexp = (size_t)P.hidden * row6;
    // Between phases 1 and 2: per-pass completion counters up to 16 tokens (no grid barrier, early passes start
    // early: a few per cent at 4 and 8 tokens), a grid barrier for larger batches.
    const bool pass_flags = P.t <= LMOE_DEC_PASS_FLAG_MAX_T;

    if (tid == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        for (int b = 0; b < NRED; b++) {
            mbar_init(&red_full[b], CW);
            mbar_init(&red_free[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == NCW) {
        // ===================== producer warp (lane 0 issues) =====================
        uint32_t n = 0; // fills issued (the same sequence the consumers count)
        auto fill = [&](const uint8_t *src0, const uint8_t *src1, uint32_t bytes_each) {
            const int s = n % NSTAGE;
            const uint32_t r = n / NSTAGE;
            mbar_wait<200>(&empty[s], (r & 1) ^ 1, P.ctrl, 0x10);
            uint8_t *dst = ring + (size_t)s * L.stage_bytes;
            mbar_expect_tx(&full[s], src1 ? 2 * bytes_each : bytes_each);
            bulk_g2s(dst, src0, bytes_each, &full[s]);
            if (src1) bulk_g2s(dst + bytes_each, src1, bytes_each, &full[s]);
            n++;
        };
        int u0, u1, u = 0;
        // phase 1, shared expert: known before routing.  Only as many fills as the ring
        // holds may be issued before the routing tables exist (consumers drain the ring
        // only after they have built them).
        unit_range(shared_passes * tiles1, u0, u1);
        bar_sync(3, C::RING); // the consumers stage hidden states in the ring while they compute the logits
        if (lane == 0) {
            for (u = u0; u < u1 && u < u0 + NSTAGE; u++) {
                const int tile = u % tiles1;
                fill(P.sh_gate + (size_t)tile * 8 * row4, P.sh_up + (size_t)tile * 8 * row4, 8 * row4);
            }
        }
        __syncwarp();
        bar_sync(2, C::THREADS); // routing tables are ready
        if (lane == 0) {
            for (; u < u1; u++) {
                const int tile = u % tiles1;
                fill(P.sh_gate + (size_t)tile * 8 * row4, P.sh_up + (size_t)tile * 8 * row4, 8 * row4);
            }
            const int n_active = s_n_active, routed_passes = s_routed_passes;
            unit_range(routed_passes * tiles1, u0, u1);
            if (u0 < u1) {
                int q = u0 / tiles1, tile = u0 - q * tiles1;
                int e = act_s[find_active(ppre_s, n_active, q)];
                for (u = u0; u < u1; u++) {
                    if (!DEC_GUARD((unsigned)e < (unsigned)E && (unsigned)tile < (unsigned)tiles1, 0x502, (e << 16) | tile)) e = 0, tile = 0;
                    fill(P.gate + e * gexp + (size_t)tile * 8 * row4, P.up + e * gexp + (size_t)tile * 8 * row4, 8 * row4);
                    if (++tile == tiles1 && u + 1 < u1) {
                        tile = 0;
                        e = act_s[find_active(ppre_s, n_active, ++q)];
                    }
                }
            }
            // phase 2 (weights do not depend on the grid barrier: keep streaming)
            unit_range(shared_passes * tiles2, u0, u1);
            for (u = u0; u < u1; u++) fill(P.sh_down + (size_t)(u % tiles2) * DOWN_ROWS * row6, nullptr, DOWN_ROWS * row6);
            unit_range(routed_passes * tiles2, u0, u1);
            if (u0 < u1) {
                int q = u0 / tiles2, tile = u0 - q * tiles2;
                int e = act_s[find_active(ppre_s, n_active, q)];
                for (u = u0; u < u1; u++) {
                    if (!DEC_GUARD((unsigned)e < (unsigned)E && (unsigned)tile < (unsigned)tiles2, 0x503, (e << 16) | tile)) e = 0, tile = 0;
                    fill(P.down + e * dexp + (size_t)tile * DOWN_ROWS * row6, nullptr, DOWN_ROWS * row6);
                    if (++tile == tiles2 && u + 1 < u1) {
                        tile = 0;
                        e = act_s[find_active(ppre_s, n_active, ++q)];
                    }
                }
            }
            // before leaving, wait (bounded) until this warp's last copies have been consumed: no bulk copy
            // of this CTA is in flight once its issuer is gone
            for (uint32_t k = n > (uint32_t)NSTAGE ? n - NSTAGE : 0; k < n; k++)
                mbar_wait<200>(&empty[k % NSTAGE], (k / NSTAGE) & 1, P.ctrl, 0x12);
        }
        return;
    }

    if (warp == NCW + 1) {
        // ===================== epilogue warp =====================
        // Sums the K-split partials of each unit in a fixed order and writes the SwiGLU activation
        // (phase 1) or the weighted partial output row (phase 2), off the consumers' critical path.
        bar_sync(2, C::THREADS);
        const Tables T{off_s, plist_s, act_s, ppre_s, s_n_active, s_routed_passes, shared_passes};
        uint32_t m = 0; // units handed over so far (the same sequence the consumers count)
        for (int phase = 1; phase <= 2; phase++) {
            const int tiles = phase == 1 ? tiles1 : tiles2;
            for (int kind = 0; kind < 2; kind++) {
                const int shared = kind == 0;
                int u0, u1;
                unit_range((shared ? shared_passes : T.routed_passes) * tiles, u0, u1);
                if (u0 >= u1) continue;
                int q = u0 / tiles, tile = u0 - q * tiles;
                Pass U;
                make_pass<NTOK>(U, P.sh_t0, P.sh_nt, K, T, shared, q);
                // Phase 2 of a pass may start, on any CTA, once all its phase-1 units are done: this CTA adds
                // the number it finished to the pass's counter whenever it leaves a pass.
                int done_in_pass = 0;
                auto publish = [&](int qq) {
                    if (pass_flags && phase == 1 && done_in_pass > 0) {
                        __syncwarp();
                        if (lane == 0) dec_publish_pass(P.sync + SYNC_PASS0 + (shared ? qq : shared_passes + qq), (uint32_t)done_in_pass);
                        __syncwarp();
                    }
                    done_in_pass = 0;
                };
                for (int u = u0; u < u1; u++, m++) {
                    const int buf = m % NRED;
                    mbar_wait<100>(&red_full[buf], (m / NRED) & 1, P.ctrl, 0x30 + phase);
                    const float *rb = red + buf * (CW * 16 * NCOL);
                    if (phase == 1) {
                        // SwiGLU: rows 0-7 gate, 8-15 up; lane = tok*8 + row
                        const int tk = lane >> 3, r = lane & 7;
                        if (tk < U.n_tok) {
                            float gv = 0.f, uv = 0.f;
#pragma unroll
                            for (int w = 0; w < CW; w++) {
#pragma unroll
                                for (int d = 0; d < NDIG; d++) {
                                    gv += rb[(w * 16 + r) * NCOL + NDIG * tk + d];
                                    uv += rb[(w * 16 + 8 + r) * NCOL + NDIG * tk + d];
                                }
                            }
                            const float sv = __fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv)));
                            const float av = __fmul_rn(sv, uv);
                            __stcg(P.act_f + (size_t)U.pair[tk] * P.ff + tile * 8 + r, av);
                        }
                    } else {
                        // weighted partial rows of this (pair, tile); summed over slots in phase 3.
                        // lane = row of the unit; warps w with w & 1 == row tile hold its K-split partials
                        const int rt = lane >> 4, r = lane & 15;
                        for (int tk = 0; tk < U.n_tok; tk++) {
                            float yv = 0.f;
#pragma unroll
                            for (int w = 0; w < CW / 2; w++) {
#pragma unroll
                                for (int d = 0; d < NDIG; d++) yv += rb[((2 * w + rt) * 16 + r) * NCOL + NDIG * tk + d];
                            }
                            const int slot = U.pair[tk] - U.tok[tk] * (K + 1);
                            if (slot < K) yv = __fmul_rn(yv, w_s[U.tok[tk] * K + slot]);
                            __stcg(P.ypart + (size_t)U.pair[tk] * P.hidden + tile * DOWN_ROWS + lane, yv);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&red_free[buf]);
                    done_in_pass++;
                    if (++tile == tiles && u + 1 < u1) {
                        tile = 0;
                        publish(q);
                        make_pass<NTOK>(U, P.sh_t0, P.sh_nt, K, T, shared, ++q);
                    }
                }
                publish(q);
            }
            // the phase's results are complete: join the consumers' grid barrier (none after phase 1 when the
            // per-pass counters are in use)
            if (phase == 2 || !pass_flags) {
                __threadfence();
                bar_arrive(4, C::EPI);
            }
        }
        return;
    }

    // ========================= consumer warps =========================
    const int g = lane >> 2, t4 = lane & 3;
    const int grp = warp / CW, wq = warp % CW;
    uint32_t gb = 0; // grid barriers passed

    if (P.first_launch && blockIdx.x == 0 && tid < 4) P.ctrl[tid] = 0u; // a fresh device flag for this call
    if (P.ext_ids == nullptr) {
        // ---- phase 0a: router logits (bit-specified reduction, see route_math.cuh) ----
        if (P.hidden == 128 * 24) {
            // Work item = (expert, group of four tokens).  A CTA serves ONE token group (CTA c: group c mod
            // #groups), so it stages only those four hidden states (as f32, in the not yet used weight ring);
            // the CTAs of a group share out the experts, one per warp.  The router row is held in registers
            // half a row at a time (all loads of a half in flight at once).  Each of the 128 partial chains
            // still runs over its 24 elements in order.
            constexpr int HH = 12;
            const int H = P.hidden;
            float *xs32 = reinterpret_cast<float *>(ring);
            const int ngr = (P.t + 3) / 4;
            const int cg = blockIdx.x % ngr, ci = blockIdx.x / ngr;
            const int n_cta = (G - cg + ngr - 1) / ngr; // CTAs serving this group
            const int t0 = 4 * cg, nt = min(4, P.t - t0);
            float4 wv[HH];
            bool preloaded = false;
            {
                // the first item's first half row is requested before the hidden states are staged
                const int e = ci + n_cta * warp;
                if (e < E) {
                    const float4 *wr = reinterpret_cast<const float4 *>(P.router + (size_t)e * H) + lane;
#pragma unroll
                    for (int j = 0; j < HH; j++) wv[j] = __ldg(wr + 32 * j);
                    preloaded = true;
                }
            }
            for (int i = tid; i < nt * (H / 4); i += CONS_THREADS)
                reinterpret_cast<float4 *>(xs32)[i] = __ldg(reinterpret_cast<const float4 *>(P.x + (size_t)t0 * H) + i);
            bar_sync(1, CONS_THREADS);
            for (int e = ci + n_cta * warp; e < E; e += n_cta * NCW) {
                const float4 *wr = reinterpret_cast<const float4 *>(P.router + (size_t)e * H) + lane;
                float a[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++) a[i][0] = a[i][1] = a[i][2] = a[i][3] = 0.f;
#pragma unroll 1
                for (int half = 0; half < 2; half++) {
                    if (!(preloaded && half == 0)) {
#pragma unroll
                        for (int j = 0; j < HH; j++) wv[j] = __ldg(wr + 32 * (HH * half + j));
                    }
                    preloaded = false;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if (i < nt) {
                            const float4 *xr = reinterpret_cast<const float4 *>(xs32 + i * H) + lane + 32 * HH * half;
#pragma unroll
                            for (int j = 0; j < HH; j++) {
                                const float4 xv = xr[32 * j];
                                a[i][0] = __fmaf_rn(xv.x, wv[j].x, a[i][0]);
                                a[i][1] = __fmaf_rn(xv.y, wv[j].y, a[i][1]);
                                a[i][2] = __fmaf_rn(xv.z, wv[j].z, a[i][2]);
                                a[i][3] = __fmaf_rn(xv.w, wv[j].w, a[i][3]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float v = lmoe_router_fold(a[i][0], a[i][1], a[i][2], a[i][3]);
                    if (lane == 0 && i < nt) P.logits[(size_t)(t0 + i) * E + e] = v;
                }
            }
        } else {
            const int ntt = (P.t + 3) / 4;
            const int H = P.hidden;
            for (int q = blockIdx.x * NCW + warp; q < E * ntt; q += G * NCW) {
                const int e = q / ntt, t0 = (q - e * ntt) * 4;
                const float *wr = P.router + (size_t)e * H;
                float a[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++) a[i][0] = a[i][1] = a[i][2] = a[i][3] = 0.f;
#pragma unroll 4
                for (int base = 4 * lane; base < H; base += 128) {
                    const float4 wv = __ldg(reinterpret_cast<const float4 *>(wr + base));
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if (t0 + i < P.t) {
                            const float4 xv = __ldg(reinterpret_cast<const float4 *>(P.x + (size_t)(t0 + i) * H + base));
                            a[i][0] = __fmaf_rn(xv.x, wv.x, a[i][0]);
                            a[i][1] = __fmaf_rn(xv.y, wv.y, a[i][1]);
                            a[i][2] = __fmaf_rn(xv.z, wv.z, a[i][2]);
                            a[i][3] = __fmaf_rn(xv.w, wv.w, a[i][3]);
                        }
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float v = lmoe_router_fold(a[i][0], a[i][1], a[i][2], a[i][3]);
                    if (lane == 0 && t0 + i < P.t) P.logits[(size_t)(t0 + i) * E + e] = v;
                }
            }
        }
        // selection bias -> shared memory (the expert-count table is not in use yet)
        float *bias_s = reinterpret_cast<float *>(cnt_s);
        for (int e = tid; e < E; e += CONS_THREADS) bias_s[e] = P.bias ? __ldg(P.bias + e) : 0.0f;
        bar_sync(3, C::RING); // the weight ring is free from here on: the producer may start
        grid_barrier(P.ctrl, P.sync, (++gb) * (uint32_t)G, tid, CONS_THREADS, 1, CONS_THREADS);

        // ---- phase 0b: selection.  Token i is handled by CTA i: each of the consumer warps ranks an equal share
        //      of the experts (register-light, rolled loops: this code runs once), warp 0 merges the candidates;
        //      ties always go to the lower expert index, so the result equals a stable descending sort.
        //      Results travel through global memory and one more grid barrier. ----
        if ((int)blockIdx.x < P.t) {
            const int tok = blockIdx.x;
            float *probs = reinterpret_cast<float *>(xc);
            uint32_t *keys = reinterpret_cast<uint32_t *>(probs + E);
            uint32_t *cand_key = keys + E, *cand_idx = cand_key + NCW * 32;
            const int eq = (E + NCW - 1) / NCW, lo = warp * eq, hi = min(E, lo + eq);
            uint32_t best = 0u;
            int best_i = 0x7fffffff;
            for (int e0 = lo; e0 < hi; e0 += 128) {
                float lg[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int e = e0 + lane + 32 * i;
                    lg[i] = e < hi ? __ldcg(P.logits + (size_t)tok * E + e) : 0.0f;
                }
#pragma unroll 1
                for (int i = 0; i < 4; i++) {
                    const int e = e0 + lane + 32 * i;
                    if (e < hi) {
                        const float p = lmoe_sigmoid_fixed(lg[i]);
                        const float sv = __fadd_rn(__fadd_rn(p, bias_s[e]), 0.0f);
                        const uint32_t u = __float_as_uint(sv);
                        uint32_t kk = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                        kk = kk == 0u ? 1u : kk;
                        probs[e] = p;
                        keys[e] = kk;
                        if (kk > best) { best = kk; best_i = e; }
                    }
                }
            }
            __syncwarp();
#pragma unroll 1
            for (int k = 0; k < K; k++) {
                const uint32_t m = __reduce_max_sync(0xffffffffu, best);
                const uint32_t idx = __reduce_min_sync(0xffffffffu, best == m ? (uint32_t)best_i : 0xffffffffu);
                if (lane == 0) { cand_key[warp * 32 + k] = m; cand_idx[warp * 32 + k] = idx; }
                if (m != 0u && (int)idx == best_i && best == m) {
                    keys[idx] = 0u;
                    best = 0u;
                    best_i = 0x7fffffff;
#pragma unroll 1
                    for (int e = lo + lane; e < hi; e += 32) {
                        const uint32_t kk = keys[e];
                        if (kk > best) { best = kk; best_i = e; }
                    }
                }
            }
            bar_sync(1, CONS_THREADS);
            if (warp == 0) {
                // lane l owns candidate l of every warp (K <= 32)
                uint32_t ck[NCW], ci[NCW];
#pragma unroll
                for (int w = 0; w < NCW; w++) {
                    ck[w] = lane < K ? cand_key[w * 32 + lane] : 0u;
                    ci[w] = lane < K ? cand_idx[w * 32 + lane] : 0xffffffffu;
                }
                float my_w = 0.0f;
#pragma unroll 1
                for (int k = 0; k < K; k++) {
                    uint32_t bk = 0u;
#pragma unroll
                    for (int w = 0; w < NCW; w++) bk = ck[w] > bk ? ck[w] : bk;
                    const uint32_t m = __reduce_max_sync(0xffffffffu, bk);
                    uint32_t bi = 0xffffffffu;
#pragma unroll
                    for (int w = 0; w < NCW; w++) bi = (ck[w] == m && ci[w] < bi) ? ci[w] : bi;
                    const uint32_t idx = __reduce_min_sync(0xffffffffu, bi);
#pragma unroll
                    for (int w = 0; w < NCW; w++) if (ci[w] == idx) ck[w] = 0u;
                    const float pw = probs[idx < (uint32_t)E ? idx : 0u];
                    if (lane == k) my_w = pw;
                    if (lane == 0) P.ids_ws[tok * K + k] = idx;
                }
                if (P.norm) {
                    float sum = 0.0f;
#pragma unroll 1
                    for (int k = 0; k < K; k++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_w, k));
                    sum = sum < 6.103515625e-5f ? 6.103515625e-5f : sum;
                    my_w = __fdiv_rn(my_w, sum);
                }
                if (P.scale != 0.0f && P.scale != 1.0f) my_w = __fmul_rn(my_w, P.scale);
                if (lane < K) P.w_ws[tok * K + lane] = my_w;
            }
        }
        grid_barrier(P.ctrl, P.sync, (++gb) * (uint32_t)G, tid, CONS_THREADS, 1, CONS_THREADS);
        for (int i = tid; i < P.t * K; i += CONS_THREADS) {
            const uint32_t id = __ldcg(P.ids_ws + i);
            const float wv = __ldcg(P.w_ws + i);
            ids_s[i] = id;
            w_s[i] = wv;
            if (blockIdx.x == 0) {
                if (P.ids_out) P.ids_out[i] = id;
                if (P.w_out) P.w_out[i] = wv;
            }
        }
    } else {
        // ---- the caller routed: take its decision as it is (an id >= n_expert marks an empty slot) ----
        bar_sync(3, C::RING);
        for (int i = tid; i < P.t * K; i += CONS_THREADS) {
            ids_s[i] = __ldg(P.ext_ids + i);
            w_s[i] = __ldg(P.ext_w + i);
        }
    }
    for (int e = tid; e < E; e += CONS_THREADS) cnt_s[e] = 0;
    bar_sync(1, CONS_THREADS);
    // ---- phase 0c: per-expert token lists ----
    for (int i = tid; i < P.t * K; i += CONS_THREADS)
        if (ids_s[i] < (uint32_t)E) atomicAdd(&cnt_s[ids_s[i]], 1u);
    bar_sync(1, CONS_THREADS);
    if (warp == 0) {
        // exclusive scans over experts: list offsets, active index, pass prefix
        const int per = (E + 31) / 32;
        const int e0 = lane * per, e1 = min(E, e0 + per);
        int c_sum = 0, a_sum = 0, p_sum = 0;
        for (int e = e0; e < e1; e++) {
            const int c = (int)cnt_s[e];
            c_sum += c;
            a_sum += c > 0;
            p_sum += (c + NTOK - 1) / NTOK;
        }
        int c_pre = c_sum, a_pre = a_sum, p_pre = p_sum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int c2 = __shfl_up_sync(0xffffffffu, c_pre, o), a2 = __shfl_up_sync(0xffffffffu, a_pre, o);
            const int p2 = __shfl_up_sync(0xffffffffu, p_pre, o);
            if (lane >= o) { c_pre += c2; a_pre += a2; p_pre += p2; }
        }
        const int c_tot = __shfl_sync(0xffffffffu, c_pre, 31), a_tot = __shfl_sync(0xffffffffu, a_pre, 31);
        const int p_tot = __shfl_sync(0xffffffffu, p_pre, 31);
        c_pre -= c_sum; a_pre -= a_sum; p_pre -= p_sum;
        for (int e = e0; e < e1; e++) {
            const int c = (int)cnt_s[e];
            off_s[e] = (uint16_t)c_pre;
            if (c > 0) {
                act_s[a_pre] = (uint16_t)e;
                ppre_s[a_pre] = (uint16_t)p_pre;
                a_pre++;
                p_pre += (c + NTOK - 1) / NTOK;
            }
            c_pre += c;
        }
        if (lane == 31) {
            off_s[E] = (uint16_t)c_tot;
            ppre_s[a_tot] = (uint16_t)p_tot;
            s_n_active = a_tot;
            s_routed_passes = p_tot;
        }
    }
    bar_sync(1, CONS_THREADS);
    for (int e = tid; e < E; e += CONS_THREADS) cnt_s[e] = 0;
    bar_sync(1, CONS_THREADS);
    for (int i = tid; i < P.t * K; i += CONS_THREADS) {
        const uint32_t e = ids_s[i];
        if (e < (uint32_t)E) {
            const uint32_t pos = atomicAdd(&cnt_s[e], 1u);
            if (DEC_GUARD(off_s[e] + pos < (uint32_t)(P.t * K), 0x506, off_s[e] + pos)) plist_s[off_s[e] + pos] = (uint16_t)i;
        }
    }
    bar_sync(1, CONS_THREADS);
    // every CTA must see the same list order (passes are cut from it): sort each short list
    for (int e = tid; e < E; e += CONS_THREADS) {
        const int o = off_s[e], c = off_s[e + 1] - o;
        for (int i = 1; i < c; i++) {
            const uint16_t v = plist_s[o + i];
            int j = i - 1;
            while (j >= 0 && plist_s[o + j] > v) { plist_s[o + j + 1] = plist_s[o + j]; j--; }
            plist_s[o + j + 1] = v;
        }
    }
    bar_sync(1, CONS_THREADS);
    bar_sync(2, C::THREADS); // release the producer and the epilogue warp: the routing tables are complete

    const Tables T{off_s, plist_s, act_s, ppre_s, s_n_active, s_routed_passes, shared_passes};

    uint32_t n_unit = 0; // units (= ring fills) before the current section, the same sequence as the producer's
    uint32_t probed = 0xffffffffu; // unit whose barriers have been tested ahead (see the unit loop), and the answers
    bool probe_data = false, probe_buf = false;
    unsigned long long xkey = ~0ull;

    // ---- phases 1 and 2 ----
    for (int phase = 1; phase <= 2; phase++) {
        const int tiles = phase == 1 ? tiles1 : tiles2;
        // column pitch of the activation cache: 32 (mod 128) bytes for the 8-byte loads of phase 1, 16 for the
        // 4-byte loads of phase 2, so that the columns of one load instruction cover distinct banks
        const int xs_ph = phase == 1 ? L.xs : L.xs - 16;
        // MMA columns beyond the staged ones alias them: their results are never read
        const int col = g < NCOL ? g : g - 2;
        const int8_t *xcol = xc + col * xs_ph;
        const __half *scol = sh + col * L.ss;
        // factors of the sub-block sum terms of this lane's two accumulator columns (x 32 for the Q6_K offset)
        const float r0 = sum_ratio<NDIG>(2 * t4) * (phase == 1 ? 1.0f : 32.0f);
        const float r1 = sum_ratio<NDIG>(2 * t4 + 1) * (phase == 1 ? 1.0f : 32.0f);
        for (int kind = 0; kind < 2; kind++) { // shared units first, then routed
            const int shared = kind == 0;
            int u0, u1;
            unit_range((shared ? shared_passes : T.routed_passes) * tiles, u0, u1);
            if (u0 >= u1) continue;
            // the section is walked pass by pass: all consumer warps stage a pass's activations together,
            // then the two groups take alternate units of the pass's slice
            for (int q = u0 / tiles; q * tiles < u1; q++) {
                const int a = max(u0, q * tiles), b = min(u1, (q + 1) * tiles);
                Pass U;
                make_pass<NTOK>(U, P.sh_t0, P.sh_nt, K, T, shared, q);
                // what the cache holds is identified by the rows staged into it
                unsigned long long key = ((unsigned long long)phase << 60) | ((unsigned long long)U.n_tok << 56);
#pragma unroll
                for (int i = 0; i < NTOK; i++) key |= (unsigned long long)(phase == 1 ? U.tok[i] : U.pair[i]) << (12 * i);
                if (key != xkey) {
                    // phase 2 of a pass needs every SwiGLU activation of the pass: wait (bounded) until the pass's
                    // counter shows all its phase-1 units done, on whichever CTAs they ran
                    if (phase == 2 && pass_flags && tid == 0)
                        dec_wait_pass(P.sync + SYNC_PASS0 + (shared ? q : shared_passes + q), (uint32_t)tiles1, P.ctrl, 0x200u + q);
                    bar_sync(1, CONS_THREADS); // everyone is done with the previous contents
                    if (phase == 1) stage_rows<NDIG, NTOK, 32, true, NCW>(P, U, xc, sh, sxs, xs_ph, L.ss, warp, lane);
                    else stage_rows<NDIG, NTOK, 16, false, NCW>(P, U, xc, sh, sxs, xs_ph, L.ss, warp, lane);
                    xkey = key;
                    bar_sync(1, CONS_THREADS);
                }
                for (int u = a; u < b; u++) {
                    const uint32_t n = n_unit + (uint32_t)(u - u0);
                    if ((int)(n % NG) != grp) continue;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    const int s = n % NSTAGE; // one ring fill per unit
                    // the answers about this unit's two barriers were asked for before the previous unit's arithmetic
                    const bool have_data = probed == n && probe_data, have_buf = probed == n && probe_buf;
                    if (!have_data) mbar_wait(&full[s], (n / NSTAGE) & 1, P.ctrl, 0x20 + phase);
                    probed = n + 1;
                    probe_data = mbar_test(&full[probed % NSTAGE], (probed / NSTAGE) & 1);
                    probe_buf = mbar_test(&red_free[probed % NRED], ((probed / NRED) & 1) ^ 1);
                    const uint8_t *stage = ring + (size_t)s * L.stage_bytes;
                    if (phase == 1) unit_q4k(stage, row4, nb4, wq, g, t4, xcol, scol, sxs, r0, r1, acc);
                    else unit_q6k(stage, row6, nb6, wq, g, t4, xcol, scol, sxs, r0, r1, acc);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[s]);
                    // K-split partials -> shared memory, handed to the epilogue warp
                    const int buf = n % NRED;
                    if (!have_buf) mbar_wait(&red_free[buf], ((n / NRED) & 1) ^ 1, P.ctrl, 0x28 + phase);
                    float *rb = red + buf * (CW * 16 * NCOL);
                    if (2 * t4 < NCOL) {
                        // accumulator rows: g and g+8 of the 16 (phase 1), 2g and 2g+1 (phase 2, see unit_q6k)
                        float *r0 = rb + (wq * 16 + (phase == 1 ? g : 2 * g)) * NCOL + 2 * t4;
                        const int second = phase == 1 ? 8 * NCOL : NCOL;
                        r0[0] = acc[0]; r0[1] = acc[1];
                        r0[second] = acc[2]; r0[second + 1] = acc[3];
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&red_full[buf]);
                }
            }
            n_unit += (uint32_t)(u1 - u0);
        }
        if (phase == 2 || !pass_flags)
            grid_barrier(P.ctrl, P.sync, (++gb) * (uint32_t)G, tid, CONS_THREADS, 4, C::EPI);
    }

    // ---- phase 3: out[t, :] = sum over slots (then the shared expert) of the weighted partial rows,
    //      in slot order (`combine`, src/ops/combine.metal:70-97, plus `routed + shared`, src/moe.rs:77) ----
    {
        const int h4 = P.hidden / 4;
        for (int i = blockIdx.x * CONS_THREADS + tid; i < P.t * h4; i += G * CONS_THREADS) {
            const int tok = i / h4, c = i - tok * h4;
            const int nslot = K + (P.has_shared && tok >= P.sh_t0 && tok < P.sh_t0 + P.sh_nt ? 1 : 0);
            const float4 *yp = reinterpret_cast<const float4 *>(P.ypart + (size_t)tok * (K + 1) * P.hidden) + c;
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            // twelve slots' loads are in flight at once (the rows come from L2: one round trip, not one per slot)
            for (int s0 = 0; s0 < nslot; s0 += 12) {
                float4 v[12];
                uint32_t present = 0u;
#pragma unroll
                for (int j = 0; j < 12; j++) {
                    const int sl = s0 + j;
                    // a slot the caller left empty has no partial row
                    const bool ok = sl < nslot && !(P.ext_ids != nullptr && sl < K && __ldg(P.ext_ids + tok * K + sl) >= (uint32_t)E);
                    v[j] = ok ? __ldcg(yp + (size_t)sl * h4) : make_float4(0.f, 0.f, 0.f, 0.f);
                    present |= (uint32_t)ok << j;
                }
#pragma unroll
                for (int j = 0; j < 12; j++) {
                    if (present & (1u << j)) {
                        sum.x = __fadd_rn(sum.x, v[j].x);
                        sum.y = __fadd_rn(sum.y, v[j].y);
                        sum.z = __fadd_rn(sum.z, v[j].z);
                        sum.w = __fadd_rn(sum.w, v[j].w);
                    }
                }
            }
            reinterpret_cast<float4 *>(P.out + (size_t)tok * P.hidden)[c] = sum;
        }
    }

    // ---- exit: the last CTA leaves the control words zeroed for the next call ----
    bar_sync(1, CONS_THREADS);
    if (tid == 0) {
        __threadfence();
        const uint32_t old = atomicAdd(&P.sync[1], 1u);
        if (old == (uint32_t)(G - 1)) {
            P.sync[0] = 0u;
            P.sync[1] = 0u;
            const int n_pass = shared_passes + T.routed_passes;
            if (pass_flags)
                for (int i = 0; i < n_pass && i < SYNC_WORDS - SYNC_PASS0; i++) P.sync[SYNC_PASS0 + i] = 0u;
            __threadfence();
        }
    }
}

} // namespace

// ---- host side ------------------------------------------------------------------------
size_t decode_workspace_bytes(int t, int hidden, int ff, int n_expert, int top_k) {
    size_t o = 65536; // control words
    o += lmoe_align_up((size_t)t * n_expert * 4, 256);
    o += 2 * lmoe_align_up((size_t)t * top_k * 4, 256);
    o += lmoe_align_up((size_t)t * (top_k + 1) * ff * 4, 256);
    o += lmoe_align_up((size_t)t * (top_k + 1) * hidden * 4, 256);
    return o;
}

int decode_max_tokens() { return DEC_MAX_T; }
size_t decode_sync_bytes() { return (size_t)SYNC_WORDS * 4; }

namespace {
// One instantiation of the kernel with its launch geometry; launch facts are looked up once per
// (device, shared-memory size).
struct DecVariant {
    const void *fn;
    int ncol, ng, threads, ncw, nstage, nred, min_ctas;
    int c_dev = -1, c_total = -1, c_occ = 0;
};
template <int NDIG, int NTOK, int NG>
DecVariant make_variant() {
    using C = Cfg<NG>;
    return DecVariant{(const void *)moe_decode_kernel<NDIG, NTOK, NG>, NDIG * NTOK, NG, C::THREADS, C::NCW, C::NSTAGE, C::NRED, C::MIN_CTAS};
}
} // namespace

// ext_ids / ext_w: NULL = route inside the kernel; otherwise the caller's decision [t, top_k].  The shared expert is
// added for the tokens [shared_first, shared_first + shared_count) of this launch (count 0: for none).
lmoe_status launch_moe_decode(const lmoe_layer *Ly, const float *x, int t, float *out, uint32_t *ids_out,
                              float *w_out, const uint32_t *ext_ids, const float *ext_w, int shared_first, int shared_count,
                              void *workspace, size_t workspace_bytes, int first_launch, cudaStream_t stream) {
    const int H = (int)Ly->hidden, F = (int)Ly->expert_ff, E = (int)Ly->n_expert, K = (int)Ly->top_k;
    if (Ly->gate->dtype != LMOE_Q4_K || Ly->down->dtype != LMOE_Q6_K)
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "the fused decode kernel is built for Q4_K gate/up and Q6_K down stacks");
    if (t < 1 || t > DEC_MAX_T) return lmoe_fail(LMOE_ERR_INVALID, "decode launch takes 1..%d tokens, got %d", DEC_MAX_T, t);
    if (H % 128 || F % 16 || H % DOWN_ROWS)
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "fused decode needs hidden %% 128 == 0 and expert_ff %% 16 == 0");
    if (t * K > 4095 || t * (K + 1) > 4095 || (t + 1) / 2 + t * K > SYNC_WORDS - SYNC_PASS0)
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "t*top_k too large");
    // One group per CTA, two CTAs per SM.  Up to 8 tokens: three digits per activation (21 bits) and two tokens
    // per pass.  From 9 tokens on: two digits (15 bits) and three tokens per pass - the same six MMA columns and
    // the same shared memory, but an expert selected by three tokens, and the shared expert, need a third fewer
    // passes (16 tokens: 187 -> 178 us, 64 tokens: 512 -> 397 us per launch).
    static thread_local DecVariant v_small = make_variant<3, 2, 1>();
    static thread_local DecVariant v_23 = make_variant<2, 3, 1>();
    DecVariant &V = t >= LMOE_DEC_V23_FROM_T ? v_23 : v_small;
    const DecLayout L(H, F, E, t, K, V.ncol, V.ncw, V.nstage, V.nred);
    static thread_local int c_dev = -1, c_sms = 0, c_max_smem = 0;
    int dev = 0;
    LMOE_CUDA(cudaGetDevice(&dev));
    if (dev != c_dev) {
        LMOE_CUDA(cudaDeviceGetAttribute(&c_sms, cudaDevAttrMultiProcessorCount, dev));
        LMOE_CUDA(cudaDeviceGetAttribute(&c_max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        c_dev = dev;
    }
    if (L.total > c_max_smem)
        return lmoe_fail(LMOE_ERR_UNSUPPORTED, "fused decode needs %d bytes of shared memory per CTA, device allows %d",
                         L.total, c_max_smem);
    if (workspace_bytes < decode_workspace_bytes(t, H, F, E, K) || !workspace)
        return lmoe_fail(LMOE_ERR_WORKSPACE, "decode workspace needs %zu bytes, got %zu",
                         decode_workspace_bytes(t, H, F, E, K), workspace_bytes);
    if (V.c_dev != dev || V.c_total != L.total) {
        LMOE_CUDA(cudaFuncSetAttribute(V.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, L.total));
        LMOE_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&V.c_occ, V.fn, V.threads, L.total));
        V.c_dev = dev;
        V.c_total = L.total;
    }
    if (V.c_occ < 1) return lmoe_fail(LMOE_ERR_UNSUPPORTED, "fused decode kernel does not fit on an SM");
    const int occ = V.c_occ > V.min_ctas ? V.min_ctas : V.c_occ, sms = c_sms;

    DecodeParams P;
    P.x = x; P.out = out; P.ids_out = ids_out; P.w_out = w_out;
    P.router = Ly->router; P.bias = Ly->bias;
    P.ext_ids = ext_ids; P.ext_w = ext_w;
    P.gate = Ly->gate->blocks(); P.up = Ly->up->blocks(); P.down = Ly->down->blocks();
    if (shared_first < 0 || shared_count < 0 || shared_first + shared_count > t)
        return lmoe_fail(LMOE_ERR_INVALID, "shared-expert token range [%d, %d) lies outside the launch's %d tokens", shared_first,
                         shared_first + shared_count, t);
    P.has_shared = Ly->sh_gate != nullptr && shared_count > 0;
    P.sh_t0 = P.has_shared ? shared_first : 0;
    P.sh_nt = P.has_shared ? shared_count : 0;
    P.sh_gate = P.has_shared ? Ly->sh_gate->blocks() : nullptr;
    P.sh_up = P.has_shared ? Ly->sh_up->blocks() : nullptr;
    P.sh_down = P.has_shared ? Ly->sh_down->blocks() : nullptr;
    P.t = t; P.hidden = H; P.ff = F; P.n_expert = E; P.top_k = K;
    P.scale = Ly->scale; P.norm = Ly->norm;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    P.ctrl = reinterpret_cast<uint32_t *>(ws);
    P.sync = Ly->sync;
    P.first_launch = first_launch;
    size_t o = 65536;
    P.logits = reinterpret_cast<float *>(ws + o); o += lmoe_align_up((size_t)t * E * 4, 256);
    P.ids_ws = reinterpret_cast<uint32_t *>(ws + o); o += lmoe_align_up((size_t)t * K * 4, 256);
    P.w_ws = reinterpret_cast<float *>(ws + o); o += lmoe_align_up((size_t)t * K * 4, 256);
    P.act_f = reinterpret_cast<float *>(ws + o); o += lmoe_align_up((size_t)t * (K + 1) * F * 4, 256);
    P.ypart = reinterpret_cast<float *>(ws + o);
    void *args[] = {&P};
    LMOE_CUDA(cudaLaunchCooperativeKernel(V.fn, dim3(occ * sms), dim3(V.threads), args, (size_t)L.total, stream));
    return LMOE_OK;
}
