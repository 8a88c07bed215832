// Pieces shared by the kernels that stream quantized rows through shared memory and feed them to the
// integer tensor-core path (the fused decode kernel and the plain Q6_K mat-vec): mbarrier / bulk-copy
// wrappers with bounded waits, the mma.sync forms, and the Q6_K super-block product.
#pragma once
#include "fused.cuh"
#include "kquant.cuh"

constexpr uint32_t SPIN_LIMIT = 1u << 22;

// ---- PTX helpers -------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The non-suspending test of the same condition: answers at once.  Used to ask about the NEXT unit's barriers before
// the current unit's arithmetic, so that the answer's latency (a few hundred cycles even for a completed phase) passes
// under the arithmetic instead of in front of it.
__device__ __forceinline__ bool mbar_test(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after SPIN_LIMIT polls, records the fact and carries on
// (results are then invalid, but every loop in the kernel stays finite).
template <int BACKOFF_NS = 0>
__device__ __forceinline__ void mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *ctrl, uint32_t where) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return;
        // once any wait of the launch has given up the results are void: every later wait returns at once,
        // so a launch that went wrong still ends quickly
        if ((i & 1023u) == 1023u && *reinterpret_cast<volatile uint32_t *>(ctrl) != 0u) return;
        // service warps (producer, epilogue) poll slowly so that they do not take issue slots from the math
        if (BACKOFF_NS > 0) __nanosleep(BACKOFF_NS);
    }
    if (atomicCAS(ctrl, 0u, (uint32_t)LMOE_FLAG_WAIT_TIMEOUT) == 0u) {
        ctrl[1] = where;
        ctrl[2] = blockIdx.x;
    }
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}


// d = a*b (fresh accumulator: C is the zero register, no moves needed)
__device__ __forceinline__ void mma16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// Integer forms: unsigned 8-bit weights (A) times signed 8-bit activation digits (B), exact s32 sums.
// k = 32: a0/a2 = row g, k slots 4t.. / 16+4t..; a1/a3 = row g+8; b0/b1 = column g, the same k slots.
__device__ __forceinline__ void imma16832_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// k = 16: a0 = row g, a1 = row g+8, b0 = column g, all k slots 4t..4t+3.
__device__ __forceinline__ void imma16816_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%7,%7,%7};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// byte i (0..3) of `w`, zero- or sign-extended
__device__ __forceinline__ int ubyte(uint32_t w, int i) { return (int)__byte_perm(w, 0u, 0x4440u + i); }
__device__ __forceinline__ int sbyte(uint32_t w, int i) {
    // selector nibbles i, 8|i, 8|i, 8|i: the byte, then its sign bit replicated (the intrinsic ignores bit 3)
    int r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(0u), "r"((uint32_t)(i | ((8 | i) * 0x1110))));
    return r;
}

// Four bytes at p + off.  MODE 0: p is word aligned.  MODE 1: p is 2 (mod 4), the bytes straddle two
// aligned words.  MODE 2: either, decided per lane (both words are always inside shared memory).
template <int MODE>
__device__ __forceinline__ uint32_t lds32(const uint8_t *p, int off) {
    if (MODE == 0) return *reinterpret_cast<const uint32_t *>(p + off);
    if (MODE == 1) {
        const uint32_t lo = *reinterpret_cast<const uint32_t *>(p + off - 2);
        const uint32_t hi = *reinterpret_cast<const uint32_t *>(p + off + 2);
        return __byte_perm(lo, hi, 0x5432);
    }
    const uintptr_t a = reinterpret_cast<uintptr_t>(p + off);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
    return __byte_perm(q[0], q[1], (a & 2) ? 0x5432u : 0x3210u);
}

__device__ __forceinline__ uint32_t sc_pair_half2(const int8_t *p) {
    const __half2 h = __floats2half2_rn((float)p[0], (float)p[1]);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// One Q6_K super-block of two rows (bg -> accumulators 0/1, bG -> 2/3) that have the same alignment.  The six-bit value of a
// weight (low nibble | two high bits << 4, 0..63) is one byte of a k = 16 integer MMA: one MMA per 16-wide
// sub-block, whose signed scale multiplies the exact integer sum.
template <int MIS>
__device__ __forceinline__ void q6k_block(const uint8_t *bg, const uint8_t *bG, int b, int t, const int8_t *xcol,
                                          const __half *scol, const float *sxs, float r0, float r1, float (&acc)[4]) {
    constexpr uint32_t M4 = 0x0F0F0F0Fu, M2 = 0x30303030u;
    const int8_t *scg = reinterpret_cast<const int8_t *>(bg + 192);
    const int8_t *scG = reinterpret_cast<const int8_t *>(bG + 192);
    const float dg = lmoe_h2f(*reinterpret_cast<const uint16_t *>(bg + 208));
    const float dG = lmoe_h2f(*reinterpret_cast<const uint16_t *>(bG + 208));
    // "-32" offset: one f16 MMA, A = the 16 sub-block scales of each row, B = 16-wide activation sums
    float co[4];
    {
        const uint32_t s0 = *reinterpret_cast<const uint32_t *>(scol + 16 * b + 2 * t);
        const uint32_t s1 = *reinterpret_cast<const uint32_t *>(scol + 16 * b + 2 * t + 8);
        mma16816_z(co, sc_pair_half2(scg + 2 * t), sc_pair_half2(scG + 2 * t), sc_pair_half2(scg + 2 * t + 8),
                   sc_pair_half2(scG + 2 * t + 8), s0, s1);
    }
    int al[4] = {0, 0, 0, 0};
#pragma unroll
    for (int n = 0; n < 2; n++) {
        const uint32_t swg0 = lds32<MIS>(bg, 192 + 8 * n), swg1 = lds32<MIS>(bg, 196 + 8 * n);
        const uint32_t swG0 = lds32<MIS>(bG, 192 + 8 * n), swG1 = lds32<MIS>(bG, 196 + 8 * n);
#pragma unroll
        for (int c = 0; c < 2; c++) {
            const int l0 = 16 * c + 4 * t;
            const uint32_t qa_g = lds32<MIS>(bg, 64 * n + l0), qb_g = lds32<MIS>(bg, 64 * n + 32 + l0);
            const uint32_t qh_g = lds32<MIS>(bg, 128 + 32 * n + l0);
            const uint32_t qa_G = lds32<MIS>(bG, 64 * n + l0), qb_G = lds32<MIS>(bG, 64 * n + 32 + l0);
            const uint32_t qh_G = lds32<MIS>(bG, 128 + 32 * n + l0);
            const int8_t *xp = xcol + 256 * b + 128 * n + l0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                // group i: q1 (ql lo | qh 0-1), q2 (ql+32 lo | qh 2-3), q3 (ql hi | qh 4-5), q4 (ql+32 hi | qh 6-7)
                const uint32_t qg = (i & 1) ? qb_g : qa_g, qG = (i & 1) ? qb_G : qa_G;
                const uint32_t lg = (i & 2) ? (qg >> 4) : qg, lG = (i & 2) ? (qG >> 4) : qG;
                const uint32_t hg = i == 0 ? (qh_g << 4) : (i == 1 ? (qh_g << 2) : (i == 2 ? qh_g : (qh_g >> 2)));
                const uint32_t hG = i == 0 ? (qh_G << 4) : (i == 1 ? (qh_G << 2) : (i == 2 ? qh_G : (qh_G >> 2)));
                const uint32_t a0 = (lg & M4) | (hg & M2), a1 = (lG & M4) | (hG & M2);
                const uint32_t xv = *reinterpret_cast<const uint32_t *>(xp + 32 * i);
                int f[4];
                imma16816_z(f, a0, a1, xv);
                // scale index within the half: 2*i + c -> byte 2*(i & 1) + c of word i >> 1
                const int sg = sbyte(i < 2 ? swg0 : swg1, 2 * (i & 1) + c);
                const int sG = sbyte(i < 2 ? swG0 : swG1, 2 * (i & 1) + c);
                al[0] += sg * f[0]; al[1] += sg * f[1]; al[2] += sG * f[2]; al[3] += sG * f[3];
            }
        }
    }
    const float2 cs = *reinterpret_cast<const float2 *>(sxs + 8 * b + 2 * t);
    // r0 / r1: 32 * sum_ratio of columns 2t / 2t+1
    acc[0] += dg * (cs.x * ((float)al[0] - r0 * co[0]));
    acc[1] += dg * (cs.y * ((float)al[1] - r1 * co[1]));
    acc[2] += dG * (cs.x * ((float)al[2] - r0 * co[2]));
    acc[3] += dG * (cs.y * ((float)al[3] - r1 * co[3]));
}
