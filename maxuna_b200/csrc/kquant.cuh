// Q4_K / Q6_K super-block field access on the device.
//
// Q4_K, 144 bytes, 256 weights:  f16 d; f16 dmin; u8 scales[12]; u8 qs[128]
//   weight(64j + l)      = d*sc[2j]  *(qs[32j+l] & 15) - dmin*m[2j]      l < 32
//   weight(64j + 32 + l) = d*sc[2j+1]*(qs[32j+l] >> 4) - dmin*m[2j+1]
// Q6_K, 210 bytes, 256 weights:  u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d
//   weight(128n + 32i + l) = d*sc[8n + 2i + l/16]*(q - 32), q 6 bits from ql/qh
// (block layouts: src/ops/mv.metal:55-75 of the reference; decode rules:
// src/ops/mm_id.metal:89-111, 136-167).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

__device__ __forceinline__ float lmoe_h2f(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// 6-bit (scale, min) pair j (0..7) of a Q4_K super-block; `s` -> scales[12].
__device__ __forceinline__ void q4k_scale_min(const uint8_t *s, int j, int &sc, int &mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0f) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// All eight (scale, min) pairs from the 12 packed bytes held as three words.
__device__ __forceinline__ void q4k_unpack_scales(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t &sc_lo,
                                                  uint32_t &sc_hi, uint32_t &mn_lo, uint32_t &mn_hi) {
    // bytes 0..3: sc0..3 (6b) + top 2 bits of sc4..7; bytes 4..7: m0..3 + top bits of m4..7;
    // bytes 8..11: low nibbles sc4..7 | m4..7 << 4.
    sc_lo = s0 & 0x3f3f3f3fu;
    mn_lo = s1 & 0x3f3f3f3fu;
    sc_hi = (s2 & 0x0f0f0f0fu) | ((s0 >> 2) & 0x30303030u);
    mn_hi = ((s2 >> 4) & 0x0f0f0f0fu) | ((s1 >> 2) & 0x30303030u);
}

__device__ __forceinline__ uint32_t ld_u32_unaligned2(const uint8_t *p) {
    // p is 2-byte aligned
    const uint16_t *q = reinterpret_cast<const uint16_t *>(p);
    return (uint32_t)q[0] | ((uint32_t)q[1] << 16);
}
