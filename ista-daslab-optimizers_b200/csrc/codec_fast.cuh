// Octet-wide (8 elements, 4 code bytes) forms of the 4-bit codec that avoid the conversion /
// special-function pipe (I2F, F2I, FRND, MUFU run at a quarter of the FP32 rate on sm_100) and
// the IEEE division per element, while returning exactly the bits of the scalar definitions
// in common.cuh (qinv, qcode_exact).
#pragma once
#include "common.cuh"

namespace mab {

constexpr float CODEC_U_MAX = 1.2676506e30f;      // 2^100
constexpr float CODEC_U_MIN = 7.8886091e-31f;     // 2^-100

// Element e (0..7) of an octet: code byte e/2 of the little-endian word, even element in the high
// nibble.  `hi` / `lo` hold the high / low nibbles of the four bytes, one per byte.
__device__ __forceinline__ void split_nibbles(uint32_t w, uint32_t& hi, uint32_t& lo) {
    hi = (w >> 4) & 0x0F0F0F0Fu;
    lo = w & 0x0F0F0F0Fu;
}

// 2^23 + (byte `i` of v) as a float: byte permute builds 0x4B0000cc without a conversion.
template <int I>
__device__ __forceinline__ float magic_byte(uint32_t v) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7540u | I));
}

// x[e] = Qinv(code_e) = RN(RN(code * u) + mn).  With F = 2^23 + code (exact), fma(F, u, -2^23 u)
// rounds the exact value code * u once, which is RN(code * u); valid while 2^23 * |u| does not
// overflow and u >= +0 (a negative u would turn the +0 of code 0 into -0); the caller checks both.
__device__ __forceinline__ void decode_octet_fast(uint32_t w, const QParams& q, float (&x)[8]) {
    uint32_t hi, lo;
    split_nibbles(w, hi, lo);
    const float nb = -(8388608.0f * q.u);
    x[0] = __fadd_rn(__fmaf_rn(magic_byte<0>(hi), q.u, nb), q.mn);
    x[1] = __fadd_rn(__fmaf_rn(magic_byte<0>(lo), q.u, nb), q.mn);
    x[2] = __fadd_rn(__fmaf_rn(magic_byte<1>(hi), q.u, nb), q.mn);
    x[3] = __fadd_rn(__fmaf_rn(magic_byte<1>(lo), q.u, nb), q.mn);
    x[4] = __fadd_rn(__fmaf_rn(magic_byte<2>(hi), q.u, nb), q.mn);
    x[5] = __fadd_rn(__fmaf_rn(magic_byte<2>(lo), q.u, nb), q.mn);
    x[6] = __fadd_rn(__fmaf_rn(magic_byte<3>(hi), q.u, nb), q.mn);
    x[7] = __fadd_rn(__fmaf_rn(magic_byte<3>(lo), q.u, nb), q.mn);
}

__device__ __forceinline__ void decode_octet_exact(uint32_t w, const QParams& q, float (&x)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = qinv((w >> (8 * (e >> 1) + ((e & 1) ? 0 : 4))) & 0xFu, q);
}

__device__ __forceinline__ void decode_octet(uint32_t w, const QParams& q, float (&x)[8]) {
    if (q.u >= 0.0f && q.u < CODEC_U_MAX) decode_octet_fast(w, q, x);   // also false for NaN
    else decode_octet_exact(w, q, x);
}

__device__ __forceinline__ uint32_t encode_octet_exact(const float (&r)[8], const QParams& q, int cnt) {
    uint32_t w = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint32_t c = (e < cnt) ? qcode_exact(r[e], q) : 0u;
        w |= c << (8 * (e >> 1) + ((e & 1) ? 0 : 4));
    }
    return w;
}

// Codes of a full octet.  s~ = (r - mn) * (1/u) + 0.5 differs from the defining
// s = RN(RN((r - mn) / u) + 0.5) by less than 2^-17 for |s| <= 16.5, so floor(s~) = floor(s)
// unless s~ lies within 2^-16 of an integer; in that (rare) case, and for u outside
// [2^-100, 2^100] (zero, subnormal, infinite), the octet is redone with the exact definition.
// The clamp to [0.25, 15.5] keeps floor() in 0..15 and maps every out-of-range s to the code the
// definition's clamp gives it.
__device__ __forceinline__ uint32_t encode_octet(const float (&r)[8], const QParams& q) {
    if (!(q.u >= CODEC_U_MIN && q.u <= CODEC_U_MAX)) return encode_octet_exact(r, q, 8);
    const float r0 = __frcp_rn(q.u);
    const float MAGIC = 12582912.0f;              // 1.5 * 2^23: low mantissa bits of x + MAGIC hold round-down(x)
    float f[8];
    bool unsafe = false;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float s = __fmaf_rn(__fsub_rn(r[e], q.mn), r0, 0.5f);
        s = fminf(fmaxf(s, 0.25f), 15.5f);
        const float fl = __fadd_rd(s, MAGIC) - MAGIC;       // floor(s), exact
        const float frac = s - fl;                           // exact, in [0, 1)
        unsafe |= fabsf(frac - 0.5f) > 0.5f - 1.52587890625e-5f;
        f[e] = fl;
    }
    if (unsafe) return encode_octet_exact(r, q, 8);
    // byte b = 16 * code(2b) + code(2b+1), built in float and read from the low mantissa byte
    const uint32_t b0 = __float_as_uint(__fmaf_rn(f[0], 16.0f, f[1]) + 8388608.0f);
    const uint32_t b1 = __float_as_uint(__fmaf_rn(f[2], 16.0f, f[3]) + 8388608.0f);
    const uint32_t b2 = __float_as_uint(__fmaf_rn(f[4], 16.0f, f[5]) + 8388608.0f);
    const uint32_t b3 = __float_as_uint(__fmaf_rn(f[6], 16.0f, f[7]) + 8388608.0f);
    return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}

}  // namespace mab
