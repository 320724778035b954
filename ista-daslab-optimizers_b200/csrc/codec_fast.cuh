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
// overflow and u >= +0 (a negative u would turn the +0 of code 0 into -0): `fast` says so.
// Two elements per instruction: the packed f32x2 forms round each component like the scalar ones.
// The constants depend on the quantisation block only; callers that decode several octets of a
// block build them once.
struct DecodeConsts { float2 u2, nb2, mn2; bool fast; };

__device__ __forceinline__ DecodeConsts decode_consts(const QParams& q) {
    DecodeConsts c;
    const float nb = -(8388608.0f * q.u);
    c.u2 = make_float2(q.u, q.u); c.nb2 = make_float2(nb, nb); c.mn2 = make_float2(q.mn, q.mn);
    c.fast = q.u >= 0.0f && q.u < CODEC_U_MAX;          // also false for NaN
    return c;
}

__device__ __forceinline__ void decode_octet_fast(uint32_t w, const DecodeConsts& c, float (&x)[8]) {
    uint32_t hi, lo;
    split_nibbles(w, hi, lo);
    float2 p;
    p = __fadd2_rn(__ffma2_rn(make_float2(magic_byte<0>(hi), magic_byte<0>(lo)), c.u2, c.nb2), c.mn2); x[0] = p.x; x[1] = p.y;
    p = __fadd2_rn(__ffma2_rn(make_float2(magic_byte<1>(hi), magic_byte<1>(lo)), c.u2, c.nb2), c.mn2); x[2] = p.x; x[3] = p.y;
    p = __fadd2_rn(__ffma2_rn(make_float2(magic_byte<2>(hi), magic_byte<2>(lo)), c.u2, c.nb2), c.mn2); x[4] = p.x; x[5] = p.y;
    p = __fadd2_rn(__ffma2_rn(make_float2(magic_byte<3>(hi), magic_byte<3>(lo)), c.u2, c.nb2), c.mn2); x[6] = p.x; x[7] = p.y;
}

__device__ __forceinline__ void decode_octet_exact(uint32_t w, const QParams& q, float (&x)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = qinv((w >> (8 * (e >> 1) + ((e & 1) ? 0 : 4))) & 0xFu, q);
}

__device__ __forceinline__ void decode_octet(uint32_t w, const QParams& q, float (&x)[8]) {
    const DecodeConsts c = decode_consts(q);
    if (c.fast) decode_octet_fast(w, c, x);
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
// unless s~ lies within 2^-16 of an integer; those (rare) elements, and every element when u is
// outside [2^-100, 2^100] (zero, subnormal, infinite), are coded with the exact definition.
// The clamp to [0.25, 15.5] keeps floor() in 0..15 and maps every out-of-range s to the code the
// definition's clamp gives it.  CLAMP = false is for callers whose statistics are the exact
// minimum and maximum of the values (bf16 data: no rounding of the statistics), where
// 0 <= r - mn <= mx - mn makes s~ fall in [0.5, 15.5 + 2^-18] by itself.
// min and max of 8 values with the 3-input min / max of sm_100.
__device__ __forceinline__ float min3(float a, float b, float c) { float d; asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
__device__ __forceinline__ float max3(float a, float b, float c) { float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d; }
__device__ __forceinline__ void octet_min_max(const float (&v)[8], float& lo, float& hi) {
    lo = fminf(min3(v[0], v[1], v[2]), min3(min3(v[3], v[4], v[5]), v[6], v[7]));
    hi = fmaxf(max3(v[0], v[1], v[2]), max3(max3(v[3], v[4], v[5]), v[6], v[7]));
}

struct EncodeConsts { float2 nmn2, r02; bool fast; };

__device__ __forceinline__ EncodeConsts encode_consts(const QParams& q) {
    EncodeConsts c;
    c.fast = q.u >= CODEC_U_MIN && q.u <= CODEC_U_MAX;
    const float r0 = c.fast ? rcp_rn_normal(q.u) : 0.0f;
    c.nmn2 = make_float2(-q.mn, -q.mn); c.r02 = make_float2(r0, r0);
    return c;
}

// Requires c.fast.
template <bool CLAMP>
__device__ __forceinline__ uint32_t encode_octet_fast(const float (&r)[8], const QParams& q, const EncodeConsts& c) {
    const float MAGIC = 12582912.0f;              // 1.5 * 2^23: low mantissa bits of x + MAGIC hold round-down(x)
    const float2 half2v = make_float2(0.5f, 0.5f);
    const float2 mg2 = make_float2(MAGIC, MAGIC), nmg2 = make_float2(-MAGIC, -MAGIC), neg1 = make_float2(-1.0f, -1.0f);
    const float2 nhalf2 = make_float2(-0.5f, -0.5f);
    float f[8], d[8];
    float worst = 0.0f;                            // largest |frac(s~) - 0.5| of the octet
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float2 s = __ffma2_rn(__fadd2_rn(make_float2(r[2 * b], r[2 * b + 1]), c.nmn2), c.r02, half2v);   // r - mn == r + (-mn)
        if (CLAMP) {
            s.x = fminf(fmaxf(s.x, 0.25f), 15.5f);
            s.y = fminf(fmaxf(s.y, 0.25f), 15.5f);
        }
        const float2 fl = __fadd2_rn(__fadd2_rd(s, mg2), nmg2);         // floor(s), exact
        const float2 dd = __fadd2_rn(__ffma2_rn(fl, neg1, s), nhalf2);   // (s - floor(s)) - 0.5, exact
        worst = fmaxf(worst, fmaxf(fabsf(dd.x), fabsf(dd.y)));
        f[2 * b] = fl.x; f[2 * b + 1] = fl.y;
        d[2 * b] = dd.x; d[2 * b + 1] = dd.y;
    }
    if (worst > 0.5f - 1.52587890625e-5f) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (fabsf(d[e]) > 0.5f - 1.52587890625e-5f) f[e] = static_cast<float>(qcode_exact(r[e], q));
    }
    // byte b = 16 * code(2b) + code(2b+1), built in float and read from the low mantissa byte
    const uint32_t b0 = __float_as_uint(__fmaf_rn(f[0], 16.0f, f[1]) + 8388608.0f);
    const uint32_t b1 = __float_as_uint(__fmaf_rn(f[2], 16.0f, f[3]) + 8388608.0f);
    const uint32_t b2 = __float_as_uint(__fmaf_rn(f[4], 16.0f, f[5]) + 8388608.0f);
    const uint32_t b3 = __float_as_uint(__fmaf_rn(f[6], 16.0f, f[7]) + 8388608.0f);
    return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}

// The same codes without the per-octet branch: `worst` returns the largest |frac(s~) - 0.5| of the
// octet, and the caller re-codes the octet with encode_octet_fast when it exceeds CODEC_SAFE_FRAC.
// Several octets coded this way in a row overlap in the pipeline.  Requires c.fast.
constexpr float CODEC_SAFE_FRAC = 0.5f - 1.52587890625e-5f;
template <bool CLAMP>
__device__ __forceinline__ uint32_t encode_octet_speculative(const float (&r)[8], const EncodeConsts& c, float& worst) {
    const float MAGIC = 12582912.0f;
    const float2 half2v = make_float2(0.5f, 0.5f);
    const float2 mg2 = make_float2(MAGIC, MAGIC), nmg2 = make_float2(-MAGIC, -MAGIC), neg1 = make_float2(-1.0f, -1.0f);
    const float2 nhalf2 = make_float2(-0.5f, -0.5f);
    float f[8];
    worst = 0.0f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float2 s = __ffma2_rn(__fadd2_rn(make_float2(r[2 * b], r[2 * b + 1]), c.nmn2), c.r02, half2v);
        if (CLAMP) {
            s.x = fminf(fmaxf(s.x, 0.25f), 15.5f);
            s.y = fminf(fmaxf(s.y, 0.25f), 15.5f);
        }
        const float2 fl = __fadd2_rn(__fadd2_rd(s, mg2), nmg2);
        const float2 dd = __fadd2_rn(__ffma2_rn(fl, neg1, s), nhalf2);
        worst = fmaxf(worst, fmaxf(fabsf(dd.x), fabsf(dd.y)));
        f[2 * b] = fl.x; f[2 * b + 1] = fl.y;
    }
    const uint32_t b0 = __float_as_uint(__fmaf_rn(f[0], 16.0f, f[1]) + 8388608.0f);
    const uint32_t b1 = __float_as_uint(__fmaf_rn(f[2], 16.0f, f[3]) + 8388608.0f);
    const uint32_t b2 = __float_as_uint(__fmaf_rn(f[4], 16.0f, f[5]) + 8388608.0f);
    const uint32_t b3 = __float_as_uint(__fmaf_rn(f[6], 16.0f, f[7]) + 8388608.0f);
    return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}

template <bool CLAMP = true>
__device__ __forceinline__ uint32_t encode_octet(const float (&r)[8], const QParams& q) {
    const EncodeConsts c = encode_consts(q);
    if (!c.fast) return encode_octet_exact(r, q, 8);
    return encode_octet_fast<CLAMP>(r, q, c);
}

// Codes of one octet by the defining form floor(RN(RN((r - mn) / u) + 0.5)) itself, two elements per
// instruction and without division or conversion instructions; u in [2^-100, 2^100].  The IEEE quotient
// comes from the correctly rounded reciprocal r0 = RN(1 / u): q = RN(d * r0) is within 1.5 ulp of d / u, one
// residual correction q <- RN(q + RN(d - q * u) * r0) (the residual is exact in an FMA) makes it faithful,
// and a second one makes it the correctly rounded quotient (Markstein's theorem on the final step of a
// division).  Values far below half a step, where the residual could underflow, get code 0 from any
// quotient below 0.5.  floor: adding 2^23 with rounding down leaves the integer in the low mantissa bits.
// CLAMP: values may lie outside [mn, mn + 15 u] (statistics rounded to bf16): s is clamped to [0, 15.5]
// before the floor, which gives the codes the defining clamp(floor(s), 0, 15) gives.
struct DivConsts { float2 nmn2, r02, nu2; };

__device__ __forceinline__ DivConsts div_consts(const QParams& q) {
    DivConsts c;
    const float r0 = (q.u >= CODEC_U_MIN && q.u <= CODEC_U_MAX) ? rcp_rn_normal(q.u) : 0.0f;   // (unused outside that range)
    c.nmn2 = make_float2(-q.mn, -q.mn); c.r02 = make_float2(r0, r0); c.nu2 = make_float2(-q.u, -q.u);
    return c;
}

template <bool CLAMP>
__device__ __forceinline__ uint32_t encode_octet_div_f32(const float (&r)[8], const DivConsts& c) {
    const float2 half2 = make_float2(0.5f, 0.5f), magic2 = make_float2(8388608.0f, 8388608.0f);
    uint32_t y[8];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float2 d = __fadd2_rn(make_float2(r[2 * p], r[2 * p + 1]), c.nmn2);   // r - mn
        float2 q = __fmul2_rn(d, c.r02);
        q = __ffma2_rn(__ffma2_rn(q, c.nu2, d), c.r02, q);
        q = __ffma2_rn(__ffma2_rn(q, c.nu2, d), c.r02, q);                          // RN(d / u)
        float2 s = __fadd2_rn(q, half2);
        if (CLAMP) {
            s.x = fminf(fmaxf(s.x, 0.0f), 15.5f);
            s.y = fminf(fmaxf(s.y, 0.0f), 15.5f);
        }
        const float2 f = __fadd2_rd(s, magic2);                                     // 2^23 + floor(s)
        y[2 * p] = __float_as_uint(f.x); y[2 * p + 1] = __float_as_uint(f.y);
    }
    // byte 0 of every float is the code; even elements go to the high nibbles
    const uint32_t ev = __byte_perm(__byte_perm(y[0], y[2], 0x0040), __byte_perm(y[4], y[6], 0x0040), 0x5410);
    const uint32_t od = __byte_perm(__byte_perm(y[1], y[3], 0x0040), __byte_perm(y[5], y[7], 0x0040), 0x5410);
    return (ev << 4) | od;
}

// Two floats -> two bf16 (round to nearest even) in one conversion; low half = first value.
__device__ __forceinline__ uint32_t pack_bf16x2_rne(float a, float b) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
    return d;
}

// |x| of two packed bf16 values.
__device__ __forceinline__ uint32_t abs_bf16x2(uint32_t a) { return a & 0x7FFF7FFFu; }

// Lane-wise maximum of two packed bf16 pairs.
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Lane-wise max(|a|, |b|); the sign bit of each lane is the xor of the operands' signs (mask it off).
__device__ __forceinline__ uint32_t maxabs_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t min_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("min.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

}  // namespace mab
