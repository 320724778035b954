// Shared device / host helpers of the MicroAdam B200 kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <algorithm>
#include "../../include/microadam_b200.h"

namespace mab {

// ----------------------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int  cuda_fail(cudaError_t e, const char* what);   // records and returns MAB_ERR_CUDA
int  device_sm_count();                            // cached per device, < 0 on failure
int  device_max_optin_smem();                      // < 0 on failure
void count_launch();                               // bumps the process-wide kernel launch counter

#define MAB_CUDA_TRY(expr)                                                     \
    do { cudaError_t _e = (expr); if (_e != cudaSuccess) return mab::cuda_fail(_e, #expr); } while (0)
#define MAB_REQUIRE(cond, code, ...)                                           \
    do { if (!(cond)) { mab::set_error(__VA_ARGS__); return (code); } } while (0)

static inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ----------------------------------------------------------------------------- element types
// bf16 values travel as their 16 bit patterns; conversions are spelled out so that the
// rounding (nearest-even) is visible and identical everywhere.
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

__device__ __forceinline__ uint16_t f32_to_bf16_bits_rne(float f) {
    // one conversion instruction; finite inputs and infinities (NaN is outside the contract of the step)
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
}

template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int code = MAB_F32;
    __device__ __forceinline__ static float load(const float* p, int64_t i) { return p[i]; }
    __device__ __forceinline__ static void store(float* p, int64_t i, float v) { p[i] = v; }
    __device__ __forceinline__ static float round(float v) { return v; }
};
template <> struct Elem<uint16_t> {   // bf16 bits
    static constexpr int code = MAB_BF16;
    __device__ __forceinline__ static float load(const uint16_t* p, int64_t i) { return bf16_bits_to_f32(p[i]); }
    __device__ __forceinline__ static void store(uint16_t* p, int64_t i, float v) { p[i] = f32_to_bf16_bits_rne(v); }
    __device__ __forceinline__ static float round(float v) { return bf16_bits_to_f32(f32_to_bf16_bits_rne(v)); }
};

// ----------------------------------------------------------------------------- 4-bit codec
// One quantisation block's decode constants: u = (max - min) / 15 with one rounding per operation.
struct QParams { float mn, u; };

// RN(d / 15).  For 2^-100 <= |d| <= 2^100 the quotient is d * RN(1/15) with one residual correction (the
// residual d - 15 q is exact in an FMA): equal to the IEEE division for every float in that range (checked
// exhaustively on a CPU), without the division's special-function instruction and its slow-path branch.
__device__ __forceinline__ float div15_rn(float d) {
    const float ad = fabsf(d);
    if (!(ad >= 7.8886091e-31f && ad <= 1.2676506e30f)) return __fdiv_rn(d, 15.0f);   // zero, tiny, huge, NaN
    const float c = 0.0666666701436042785644531f;                                      // RN(1 / 15)
    const float q = __fmul_rn(d, c);
    return __fmaf_rn(__fmaf_rn(-15.0f, q, d), c, q);
}

// RN(1 / u) for 2^-100 <= u <= 2^100: the approximate reciprocal (within 3 ulp) and two Newton steps give the
// correctly rounded one for every float in that range but those whose mantissa bits are all ones (checked
// exhaustively on a CPU, for every start within 3 ulp); those take the library's form.
__device__ __forceinline__ float rcp_rn_normal(float u) {
    if ((__float_as_uint(u) & 0x7FFFFFu) == 0x7FFFFFu) return __frcp_rn(u);
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(u));
    float e = __fmaf_rn(-u, y, 1.0f);
    y = __fmaf_rn(y, e, y);
    e = __fmaf_rn(-u, y, 1.0f);
    return __fmaf_rn(y, e, y);
}

__device__ __forceinline__ QParams qparams(uint16_t mn_bits, uint16_t mx_bits) {
    QParams q;
    q.mn = bf16_bits_to_f32(mn_bits);
    q.u = div15_rn(__fsub_rn(bf16_bits_to_f32(mx_bits), q.mn));
    return q;
}

// Qinv of one code: f32(code) * u, then + min; two roundings, never fused.
__device__ __forceinline__ float qinv(uint32_t code, const QParams& q) {
    return __fadd_rn(__fmul_rn(static_cast<float>(code), q.u), q.mn);
}

// Q of one value: 0 when u == 0, else clamp(floor((r - min) / u + 0.5), 0, 15).
__device__ __forceinline__ uint32_t qcode_exact(float r, const QParams& q) {
    if (q.u == 0.0f) return 0u;
    float s = __fadd_rn(__fdiv_rn(__fsub_rn(r, q.mn), q.u), 0.5f);
    float c = floorf(s);
    c = fminf(fmaxf(c, 0.0f), 15.0f);   // NaN (0/0 cannot occur with u != 0; inf - inf can) -> 0 through fmaxf
    return static_cast<uint32_t>(c);
}

// ----------------------------------------------------------------------------- block primitives
__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

// Exclusive prefix sum of one int per thread over the block; `total` gets the block sum.
// `scratch` holds at least 33 ints.  Contains two __syncthreads().
__device__ __forceinline__ int block_exclusive_scan(int v, int* scratch, int& total) {
    const int lane = lane_id(), warp = warp_id();
    const int nwarps = (blockDim.x + 31) >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) scratch[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int w = (lane < nwarps) ? scratch[lane] : 0;
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        scratch[lane] = winc - w;           // exclusive warp offsets
        if (lane == 31) scratch[32] = winc;  // block total
    }
    __syncthreads();
    total = scratch[32];
    int r = scratch[warp] + inc - v;
    return r;
}

}  // namespace mab
