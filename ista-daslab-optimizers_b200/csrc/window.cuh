// Sparse window -> dense Adam-style update for one sub-range of a top-k block, in shared memory.
//
// A top-k block is cut into sub-ranges of at most WIN_SR elements (a multiple of 128, so that
// every sub-range starts on a quantisation-block boundary for quant_block_size <= 128).  For one
// sub-range the CTA
//   1. zeroes two float accumulators (first and second moment) of WIN_SR elements,
//   2. walks the window entries of the block (rows r < rows, the block's slice of I / V) row after row with a
//      barrier between rows and adds those whose position falls in the sub-range (positions are unique inside
//      a row, so a row needs no atomics, and the fixed row order makes the float sums reproducible bit for
//      bit on any grid and any GPU count),
//   3. turns (m, v) into the update u wherever the second moment is non-zero (one pass over the
//      accumulators instead of a second pass over the entries), leaving u = 0 elsewhere in the first array.
// The caller then streams over the sub-range reading u from shared memory.
#pragma once
#include "common.cuh"

namespace mab {

constexpr int WIN_SR = 7296;          // 57 * 128 elements per sub-range: a 29 056-element block is four sub-ranges
constexpr int WIN_THREADS = 512;      // two CTAs per SM
constexpr int WIN_EPT = 4;            // window entries of a row a thread holds in registers
constexpr int WIN_SMEM_BYTES = 2 * WIN_SR * 4;
constexpr int WIN_MAX_TENSORS = 512;  // tensors per launch (their unit prefix sits in shared memory)

struct WindowArgs {
    int   rows;                       // valid window rows: min(steps, m)
    int   m;                          // allocated window rows
    float w1[MAB_MAX_WINDOW];         // beta1^age(r) * (1 - beta1), indexed by row
    float w2[MAB_MAX_WINDOW];
    float bc1, bc2, eps;              // 1 - beta1^steps, 1 - beta2^steps
    float alpha, one_minus_alpha;
    int   qbs;
    int   lanes_per_qb;               // qbs / 8 (fused path only)
    double* probe;                    // nullptr, or the probe buffer the step adds the update's statistics to
};

struct WindowSmem {
    float*    m_acc;                  // after finalize: u
    float*    v_acc;
    __device__ explicit WindowSmem(unsigned char* base)
        : m_acc(reinterpret_cast<float*>(base)), v_acc(m_acc + WIN_SR) {}
};

// Fast (not correctly rounded) form of m_hat / (sqrt(v_hat) + eps): the update is specified to
// a tolerance, and the approximations are deterministic.
__device__ __forceinline__ float adam_update_fast(float m, float v, float inv_bc1, float inv_bc2, float eps) {
    float s;
    asm("sqrt.approx.f32 %0, %1;" : "=f"(s) : "f"(v * inv_bc2));
    return __fdividef(m * inv_bc1, s + eps);
}

// I_blk / V_blk point at the block's slice of row 0; row_pitch = k; kcnt entries per row;
// sub-range = block positions [s0, s0 + len).  Leaves u in sm.m_acc[0..len).  Ends with a barrier.
__device__ __forceinline__ void window_to_update(const int16_t* __restrict__ I_blk, const uint16_t* __restrict__ V_blk,
                                                 int64_t row_pitch, int kcnt, int s0, int len,
                                                 const WindowArgs& a, WindowSmem& sm) {
    const int t = threadIdx.x;
    for (int i = t; i < WIN_SR; i += WIN_THREADS) { sm.m_acc[i] = 0.0f; sm.v_acc[i] = 0.0f; }
    __syncthreads();
    // row after row, straight from global memory; a thread's first WIN_EPT entries of the next row are fetched
    // before the work on the current one (one exposed load latency per row at most)
    int n_pos[WIN_EPT];
    uint32_t n_val[WIN_EPT];
#pragma unroll
    for (int e = 0; e < WIN_EPT; ++e) {
        const int j = t + e * WIN_THREADS;
        n_pos[e] = (j < kcnt) ? (int)I_blk[j] : -1;
        n_val[e] = (j < kcnt) ? (uint32_t)V_blk[j] : 0u;
    }
    for (int r = 0; r < a.rows; ++r) {
        const int16_t* I_r = I_blk + (int64_t)r * row_pitch;
        const uint16_t* V_r = V_blk + (int64_t)r * row_pitch;
        const float w1 = a.w1[r], w2 = a.w2[r];
        int pos[WIN_EPT];
        uint32_t vb[WIN_EPT];
#pragma unroll
        for (int e = 0; e < WIN_EPT; ++e) { pos[e] = n_pos[e] - s0; vb[e] = n_val[e]; }
        if (r + 1 < a.rows) {
#pragma unroll
            for (int e = 0; e < WIN_EPT; ++e) {
                const int j = t + e * WIN_THREADS;
                if (j < kcnt) { n_pos[e] = (int)I_r[row_pitch + j]; n_val[e] = (uint32_t)V_r[row_pitch + j]; }
            }
        }
#pragma unroll
        for (int e = 0; e < WIN_EPT; ++e) {
            if (t + e * WIN_THREADS < kcnt && pos[e] >= 0 && pos[e] < len) {
                const float val = __uint_as_float(vb[e] << 16);
                sm.m_acc[pos[e]] = __fadd_rn(sm.m_acc[pos[e]], __fmul_rn(val, w1));
                sm.v_acc[pos[e]] = __fadd_rn(sm.v_acc[pos[e]], __fmul_rn(__fmul_rn(val, val), w2));
            }
        }
        for (int j = t + WIN_EPT * WIN_THREADS; j < kcnt; j += WIN_THREADS) {   // rows longer than WIN_EPT entries per thread
            const int p = (int)I_r[j] - s0;
            if (p >= 0 && p < len) {
                const float val = __uint_as_float((uint32_t)V_r[j] << 16);
                sm.m_acc[p] = __fadd_rn(sm.m_acc[p], __fmul_rn(val, w1));
                sm.v_acc[p] = __fadd_rn(sm.v_acc[p], __fmul_rn(__fmul_rn(val, val), w2));
            }
        }
        __syncthreads();
    }
    // a position nothing was added to, or only zeros, has v == 0 and m == 0, and its update 0 / (0 + eps) is 0 as well
    const float inv_bc1 = 1.0f / a.bc1, inv_bc2 = 1.0f / a.bc2;
    for (int i = t; i < len; i += WIN_THREADS) {
        const float v = sm.v_acc[i];
        if (v != 0.0f) sm.m_acc[i] = adam_update_fast(sm.m_acc[i], v, inv_bc1, inv_bc2, a.eps);
    }
    __syncthreads();
}

}  // namespace mab
