// Sparse window -> dense Adam-style update for one sub-range of a top-k block, in shared memory.
//
// A top-k block is cut into sub-ranges of at most WIN_SR elements (a multiple of 128, so that
// every sub-range starts on a quantisation-block boundary for quant_block_size <= 128).  For one
// sub-range the CTA
//   1. zeroes two float accumulators (first and second moment) of WIN_SR elements,
//   2. loads the window entries of the block (rows r < rows, the block's slice of I / V),
//      keeps those whose position falls in the sub-range in "slots",
//   3. adds them row after row with a barrier between rows (positions are unique inside a
//      row, so a row needs no atomics, and the fixed row order makes the float sums
//      reproducible bit for bit on any grid and any GPU count),
//   4. turns (m, v) into the update u at the touched positions only (the expensive divide and
//      square root run on ~10 % of the elements), leaving u = 0 elsewhere in the first array.
// The caller then streams over the sub-range reading u from shared memory.
#pragma once
#include "common.cuh"

namespace mab {

constexpr int WIN_SR = 7296;          // 57 * 128 elements per sub-range
constexpr int WIN_THREADS = 512;
constexpr int WIN_SLOTS = 3072;       // window entries examined per batch
constexpr int WIN_SLOTS_PER_THREAD = WIN_SLOTS / WIN_THREADS;
constexpr int WIN_SMEM_BYTES = 2 * WIN_SR * 4 + WIN_SLOTS * 4;
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
    uint32_t* slots;                  // (bf16 value bits << 16) | (local position), or 0xFFFFFFFF
    __device__ explicit WindowSmem(unsigned char* base)
        : m_acc(reinterpret_cast<float*>(base)), v_acc(m_acc + WIN_SR),
          slots(reinterpret_cast<uint32_t*>(v_acc + WIN_SR)) {}
};

__device__ __forceinline__ float adam_update_value(float m, float v, const WindowArgs& a) {
    const float m_hat = __fdiv_rn(m, a.bc1);
    const float v_hat = __fdiv_rn(v, a.bc2);
    return __fdiv_rn(m_hat, __fadd_rn(__fsqrt_rn(v_hat), a.eps));
}

// I_blk / V_blk point at the block's slice of row 0; row_pitch = k; kcnt entries per row;
// sub-range = block positions [s0, s0 + len).  Leaves u in sm.m_acc[0..len).  Ends with a barrier.
__device__ __forceinline__ void window_to_update(const int16_t* __restrict__ I_blk, const uint16_t* __restrict__ V_blk,
                                                 int64_t row_pitch, int kcnt, int s0, int len,
                                                 const WindowArgs& a, WindowSmem& sm) {
    const int t = threadIdx.x;
    for (int i = t; i < WIN_SR; i += WIN_THREADS) { sm.m_acc[i] = 0.0f; sm.v_acc[i] = 0.0f; }
    const int64_t total = (int64_t)a.rows * kcnt;            // flattened (row, j) entries
    const int nbatch = (int)((total + WIN_SLOTS - 1) / WIN_SLOTS);

    for (int pass = 0; pass < 2; ++pass) {                   // 0: accumulate, 1: finalize
        for (int bi = 0; bi < nbatch; ++bi) {
            const int64_t q0 = (int64_t)bi * WIN_SLOTS;
            const int nq = (int)min((int64_t)WIN_SLOTS, total - q0);
            if (pass == 0 || nbatch > 1) {
                __syncthreads();                             // slots free (and, first time, zeroing done)
#pragma unroll
                for (int s = 0; s < WIN_SLOTS_PER_THREAD; ++s) {
                    const int q = s * WIN_THREADS + t;
                    uint32_t slot = 0xFFFFFFFFu;
                    if (q < nq) {
                        const int64_t g = q0 + q;
                        const int r = (int)(g / kcnt), j = (int)(g - (int64_t)r * kcnt);
                        const int pos = (int)I_blk[(int64_t)r * row_pitch + j] - s0;
                        if (pos >= 0 && pos < len)
                            slot = ((uint32_t)V_blk[(int64_t)r * row_pitch + j] << 16) | (uint32_t)pos;
                    }
                    sm.slots[q] = slot;
                }
                __syncthreads();
            }
            if (pass == 0) {
                const int r_lo = (int)(q0 / kcnt), r_hi = (int)((q0 + nq - 1) / kcnt);
                for (int r = r_lo; r <= r_hi; ++r) {
                    const int lo = (int)max((int64_t)r * kcnt - q0, (int64_t)0);
                    const int hi = (int)min((int64_t)(r + 1) * kcnt - q0, (int64_t)nq);
                    const float w1 = a.w1[r], w2 = a.w2[r];
                    for (int q = lo + t; q < hi; q += WIN_THREADS) {
                        const uint32_t slot = sm.slots[q];
                        if (slot != 0xFFFFFFFFu) {
                            const int pos = slot & 0xFFFF;
                            const float val = __uint_as_float(slot & 0xFFFF0000u);
                            sm.m_acc[pos] = __fadd_rn(sm.m_acc[pos], __fmul_rn(val, w1));
                            sm.v_acc[pos] = __fadd_rn(sm.v_acc[pos], __fmul_rn(__fmul_rn(val, val), w2));
                        }
                    }
                    __syncthreads();
                }
            } else {
                float u[WIN_SLOTS_PER_THREAD];
#pragma unroll
                for (int s = 0; s < WIN_SLOTS_PER_THREAD; ++s) {
                    const int q = s * WIN_THREADS + t;
                    u[s] = 0.0f;
                    const uint32_t slot = (q < nq) ? sm.slots[q] : 0xFFFFFFFFu;
                    if (slot != 0xFFFFFFFFu) {
                        const int pos = slot & 0xFFFF;
                        const float v = sm.v_acc[pos];
                        u[s] = (v < 0.0f) ? sm.m_acc[pos] : adam_update_value(sm.m_acc[pos], v, a);
                    }
                }
                __syncthreads();
#pragma unroll
                for (int s = 0; s < WIN_SLOTS_PER_THREAD; ++s) {
                    const int q = s * WIN_THREADS + t;
                    const uint32_t slot = (q < nq) ? sm.slots[q] : 0xFFFFFFFFu;
                    if (slot != 0xFFFFFFFFu) {
                        const int pos = slot & 0xFFFF;
                        sm.m_acc[pos] = u[s];       // duplicates of a position write the same value
                        sm.v_acc[pos] = -1.0f;      // marks "already an update" for later batches
                    }
                }
            }
        }
    }
    __syncthreads();
}

}  // namespace mab
