// Declarations shared by the two fused kernels and the host-side step driver.
#pragma once
#include "common.cuh"
#include "window.cuh"

namespace mab {

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Elements between consecutive rows of a tensor's I and V.
__host__ __device__ __forceinline__ int64_t row_pitch_of(const mab_tensor& t) { return t.row_pitch > 0 ? (int64_t)t.row_pitch : t.k; }

// Index of the tensor whose unit range contains `unit`: largest i with first[i] <= unit.
// first[0..n] is ascending with first[n] = total units; tensors without units repeat a value.
__device__ __forceinline__ int find_tensor(const int* first, int n, int unit) {
    int lo = 0, hi = n;                      // invariant: first[lo] <= unit < first[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (first[mid] <= unit) lo = mid; else hi = mid;
    }
    return lo;
}

// window_adam.cu
int fill_window_args(WindowArgs& a, int64_t steps, int m, double beta1, double beta2, double eps, float alpha, int qbs);
int launch_window_step(const mab_tensor* dev_tensors, int n_tensors, int units_tile, int units_wide, int max_k, int max_dbs,
                       int param_dtype, const WindowArgs& a, cudaStream_t s);
int units_b_of(const mab_tensor& t);
int launch_wait_selftest(int probe_limit, cudaStream_t s);

// probe.cu: adds sum g^2 (which & PROBE_G) and sum Qinv(e)^2 (which & PROBE_E) of the tensors to
// out[MAB_PROBE_NORM_G] / out[MAB_PROBE_NORM_E]
enum { PROBE_G = 1, PROBE_E = 2 };
int launch_probe(const mab_tensor* dev_tensors, int n_tensors, int total_units, int qbs, double* out, cudaStream_t s,
                 int which = PROBE_G | PROBE_E);

// Quantisation blocks of any size (a multiple of 8 elements), which ignore the borders of the top-k blocks
// (micro_adam.py:217-231): kernel A then leaves the residual in the gradient buffer and merges each block's
// extremes into two scratch arrays; requant_loose.cu turns them into statistics and codes.
struct LooseArgs {
    int qbs;                       // quant_block_size
    uint32_t* st_min;              // order-preserving key of the minimum per quantisation block (initialised to 0xFFFFFFFF)
    uint32_t* st_max;              // ... of the maximum (initialised to 0)
    const int64_t* qb_first;       // first scratch entry of every tensor of the call
};

constexpr int LOOSE_MAX_QB = 32768 / 64 + 2;        // quantisation blocks (>= 64 elements) a tile of at most 32768 elements can touch

// Monotone map float -> uint32 (negative values below positive ones, -0 below +0) and back.
__device__ __forceinline__ uint32_t ord_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);
}
__device__ __forceinline__ float ord_value(uint32_t k) {
    return __uint_as_float(k ^ ((k & 0x80000000u) ? 0x80000000u : 0xFFFFFFFFu));
}

// Quantisation block (relative to the tile's first) of the octet that starts `r` elements after that block's start;
// `big`: the block is at least as long as the longest tile, so the answer is 0 or 1.
__device__ __forceinline__ int loose_block(int r, int qbs, bool big) {
    return big ? (r >= qbs ? 1 : 0) : (int)((unsigned)r / (unsigned)qbs);
}

// ef_topk_quant.cu
int launch_ef_topk_quant(const mab_tensor* dev_tensors, int n_tensors, int total_units, int grad_dtype,
                         int qbs, int max_dbs, cudaStream_t s, const LooseArgs* loose = nullptr);
int units_a_of(const mab_tensor& t);

// requant_loose.cu: statistics (bf16) and codes of the residual kernel A left in the gradient buffers
int launch_requant_loose(const mab_tensor* dev_tensors, int n_tensors, int total_units, int grad_dtype,
                         const LooseArgs& la, cudaStream_t s);

// ef_topk_quant_bf16.cu: returns 1 (without launching) when two CTAs of its shared memory do not fit an SM
int launch_ef_topk_quant_bf16(const mab_tensor* dev_tensors, int n_tensors, int total_units, int qbs, int max_dbs, cudaStream_t s,
                              const LooseArgs* loose = nullptr);

// Each kernel file keeps its own "a bounded wait gave up" flag (no relocatable device code): these read
// it into *out and optionally clear it.
int copy_timeout_f32(int* out, bool clear);      // ef_topk_quant.cu
int copy_timeout_bf16(int* out, bool clear);     // ef_topk_quant_bf16.cu
int copy_timeout_window(int* out, bool clear);   // window_adam.cu

}  // namespace mab
