// The logging probes of the step that only need the step's inputs and its final state
// (micro_adam.py:155-156, 320-324): sum g^2 over the gradients and sum Qinv(e)^2 over the error feedback the
// step leaves behind, for all tensors of a fused call in one launch.  (The probes of the update itself - sum u^2,
// the zeros of u, the quantisation error of alpha == -2 - are taken inside kernel B, where those values exist.)
#include "common.cuh"
#include "fused.cuh"

namespace mab {

constexpr int PR_THREADS = 256;

template <typename TG>
__device__ __forceinline__ void probe_tile(const mab_tensor& T, int blk, int64_t qbs, int which, float& sum_g, float& sum_e) {
    const int dbs = T.d_block_size;
    const int64_t base = (int64_t)blk * dbs;
    const int n = (int)min((int64_t)dbs, T.d - base);
    const TG* g = reinterpret_cast<const TG*>(T.grad) + base;
    const uint8_t* ef = T.error + (base >> 1);                      // dbs is even whenever a tensor has more than one block
    for (int o = threadIdx.x; o * 8 < n; o += PR_THREADS) {
        const int cnt = min(8, n - o * 8);
        if (which & PROBE_G)
            for (int e = 0; e < cnt; ++e) {
                const float gv = Elem<TG>::load(g, o * 8 + e);
                sum_g = fmaf(gv, gv, sum_g);
            }
        if (which & PROBE_E) {
            const int64_t qb = (base + (int64_t)o * 8) / qbs;        // an octet never straddles a quantisation block (qbs is a multiple of 8)
            const QParams q = qparams(T.min_vals[qb], T.max_vals[qb]);
            for (int e = 0; e < cnt; ++e) {
                const uint32_t byte = ef[(o * 8 + e) >> 1];
                const uint32_t code = (e & 1) ? (byte & 0xFu) : (byte >> 4);
                const float x = Elem<TG>::round(__fadd_rn(0.0f, qinv(code, q)));   // what asymm_block_quant_inv leaves in a zeroed gradient buffer
                sum_e = fmaf(x, x, sum_e);
            }
        }
    }
}

__global__ void __launch_bounds__(PR_THREADS)
probe_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int64_t qbs, int which, double* __restrict__ out) {
    __shared__ int s_first[WIN_MAX_TENSORS + 1];
    __shared__ float s_part[2][PR_THREADS / 32];
    for (int i = threadIdx.x; i < n_tensors; i += PR_THREADS) s_first[i] = tensors[i].first_unit_a;
    if (threadIdx.x == 0) s_first[n_tensors] = total_units;
    __syncthreads();
    double tot_g = 0.0, tot_e = 0.0;                                 // thread 0: this CTA's totals
    int ti = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        if (unit >= s_first[ti + 1]) ti = find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        float sum_g = 0.0f, sum_e = 0.0f;                            // per tile in fp32 (at most 128 terms per thread), across tiles in fp64
        if (T.grad_dtype == MAB_F32) probe_tile<float>(T, unit - s_first[ti], qbs, which, sum_g, sum_e);
        else probe_tile<uint16_t>(T, unit - s_first[ti], qbs, which, sum_g, sum_e);
#pragma unroll
        for (int o = 16; o; o >>= 1) { sum_g += __shfl_xor_sync(0xffffffffu, sum_g, o); sum_e += __shfl_xor_sync(0xffffffffu, sum_e, o); }
        if (lane_id() == 0) { s_part[0][warp_id()] = sum_g; s_part[1][warp_id()] = sum_e; }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int w = 0; w < PR_THREADS / 32; ++w) { tot_g += (double)s_part[0][w]; tot_e += (double)s_part[1][w]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (which & PROBE_G) atomicAdd(&out[MAB_PROBE_NORM_G], tot_g);
        if (which & PROBE_E) atomicAdd(&out[MAB_PROBE_NORM_E], tot_e);
    }
}

int launch_probe(const mab_tensor* dev_tensors, int n_tensors, int total_units, int qbs, double* out, cudaStream_t s, int which) {
    const int grid = (int)std::min<int64_t>(total_units, (int64_t)device_sm_count() * 8);
    probe_kernel<<<grid, PR_THREADS, 0, s>>>(dev_tensors, n_tensors, total_units, (int64_t)qbs, which, out);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "probe_kernel launch");
}

}  // namespace mab
