// Kernel A of the step (micro_adam.py:190-231), one CTA per top-k block, the block held in
// registers from the gradient load to the error-feedback store:
//   a = g + Qinv(e)            dequantise the 4-bit error feedback and add the gradient
//   I[row], V[row]             exact block top-k of |a| (ties to the lower position, ascending)
//   a[I] = 0                   the residual
//   min / max per quant block  as bf16
//   e = Q(a)                   requantise the residual
// The gradient buffer is only read.  HBM traffic per element: the gradient, one nibble in, one
// nibble out, plus the per-block statistics and the k selected (index, value) pairs.
#include "common.cuh"
#include "select.cuh"
#include "fused.cuh"

namespace mab {

constexpr int A_MAX_TENSORS = 512;

template <typename TG> struct GradOctet;
template <> struct GradOctet<float> {
    __device__ __forceinline__ static void load(const float* p, float (&v)[8], bool vec, int n) {
        if (vec) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = (e < n) ? p[e] : 0.0f;
        }
    }
};
template <> struct GradOctet<uint16_t> {
    __device__ __forceinline__ static void load(const uint16_t* p, float (&v)[8], bool vec, int n) {
        if (vec) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
            v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
            v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
            v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
            v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = (e < n) ? bf16_bits_to_f32(p[e]) : 0.0f;
        }
    }
};

// code of element e (0..7) of an octet whose 4 code bytes sit little-endian in `w`:
// byte e/2, even element in the high nibble
__device__ __forceinline__ uint32_t octet_code(uint32_t w, int e) { return (w >> (8 * (e >> 1) + ((e & 1) ? 0 : 4))) & 0xFu; }

template <typename TG>
__global__ void __launch_bounds__(SEL_THREADS, 1)
ef_topk_quant_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int qbs, int lanes_per_qb) {
    __shared__ SelectSmem sm;
    __shared__ int s_first[A_MAX_TENSORS + 1];
    for (int i = threadIdx.x; i < n_tensors; i += SEL_THREADS) s_first[i] = tensors[i].first_unit_a;
    if (threadIdx.x == 0) s_first[n_tensors] = total_units;
    __syncthreads();

    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        const int ti = find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const int dbs = T.d_block_size, nfull = T.topk_full_blocks_count;
        const int64_t base = (int64_t)blk * dbs;
        const int n = (int)min((int64_t)dbs, T.d - base);
        const int k = (blk < nfull) ? T.k_block_size_many : T.k_block_size_few;
        const TG* g = reinterpret_cast<const TG*>(T.grad) + base;
        const uint8_t* ef_in = T.error + (base >> 1);
        const bool vec_g = aligned16(g), vec_e = (reinterpret_cast<uintptr_t>(ef_in) & 3) == 0;

        // ---- a = g + Qinv(e), rounded to the gradient's element type ------------------------
        float a[SEL_OCTETS][8];
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            const int o = j * SEL_THREADS + (int)threadIdx.x;
            const int cnt = max(0, min(8, n - o * 8));
            if (cnt > 0) {
                const int64_t qb = (base + (int64_t)o * 8) / qbs;
                const QParams q = qparams(T.min_vals[qb], T.max_vals[qb]);
                uint32_t w = 0;
                if (vec_e && cnt == 8) w = __ldg(reinterpret_cast<const uint32_t*>(ef_in + o * 4));
                else {
#pragma unroll
                    for (int b = 0; b < 4; ++b) if (2 * b < cnt) w |= (uint32_t)ef_in[o * 4 + b] << (8 * b);
                }
                float gv[8];
                GradOctet<TG>::load(g + o * 8, gv, vec_g && cnt == 8, cnt);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float x = qinv(octet_code(w, e), q);
                    a[j][e] = (e < cnt) ? Elem<TG>::round(__fadd_rn(gv[e], __fmul_rn(1.0f, x))) : 0.0f;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[j][e] = 0.0f;
            }
        }

        // ---- exact top-k ---------------------------------------------------------------------
        int need;
        const int T_key = block_kth_key_bisect(a, k, sm, need);
        publish_masks(a, T_key, sm);
        resolve_selection(need, sm);
        const int64_t row_off = (int64_t)T.ring_index * T.k + (int64_t)blk * T.k_block_size_many;
        emit_indices(sm, T.I + row_off);

        // ---- V[row] = bf16(a[I]); a[I] = 0; statistics; e = Q(a) ---------------------------------
        uint16_t* v_out = T.V + row_off;
        uint8_t* ef_out = T.error + (base >> 1);
        const uint8_t* sel_bytes = reinterpret_cast<const uint8_t*>(sm.sel_bm);
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            const int o = j * SEL_THREADS + (int)threadIdx.x;
            const int cnt = max(0, min(8, n - o * 8));
            const uint32_t sel = sel_bytes[o];
            if (sel) {
                const int word = o >> 2;
                int p = sm.sel_before[word] + __popc(sm.sel_bm[word] & ((1u << (8 * (o & 3))) - 1u));
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (sel & (1u << e)) { v_out[p++] = f32_to_bf16_bits_rne(a[j][e]); a[j][e] = 0.0f; }
            }
            float lo = INFINITY, hi = -INFINITY;
#pragma unroll
            for (int e = 0; e < 8; ++e) if (e < cnt) { lo = fminf(lo, a[j][e]); hi = fmaxf(hi, a[j][e]); }
            for (int off = 1; off < lanes_per_qb; off <<= 1) {
                lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
                hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
            }
            if (cnt > 0) {
                const int64_t ge = base + (int64_t)o * 8;
                const int64_t qb = ge / qbs;
                const uint16_t mn_b = f32_to_bf16_bits_rne(lo), mx_b = f32_to_bf16_bits_rne(hi);
                if (ge % qbs == 0) { T.min_vals[qb] = mn_b; T.max_vals[qb] = mx_b; }
                const QParams q2 = qparams(mn_b, mx_b);
                uint32_t w = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t c = (e < cnt) ? qcode_exact(a[j][e], q2) : 0u;
                    w |= c << (8 * (e >> 1) + ((e & 1) ? 0 : 4));
                }
                if (vec_e && cnt == 8) *reinterpret_cast<uint32_t*>(ef_out + o * 4) = w;
                else {
#pragma unroll
                    for (int b = 0; b < 4; ++b) if (2 * b < cnt) ef_out[o * 4 + b] = (uint8_t)(w >> (8 * b));
                }
            }
        }
        __syncthreads();   // selection scratch is reused by the next unit
    }
}

int units_a_of(const mab_tensor& t) { return t.topk_full_blocks_count + (t.k_block_size_few > 0 ? 1 : 0); }

int launch_ef_topk_quant(const mab_tensor* dev_tensors, int n_tensors, int total_units, int grad_dtype,
                         int qbs, cudaStream_t s) {
    const int grid = (int)std::min<int64_t>(total_units, (int64_t)device_sm_count());
    const int lanes = qbs / 8;
    if (grad_dtype == MAB_F32)
        ef_topk_quant_kernel<float><<<grid, SEL_THREADS, 0, s>>>(dev_tensors, n_tensors, total_units, qbs, lanes);
    else
        ef_topk_quant_kernel<uint16_t><<<grid, SEL_THREADS, 0, s>>>(dev_tensors, n_tensors, total_units, qbs, lanes);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "ef_topk_quant_kernel launch");
    return MAB_OK;
}

}  // namespace mab
