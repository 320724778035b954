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
#include "select_fast.cuh"
#include "codec_fast.cuh"
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

template <typename TG>
__global__ void __launch_bounds__(SEL_THREADS, 1)
ef_topk_quant_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int qshift) {
    __shared__ SelectSmem sm;
    __shared__ FastSelSmem fs;
    __shared__ int s_first[A_MAX_TENSORS + 1];
    int guess = 0;                                  // lower bound found for the previous tile, as key bits
    for (int i = threadIdx.x; i < n_tensors; i += SEL_THREADS) s_first[i] = tensors[i].first_unit_a;
    if (threadIdx.x == 0) s_first[n_tensors] = total_units;
    __syncthreads();
    const int oshift = qshift - 3;                  // octets per quantisation block, as a shift
    const int lanes_per_qb = 1 << oshift;

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
        const uint16_t* mn_in = T.min_vals + (base >> qshift);     // statistics of the tile's first block
        const uint16_t* mx_in = T.max_vals + (base >> qshift);
        const bool vec_g = aligned16(g), vec_e = (reinterpret_cast<uintptr_t>(ef_in) & 3) == 0;

        // ---- a = g + Qinv(e), rounded to the gradient's element type ------------------------
        float a[SEL_OCTETS][8];
        float omax[SEL_OCTETS];
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            const int o = j * SEL_THREADS + (int)threadIdx.x;
            const int cnt = n - o * 8;               // >= 8: full octet, 1..7: the tensor's last, <= 0: none
            omax[j] = 0.0f;
            if (cnt >= 8) {
                const QParams q = qparams(mn_in[o >> oshift], mx_in[o >> oshift]);
                uint32_t w;
                if (vec_e) w = __ldg(reinterpret_cast<const uint32_t*>(ef_in + o * 4));
                else w = ef_in[o * 4] | ((uint32_t)ef_in[o * 4 + 1] << 8) | ((uint32_t)ef_in[o * 4 + 2] << 16) | ((uint32_t)ef_in[o * 4 + 3] << 24);
                float gv[8], x[8];
                GradOctet<TG>::load(g + o * 8, gv, vec_g, 8);
                decode_octet(w, q, x);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    a[j][e] = Elem<TG>::round(__fadd_rn(gv[e], x[e]));
                    omax[j] = fmaxf(omax[j], fabsf(a[j][e]));
                }
            } else if (cnt > 0) {
                const QParams q = qparams(mn_in[o >> oshift], mx_in[o >> oshift]);
                uint32_t w = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) if (2 * b < cnt) w |= (uint32_t)ef_in[o * 4 + b] << (8 * b);
                float gv[8], x[8];
                GradOctet<TG>::load(g + o * 8, gv, false, cnt);
                decode_octet_exact(w, q, x);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    a[j][e] = (e < cnt) ? Elem<TG>::round(__fadd_rn(gv[e], x[e])) : 0.0f;
                    omax[j] = fmaxf(omax[j], fabsf(a[j][e]));
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[j][e] = 0.0f;
            }
        }

        // ---- exact top-k ---------------------------------------------------------------------
        const int64_t row_off = (int64_t)T.ring_index * T.k + (int64_t)blk * T.k_block_size_many;
        uint16_t* v_out = T.V + row_off;
        int n_cand = 0;
        const bool fast = fast_select(a, omax, n, k, guess, sm, fs, n_cand);
        if (!fast) {
            int need;
            const int T_key = block_kth_key_bisect(a, k, sm, need);
            publish_masks(a, T_key, sm);
            resolve_selection(need, sm);
        }
        emit_indices(sm, T.I + row_off);
        if (fast) {
            // V[row] = bf16(a[I]) from the candidate list, in the order the bitmap defines
            for (int i = threadIdx.x; i < n_cand; i += SEL_THREADS) {
                const uint32_t pos = fs.cand_pos[i];
                if (pos & 0x8000u) {
                    const uint32_t q = pos & 0x7FFFu, w = q >> 5;
                    v_out[sm.sel_before[w] + __popc(sm.sel_bm[w] & ((1u << (q & 31)) - 1u))] = f32_to_bf16_bits_rne(fs.cand_val[i]);
                }
            }
        }

        // ---- a[I] = 0 (slow path: also V[row]); statistics; e = Q(a) ------------------------------
        uint8_t* ef_out = T.error + (base >> 1);
        uint16_t* mn_out = T.min_vals + (base >> qshift);
        uint16_t* mx_out = T.max_vals + (base >> qshift);
        const uint8_t* sel_bytes = reinterpret_cast<const uint8_t*>(sm.sel_bm);
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            const int o = j * SEL_THREADS + (int)threadIdx.x;
            const int cnt = n - o * 8;
            const uint32_t sel = sel_bytes[o];
            if (fast) {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[j][e] = (sel & (1u << e)) ? 0.0f : a[j][e];
            } else if (sel) {
                const int word = o >> 2;
                int p = sm.sel_before[word] + __popc(sm.sel_bm[word] & ((1u << (8 * (o & 3))) - 1u));
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (sel & (1u << e)) { v_out[p++] = f32_to_bf16_bits_rne(a[j][e]); a[j][e] = 0.0f; }
            }
            float lo = INFINITY, hi = -INFINITY;
            if (cnt >= 8) {
#pragma unroll
                for (int e = 0; e < 8; ++e) { lo = fminf(lo, a[j][e]); hi = fmaxf(hi, a[j][e]); }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) if (e < cnt) { lo = fminf(lo, a[j][e]); hi = fmaxf(hi, a[j][e]); }
            }
            for (int off = 1; off < lanes_per_qb; off <<= 1) {
                lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
                hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
            }
            if (cnt > 0) {
                const uint16_t mn_b = f32_to_bf16_bits_rne(lo), mx_b = f32_to_bf16_bits_rne(hi);
                if ((o & (lanes_per_qb - 1)) == 0) { mn_out[o >> oshift] = mn_b; mx_out[o >> oshift] = mx_b; }
                const QParams q2 = qparams(mn_b, mx_b);
                if (cnt >= 8) {
                    const uint32_t w = encode_octet(a[j], q2);
                    if (vec_e) *reinterpret_cast<uint32_t*>(ef_out + o * 4) = w;
                    else {
#pragma unroll
                        for (int b = 0; b < 4; ++b) ef_out[o * 4 + b] = (uint8_t)(w >> (8 * b));
                    }
                } else {
                    const uint32_t w = encode_octet_exact(a[j], q2, cnt);
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
    int qshift = 0;
    while ((1 << qshift) < qbs) ++qshift;
    if (grad_dtype == MAB_F32)
        ef_topk_quant_kernel<float><<<grid, SEL_THREADS, 0, s>>>(dev_tensors, n_tensors, total_units, qshift);
    else
        ef_topk_quant_kernel<uint16_t><<<grid, SEL_THREADS, 0, s>>>(dev_tensors, n_tensors, total_units, qshift);
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "ef_topk_quant_kernel launch");
    return MAB_OK;
}

}  // namespace mab

#ifdef MAB_STATS
extern "C" int mab_debug_stats(unsigned long long* out16, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out16, mab::g_stats, sizeof(mab::g_stats));
    if (e == cudaSuccess && reset) { unsigned long long z[16] = {0}; e = cudaMemcpyToSymbol(mab::g_stats, z, sizeof(z)); }
    return e == cudaSuccess ? 0 : -3;
}
#endif
