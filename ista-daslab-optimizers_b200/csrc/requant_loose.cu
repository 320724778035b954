// Second half of kernel A's work when quantisation blocks ignore the borders of the top-k blocks
// (micro_adam.py:217-231 for any quant_block_size): ef_topk_quant_kernel<.., true> left the residual in the
// gradient buffer and the extremes of every quantisation block, merged over the tiles that touch it, in two
// scratch arrays.  This kernel rounds those extremes to bf16 (min_vals / max_vals) and writes the 4-bit codes
// e = Q(residual).  HBM traffic per element: the residual once, one nibble out.
#include "common.cuh"
#include "codec_fast.cuh"
#include "fused.cuh"

namespace mab {

constexpr int RQ_THREADS = 256;

// A whole octet of the residual, 16-byte aligned: loaded as raw words (so that several octets in flight cost few
// registers), turned into floats when it is worked on.
template <typename TG> struct ResidualOctet;
template <> struct ResidualOctet<float> {
    struct Raw { float4 lo, hi; };
    __device__ __forceinline__ static Raw load(const float* p) {
        Raw r;
        r.lo = __ldg(reinterpret_cast<const float4*>(p)); r.hi = __ldg(reinterpret_cast<const float4*>(p) + 1);
        return r;
    }
    __device__ __forceinline__ static void unpack(const Raw& r, float (&v)[8]) {
        v[0] = r.lo.x; v[1] = r.lo.y; v[2] = r.lo.z; v[3] = r.lo.w; v[4] = r.hi.x; v[5] = r.hi.y; v[6] = r.hi.z; v[7] = r.hi.w;
    }
};
template <> struct ResidualOctet<uint16_t> {
    struct Raw { uint4 w; };
    __device__ __forceinline__ static Raw load(const uint16_t* p) {
        Raw r;
        r.w = __ldg(reinterpret_cast<const uint4*>(p));
        return r;
    }
    __device__ __forceinline__ static void unpack(const Raw& r, float (&v)[8]) {
        v[0] = __uint_as_float(r.w.x << 16); v[1] = __uint_as_float(r.w.x & 0xFFFF0000u);
        v[2] = __uint_as_float(r.w.y << 16); v[3] = __uint_as_float(r.w.y & 0xFFFF0000u);
        v[4] = __uint_as_float(r.w.z << 16); v[5] = __uint_as_float(r.w.z & 0xFFFF0000u);
        v[6] = __uint_as_float(r.w.w << 16); v[7] = __uint_as_float(r.w.w & 0xFFFF0000u);
    }
};

template <typename TG>
__global__ void __launch_bounds__(RQ_THREADS, 4)
requant_loose_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, LooseArgs la) {
    __shared__ int s_first[WIN_MAX_TENSORS + 1];
    for (int i = threadIdx.x; i < n_tensors; i += RQ_THREADS) s_first[i] = tensors[i].first_unit_a;
    if (threadIdx.x == 0) s_first[n_tensors] = total_units;
    __syncthreads();
    const bool big = la.qbs >= 32768;
    int ti = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        if (unit >= s_first[ti + 1] || unit < s_first[ti]) ti = find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const int64_t base = (int64_t)blk * T.d_block_size;
        const int n = (int)min((int64_t)T.d_block_size, T.d - base);
        const TG* r_in = reinterpret_cast<const TG*>(T.grad) + base;
        uint8_t* ef_out = T.error + (base >> 1);
        const bool vec_r = aligned16(r_in), vec_e = (reinterpret_cast<uintptr_t>(ef_out) & 3) == 0;
        const int64_t qb0 = base / la.qbs;
        const int rem0 = (int)(base - qb0 * la.qbs);
        const uint32_t* st_min = la.st_min + la.qb_first[ti] + qb0;
        const uint32_t* st_max = la.st_max + la.qb_first[ti] + qb0;
        int cached = -1;                                 // the block whose constants the thread holds
        uint16_t mn_b = 0, mx_b = 0;
        QParams q = {0.0f, 0.0f};
        DivConsts dc = {};
        bool fast = false;                               // the block's step is in the range of the division-free encoder
        // constants of the block an octet lies in (kept while consecutive octets stay in it); the octet that opens
        // a block writes its statistics: a tile that starts inside a block leaves them to the tile that holds
        // the block's first element
        auto enter_block = [&](int o) {
            const int r = rem0 + o * 8;
            const int qi = loose_block(r, la.qbs, big);
            if (qi != cached) {
                cached = qi;
                mn_b = f32_to_bf16_bits_rne(ord_value(__ldg(st_min + qi)));
                mx_b = f32_to_bf16_bits_rne(ord_value(__ldg(st_max + qi)));
                q = qparams(mn_b, mx_b);
                fast = q.u >= CODEC_U_MIN && q.u <= CODEC_U_MAX;
                dc = div_consts(q);
            }
            if (r - qi * la.qbs == 0) { T.min_vals[qb0 + qi] = mn_b; T.max_vals[qb0 + qi] = mx_b; }
        };
        const int n_whole = n >> 3;                      // octets without padding
        if (vec_r && vec_e) {
            constexpr int U = 4;                         // octets in flight per thread
            for (int o0 = threadIdx.x; o0 < n_whole; o0 += U * RQ_THREADS) {
                typename ResidualOctet<TG>::Raw raw[U];
#pragma unroll
                for (int i = 0; i < U; ++i) {
                    const int o = o0 + i * RQ_THREADS;
                    if (o < n_whole) raw[i] = ResidualOctet<TG>::load(r_in + o * 8);
                }
#pragma unroll
                for (int i = 0; i < U; ++i) {
                    const int o = o0 + i * RQ_THREADS;
                    if (o < n_whole) {
                        enter_block(o);
                        float a[8];
                        ResidualOctet<TG>::unpack(raw[i], a);
                        // fp32 residuals can lie outside the bf16-rounded statistics (clamp); bf16 ones cannot
                        reinterpret_cast<uint32_t*>(ef_out)[o] = fast ? encode_octet_div_f32<sizeof(TG) == 4>(a, dc)
                                                                      : encode_octet_exact(a, q, 8);
                    }
                }
            }
        } else {
            for (int o = threadIdx.x; o < n_whole; o += RQ_THREADS) {
                float a[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = Elem<TG>::load(r_in, o * 8 + e);
                enter_block(o);
                const uint32_t w = fast ? encode_octet_div_f32<sizeof(TG) == 4>(a, dc) : encode_octet_exact(a, q, 8);
#pragma unroll
                for (int b = 0; b < 4; ++b) ef_out[o * 4 + b] = (uint8_t)(w >> (8 * b));
            }
        }
        if ((n & 7) != 0 && threadIdx.x == RQ_THREADS - 1) {     // the tensor's last, short octet
            const int o = n_whole, cnt = n & 7;
            float a[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = (e < cnt) ? Elem<TG>::load(r_in, o * 8 + e) : 0.0f;
            enter_block(o);
            const uint32_t w = encode_octet_exact(a, q, cnt);
#pragma unroll
            for (int b = 0; b < 4; ++b) if (2 * b < cnt) ef_out[o * 4 + b] = (uint8_t)(w >> (8 * b));
        }
    }
}

int launch_requant_loose(const mab_tensor* dev_tensors, int n_tensors, int total_units, int grad_dtype,
                         const LooseArgs& la, cudaStream_t s) {
    const int grid = (int)std::min<int64_t>(total_units, (int64_t)device_sm_count() * 8);
    if (grad_dtype == MAB_F32) requant_loose_kernel<float><<<grid, RQ_THREADS, 0, s>>>(dev_tensors, n_tensors, total_units, la);
    else requant_loose_kernel<uint16_t><<<grid, RQ_THREADS, 0, s>>>(dev_tensors, n_tensors, total_units, la);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "requant_loose_kernel launch");
}

}  // namespace mab
