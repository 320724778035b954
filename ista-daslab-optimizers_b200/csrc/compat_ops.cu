// One kernel per native call of the reference's MicroAdam step (micro_adam.py:190-231), for
// any quantisation block size and any tensor size.  The fused kernels cover the common
// geometries faster; these are the general path and the operator-level drop-in surface.
#include "common.cuh"
#include "select.cuh"
#include "select_fast.cuh"
#include "codec_fast.cuh"

namespace mab {

constexpr int EW_THREADS = 256;
constexpr int EW_CHUNK = 16;   // elements per thread and step: 8 bytes of codes

// Walks EW_CHUNK consecutive elements starting at i0 and keeps the decode constants of the
// quantisation block the walk is in: one integer division per chunk instead of one per element.
struct BlockWalker {
    int64_t b, rem, qbs;
    const uint16_t* mn; const uint16_t* mx;
    QParams q;
    __device__ BlockWalker(int64_t i0, int64_t qbs_, const uint16_t* mn_, const uint16_t* mx_)
        : b(i0 / qbs_), rem(i0 % qbs_), qbs(qbs_), mn(mn_), mx(mx_) { q = qparams(mn[b], mx[b]); }
    __device__ void next() { if (++rem == qbs) { rem = 0; ++b; q = qparams(mn[b], mx[b]); } }
};

template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
quant_inv_kernel(int64_t d, int64_t qbs, const uint8_t* __restrict__ error, const uint16_t* __restrict__ mn,
                 const uint16_t* __restrict__ mx, T* __restrict__ x, float alpha) {
    const int64_t nchunks = (d + EW_CHUNK - 1) / EW_CHUNK;
    for (int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; c < nchunks; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = c * EW_CHUNK;
        const int n = (int)min((int64_t)EW_CHUNK, d - i0);
        BlockWalker w(i0, qbs, mn, mx);
        for (int e = 0; e < n; ++e) {
            const int64_t i = i0 + e;
            const uint32_t byte = error[i >> 1];
            const uint32_t code = (e & 1) ? (byte & 0xFu) : (byte >> 4);
            const float t = __fmul_rn(alpha, qinv(code, w.q));
            Elem<T>::store(x, i, __fadd_rn(Elem<T>::load(x, i), t));
            if (e + 1 < n) w.next();
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
quant_kernel(int64_t d, int64_t qbs, uint8_t* __restrict__ error, const uint16_t* __restrict__ mn,
             const uint16_t* __restrict__ mx, const T* __restrict__ x) {
    const int64_t nchunks = (d + EW_CHUNK - 1) / EW_CHUNK;
    for (int64_t c = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; c < nchunks; c += (int64_t)gridDim.x * blockDim.x) {
        const int64_t i0 = c * EW_CHUNK;
        const int n = (int)min((int64_t)EW_CHUNK, d - i0);
        BlockWalker w(i0, qbs, mn, mx);
        uint32_t byte = 0;
        for (int e = 0; e < n; ++e) {
            const uint32_t code = qcode_exact(Elem<T>::load(x, i0 + e), w.q);
            if (e & 1) { error[(i0 + e) >> 1] = (uint8_t)(byte | code); byte = 0; }
            else byte = code << 4;
            if (e + 1 < n) w.next();
        }
        if (n & 1) error[(i0 + n - 1) >> 1] = (uint8_t)byte;   // odd d: low nibble of the last byte is 0
    }
}

// ---- octet-wide forms of the three codec operators ----------------------------------------------------------
//
// One thread per 8 consecutive elements, consecutive lanes on consecutive octets, vector loads and stores.
// Conditions (checked by the callers): d and qbs multiples of 8 (an octet lies in one quantisation block and
// no octet is short), x 16-byte aligned, error 4-byte aligned.  Same arithmetic as the element-wise kernels
// above, so the two forms give the same bits.

template <typename T> struct XOctet;
template <> struct XOctet<float> {
    __device__ __forceinline__ static void load(const float* p, float (&v)[8]) {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    __device__ __forceinline__ static void store(float* p, const float (&v)[8]) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct XOctet<uint16_t> {
    __device__ __forceinline__ static void load(const uint16_t* p, float (&v)[8]) {
        const uint4 a = *reinterpret_cast<const uint4*>(p);
        v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
        v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
        v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
        v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
    }
    __device__ __forceinline__ static void store(uint16_t* p, const float (&v)[8]) {
        uint4 w;
        w.x = pack_bf16x2_rne(v[0], v[1]); w.y = pack_bf16x2_rne(v[2], v[3]);
        w.z = pack_bf16x2_rne(v[4], v[5]); w.w = pack_bf16x2_rne(v[6], v[7]);
        *reinterpret_cast<uint4*>(p) = w;
    }
};

// Quantisation block of octet o: a shift when qbs is a power of two (qshift >= 0), else a division.
__device__ __forceinline__ int64_t octet_block(int64_t o, int64_t qbs, int qshift) {
    return qshift >= 0 ? (o << 3) >> qshift : (o << 3) / qbs;
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
quant_inv_octet_kernel(int64_t n_oct, int64_t qbs, int qshift, const uint8_t* __restrict__ error, const uint16_t* __restrict__ mn,
                       const uint16_t* __restrict__ mx, T* __restrict__ x, float alpha) {
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < n_oct; o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = octet_block(o, qbs, qshift);
        const QParams q = qparams(mn[b], mx[b]);
        float v[8], r[8];
        XOctet<T>::load(x + o * 8, v);
        decode_octet(reinterpret_cast<const uint32_t*>(error)[o], q, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __fadd_rn(v[e], __fmul_rn(alpha, r[e]));
        XOctet<T>::store(x + o * 8, v);
    }
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
quant_octet_kernel(int64_t n_oct, int64_t qbs, int qshift, uint8_t* __restrict__ error, const uint16_t* __restrict__ mn,
                   const uint16_t* __restrict__ mx, const T* __restrict__ x) {
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < n_oct; o += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = octet_block(o, qbs, qshift);
        const QParams q = qparams(mn[b], mx[b]);
        float v[8];
        XOctet<T>::load(x + o * 8, v);
        // the division-free form needs a step in range and quotients that stay far from overflow (the caller's values
        // need not lie between the statistics); everything else takes the defining form
        bool fast = q.u >= CODEC_U_MIN && q.u <= CODEC_U_MAX;
        const DivConsts dc = div_consts(q);
        if (fast) {
            float big = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) big = fmaxf(big, fabsf(__fmul_rn(__fsub_rn(v[e], q.mn), dc.r02.x)));
            fast = big < 64.0f;                      // false for NaN as well
        }
        reinterpret_cast<uint32_t*>(error)[o] = fast ? encode_octet_div_f32<true>(v, dc) : encode_octet_exact(v, q, 8);
    }
}

// Power-of-two qbs in [8, 256]: the qbs / 8 lanes of a block combine their octets' extremes by shuffles.
template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
quant_stats_octet_kernel(int64_t n_oct, int qshift, uint16_t* __restrict__ mn, uint16_t* __restrict__ mx, const T* __restrict__ x) {
    const int lanes = 1 << (qshift - 3);
    const int64_t n_pad = (n_oct + 31) & ~(int64_t)31;           // whole warps take part in the shuffles
    for (int64_t o = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; o < n_pad; o += (int64_t)gridDim.x * blockDim.x) {
        float lo = INFINITY, hi = -INFINITY;
        if (o < n_oct) {
            float v[8];
            XOctet<T>::load(x + o * 8, v);
            octet_min_max(v, lo, hi);
        }
        for (int off = 1; off < lanes; off <<= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
        }
        if (o < n_oct && (o & (lanes - 1)) == 0) {
            const int64_t b = (o << 3) >> qshift;
            mn[b] = f32_to_bf16_bits_rne(lo); mx[b] = f32_to_bf16_bits_rne(hi);
        }
    }
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(EW_THREADS)
copy_values_kernel(int64_t k, int64_t dbs, int64_t kbs, const int16_t* __restrict__ idx, const TI* __restrict__ inp,
                   TO* __restrict__ out, int direction) {
    for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < k; j += (int64_t)gridDim.x * blockDim.x) {
        const int64_t g = (j / kbs) * dbs + (int64_t)idx[j];
        if (direction == MAB_D2K) Elem<TO>::store(out, j, Elem<TI>::load(inp, g));
        else Elem<TO>::store(out, g, Elem<TI>::load(inp, j));
    }
}

template <typename T>
__global__ void __launch_bounds__(EW_THREADS)
zerorize_kernel(T* __restrict__ x, const int16_t* __restrict__ idx, int64_t k, int64_t dbs, int64_t kbs) {
    for (int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; j < k; j += (int64_t)gridDim.x * blockDim.x)
        x[(j / kbs) * dbs + (int64_t)idx[j]] = 0;   // all-zero bits are +0 in both element types
}

// One CTA per quantisation block when blocks are long, one warp per block otherwise.
template <typename T, bool CTA_PER_BLOCK>
__global__ void __launch_bounds__(EW_THREADS)
quant_stats_kernel(int64_t d, int64_t qbs, int64_t nblocks, uint16_t* __restrict__ mn, uint16_t* __restrict__ mx,
                   const T* __restrict__ x) {
    __shared__ float s_lo[EW_THREADS / 32], s_hi[EW_THREADS / 32];
    const int lane = lane_id(), warp = warp_id();
    const int64_t stride = CTA_PER_BLOCK ? gridDim.x : (int64_t)gridDim.x * (EW_THREADS / 32);
    const int64_t first = CTA_PER_BLOCK ? blockIdx.x : (int64_t)blockIdx.x * (EW_THREADS / 32) + warp;
    for (int64_t b = first; b < nblocks; b += stride) {
        const int64_t lo_i = b * qbs, hi_i = min(d, lo_i + qbs);
        float lo = INFINITY, hi = -INFINITY;
        const int step = CTA_PER_BLOCK ? EW_THREADS : 32;
        const int me = CTA_PER_BLOCK ? (int)threadIdx.x : lane;
        for (int64_t i = lo_i + me; i < hi_i; i += step) {
            const float v = Elem<T>::load(x, i);
            lo = fminf(lo, v); hi = fmaxf(hi, v);
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        if (CTA_PER_BLOCK) {
            if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; }
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < EW_THREADS / 32; ++w) { lo = fminf(lo, s_lo[w]); hi = fmaxf(hi, s_hi[w]); }
                mn[b] = f32_to_bf16_bits_rne(lo); mx[b] = f32_to_bf16_bits_rne(hi);
            }
            __syncthreads();
        } else if (lane == 0) {
            mn[b] = f32_to_bf16_bits_rne(lo); mx[b] = f32_to_bf16_bits_rne(hi);
        }
    }
}

// One CTA per top-k block: keys to registers, exact k-th key (through the candidates of select_fast.cuh, by
// bisection where that does not apply), ordered emission.
template <typename T>
__global__ void __launch_bounds__(SEL_THREADS, 1)
block_topk_kernel(int64_t d, int dbs, int nfull, int k_many, int k_few, const T* __restrict__ x,
                  int16_t* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char topk_raw[];            // [SelectSmem | FastSelSmem]
    SelectSmem& sm = *reinterpret_cast<SelectSmem*>(topk_raw);
    FastSelSmem& fs = *reinterpret_cast<FastSelSmem*>(topk_raw + sizeof(SelectSmem));
    const int nblocks = nfull + (k_few > 0 ? 1 : 0);
    int guess = 0;
    for (int blk = blockIdx.x; blk < nblocks; blk += gridDim.x) {
        const int64_t base = (int64_t)blk * dbs;
        const int n = (int)min((int64_t)dbs, d - base);
        const int k = (blk < nfull) ? k_many : k_few;
        const bool vec = (reinterpret_cast<uintptr_t>(x + base) & 15) == 0;
        float key[SEL_OCTETS][8], omax[SEL_OCTETS];
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            const int o = j * SEL_THREADS + (int)threadIdx.x;
            if (vec && o * 8 + 8 <= n) {
                XOctet<T>::load(x + base + o * 8, key[j]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) key[j][e] = (o * 8 + e < n) ? Elem<T>::load(x, base + o * 8 + e) : 0.0f;
            }
            omax[j] = 0.0f;
#pragma unroll
            for (int e = 0; e < 8; ++e) omax[j] = fmaxf(omax[j], fabsf(key[j][e]));
        }
        int n_cand, oct_slot[SEL_OCTETS];
        bool compact_octets;
        if (!fast_select(key, omax, n, k, guess, sm, fs, n_cand, oct_slot, compact_octets, sizeof(T) == 2 ? 16 : 0)) {
            int need;
            const int T_key = block_kth_key_bisect(key, k, sm, need);
            publish_masks(key, T_key, sm);
            resolve_selection(need, sm);
        }
        emit_indices(sm, out + (int64_t)blk * k_many);
        __syncthreads();
    }
}

static int grid_for(int64_t work_items, int threads) {
    int64_t g = ceil_div64(work_items, threads);
    const int64_t cap = (int64_t)device_sm_count() * 16;
    return (int)std::max<int64_t>(1, std::min<int64_t>(g, cap));
}

}  // namespace mab

using namespace mab;

#define MAB_CHECK_LAUNCH(name)                                                     \
    do { mab::count_launch(); cudaError_t _e = cudaGetLastError(); if (_e != cudaSuccess) return cuda_fail(_e, name); } while (0)

// log2 of a power of two, else -1.
static int shift_of(int64_t v) {
    if (v <= 0 || (v & (v - 1)) != 0) return -1;
    int sh = 0;
    while (((int64_t)1 << sh) < v) ++sh;
    return sh;
}

// Whether the octet-wide kernels apply: whole octets inside one quantisation block each, vector-aligned buffers.
static bool octet_form_ok(int64_t d, int64_t qbs, const void* x, const void* error) {
    return d % 8 == 0 && qbs % 8 == 0 && aligned_to(x, 16) && aligned_to(error, 4);
}

static int check_dtype(int dt, const char* what) {
    MAB_REQUIRE(dt == MAB_F32 || dt == MAB_BF16, MAB_ERR_UNSUPPORTED, "%s: dtype code %d is neither MAB_F32 nor MAB_BF16", what, dt);
    return MAB_OK;
}

extern "C" int mab_asymm_block_quant_inv(int64_t d, int64_t qbs, const uint8_t* error, const uint16_t* mn,
                                         const uint16_t* mx, void* x, int x_dtype, float alpha, void* stream) {
    MAB_REQUIRE(d >= 0 && qbs > 0, MAB_ERR_BAD_ARG, "asymm_block_quant_inv: d=%lld qbs=%lld", (long long)d, (long long)qbs);
    if (d == 0) return MAB_OK;
    MAB_REQUIRE(error && mn && mx && x, MAB_ERR_BAD_ARG, "asymm_block_quant_inv: null pointer");
    if (int rc = check_dtype(x_dtype, "asymm_block_quant_inv")) return rc;
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)stream;
    if (octet_form_ok(d, qbs, x, error)) {
        const int grid = grid_for(d / 8, EW_THREADS);
        if (x_dtype == MAB_F32) quant_inv_octet_kernel<float><<<grid, EW_THREADS, 0, s>>>(d / 8, qbs, shift_of(qbs), error, mn, mx, (float*)x, alpha);
        else quant_inv_octet_kernel<uint16_t><<<grid, EW_THREADS, 0, s>>>(d / 8, qbs, shift_of(qbs), error, mn, mx, (uint16_t*)x, alpha);
    } else {
        const int grid = grid_for(ceil_div64(d, EW_CHUNK), EW_THREADS);
        if (x_dtype == MAB_F32) quant_inv_kernel<float><<<grid, EW_THREADS, 0, s>>>(d, qbs, error, mn, mx, (float*)x, alpha);
        else quant_inv_kernel<uint16_t><<<grid, EW_THREADS, 0, s>>>(d, qbs, error, mn, mx, (uint16_t*)x, alpha);
    }
    MAB_CHECK_LAUNCH("asymm_block_quant_inv");
    return MAB_OK;
}

extern "C" int mab_asymm_block_quant(int64_t d, int64_t qbs, uint8_t* error, const uint16_t* mn, const uint16_t* mx,
                                     const void* x, int x_dtype, void* stream) {
    MAB_REQUIRE(d >= 0 && qbs > 0, MAB_ERR_BAD_ARG, "asymm_block_quant: d=%lld qbs=%lld", (long long)d, (long long)qbs);
    if (d == 0) return MAB_OK;
    MAB_REQUIRE(error && mn && mx && x, MAB_ERR_BAD_ARG, "asymm_block_quant: null pointer");
    if (int rc = check_dtype(x_dtype, "asymm_block_quant")) return rc;
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)stream;
    if (octet_form_ok(d, qbs, x, error)) {
        const int grid = grid_for(d / 8, EW_THREADS);
        if (x_dtype == MAB_F32) quant_octet_kernel<float><<<grid, EW_THREADS, 0, s>>>(d / 8, qbs, shift_of(qbs), error, mn, mx, (const float*)x);
        else quant_octet_kernel<uint16_t><<<grid, EW_THREADS, 0, s>>>(d / 8, qbs, shift_of(qbs), error, mn, mx, (const uint16_t*)x);
    } else {
        const int grid = grid_for(ceil_div64(d, EW_CHUNK), EW_THREADS);
        if (x_dtype == MAB_F32) quant_kernel<float><<<grid, EW_THREADS, 0, s>>>(d, qbs, error, mn, mx, (const float*)x);
        else quant_kernel<uint16_t><<<grid, EW_THREADS, 0, s>>>(d, qbs, error, mn, mx, (const uint16_t*)x);
    }
    MAB_CHECK_LAUNCH("asymm_block_quant");
    return MAB_OK;
}

extern "C" int mab_copy_values(int64_t d, int64_t k, int64_t dbs, int64_t kbs, const int16_t* indices, const void* inp,
                               int inp_dtype, void* out, int out_dtype, int direction, void* stream) {
    MAB_REQUIRE(d >= 0 && k >= 0 && dbs > 0 && kbs > 0, MAB_ERR_BAD_ARG, "copy_values: bad sizes");
    MAB_REQUIRE(direction == MAB_D2K || direction == MAB_K2D, MAB_ERR_BAD_ARG, "copy_values: direction %d", direction);
    if (k == 0) return MAB_OK;
    MAB_REQUIRE(indices && inp && out, MAB_ERR_BAD_ARG, "copy_values: null pointer");
    if (int rc = check_dtype(inp_dtype, "copy_values")) return rc;
    if (int rc = check_dtype(out_dtype, "copy_values")) return rc;
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    const int grid = grid_for(k, EW_THREADS);
    cudaStream_t s = (cudaStream_t)stream;
#define LAUNCH_CV(TI, TO) copy_values_kernel<TI, TO><<<grid, EW_THREADS, 0, s>>>(k, dbs, kbs, indices, (const TI*)inp, (TO*)out, direction)
    if (inp_dtype == MAB_F32 && out_dtype == MAB_F32) LAUNCH_CV(float, float);
    else if (inp_dtype == MAB_F32) LAUNCH_CV(float, uint16_t);
    else if (out_dtype == MAB_F32) LAUNCH_CV(uint16_t, float);
    else LAUNCH_CV(uint16_t, uint16_t);
#undef LAUNCH_CV
    MAB_CHECK_LAUNCH("copy_values");
    return MAB_OK;
}

extern "C" int mab_zerorize_block_components(void* x, int x_dtype, const int16_t* indices, int64_t d, int64_t k,
                                             int64_t dbs, int64_t kbs, void* stream) {
    MAB_REQUIRE(d >= 0 && k >= 0 && dbs > 0 && kbs > 0, MAB_ERR_BAD_ARG, "zerorize_block_components: bad sizes");
    if (k == 0) return MAB_OK;
    MAB_REQUIRE(x && indices, MAB_ERR_BAD_ARG, "zerorize_block_components: null pointer");
    if (int rc = check_dtype(x_dtype, "zerorize_block_components")) return rc;
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    const int grid = grid_for(k, EW_THREADS);
    cudaStream_t s = (cudaStream_t)stream;
    if (x_dtype == MAB_F32) zerorize_kernel<float><<<grid, EW_THREADS, 0, s>>>((float*)x, indices, k, dbs, kbs);
    else zerorize_kernel<uint16_t><<<grid, EW_THREADS, 0, s>>>((uint16_t*)x, indices, k, dbs, kbs);
    MAB_CHECK_LAUNCH("zerorize_block_components");
    return MAB_OK;
}

extern "C" int mab_quant_stats(int64_t d, int64_t qbs, uint16_t* mn, uint16_t* mx, const void* x, int x_dtype, void* stream) {
    MAB_REQUIRE(d >= 0 && qbs > 0, MAB_ERR_BAD_ARG, "quant_stats: d=%lld qbs=%lld", (long long)d, (long long)qbs);
    if (d == 0) return MAB_OK;
    MAB_REQUIRE(mn && mx && x, MAB_ERR_BAD_ARG, "quant_stats: null pointer");
    if (int rc = check_dtype(x_dtype, "quant_stats")) return rc;
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    const int64_t nblocks = ceil_div64(d, qbs);
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t cap = (int64_t)device_sm_count() * 16;
    if (d % 8 == 0 && shift_of(qbs) >= 3 && qbs <= 256 && aligned_to(x, 16)) {
        const int grid = grid_for(d / 8, EW_THREADS);
        if (x_dtype == MAB_F32) quant_stats_octet_kernel<float><<<grid, EW_THREADS, 0, s>>>(d / 8, shift_of(qbs), mn, mx, (const float*)x);
        else quant_stats_octet_kernel<uint16_t><<<grid, EW_THREADS, 0, s>>>(d / 8, shift_of(qbs), mn, mx, (const uint16_t*)x);
    } else if (qbs >= 2048) {
        const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(nblocks, cap));
        if (x_dtype == MAB_F32) quant_stats_kernel<float, true><<<grid, EW_THREADS, 0, s>>>(d, qbs, nblocks, mn, mx, (const float*)x);
        else quant_stats_kernel<uint16_t, true><<<grid, EW_THREADS, 0, s>>>(d, qbs, nblocks, mn, mx, (const uint16_t*)x);
    } else {
        const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(ceil_div64(nblocks, EW_THREADS / 32), cap));
        if (x_dtype == MAB_F32) quant_stats_kernel<float, false><<<grid, EW_THREADS, 0, s>>>(d, qbs, nblocks, mn, mx, (const float*)x);
        else quant_stats_kernel<uint16_t, false><<<grid, EW_THREADS, 0, s>>>(d, qbs, nblocks, mn, mx, (const uint16_t*)x);
    }
    MAB_CHECK_LAUNCH("quant_stats");
    return MAB_OK;
}

extern "C" int mab_block_topk(int64_t d, int64_t dbs, int64_t k_many, int64_t k_few, const void* x, int x_dtype,
                              int16_t* out, void* stream) {
    MAB_REQUIRE(d >= 0 && dbs > 0 && k_many >= 0 && k_few >= 0, MAB_ERR_BAD_ARG, "block_topk: bad sizes");
    if (d == 0) return MAB_OK;
    MAB_REQUIRE(dbs <= SEL_MAX_TILE, MAB_ERR_LIMIT, "block_topk: d_block_size %lld exceeds %d", (long long)dbs, SEL_MAX_TILE);
    MAB_REQUIRE(x && out, MAB_ERR_BAD_ARG, "block_topk: null pointer");
    if (int rc = check_dtype(x_dtype, "block_topk")) return rc;
    const int64_t nfull = d / dbs;
    const int64_t tail = d - nfull * dbs;
    MAB_REQUIRE(k_many <= dbs && k_few <= tail && (nfull == 0 || k_many >= 1), MAB_ERR_BAD_ARG,
                "block_topk: k (%lld, %lld) does not fit blocks of %lld / %lld", (long long)k_many, (long long)k_few,
                (long long)dbs, (long long)tail);
    MAB_REQUIRE(nfull < INT32_MAX, MAB_ERR_LIMIT, "block_topk: too many blocks");
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    const int64_t nblocks = nfull + (k_few > 0 ? 1 : 0);
    if (nblocks == 0) return MAB_OK;
    const int grid = (int)std::min<int64_t>(nblocks, (int64_t)device_sm_count() * 4);
    cudaStream_t s = (cudaStream_t)stream;
    const int smem = (int)(sizeof(SelectSmem) + sizeof(FastSelSmem));
    if (x_dtype == MAB_F32) {
        MAB_CUDA_TRY(cudaFuncSetAttribute(block_topk_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        block_topk_kernel<float><<<grid, SEL_THREADS, smem, s>>>(d, (int)dbs, (int)nfull, (int)k_many, (int)k_few, (const float*)x, out);
    } else {
        MAB_CUDA_TRY(cudaFuncSetAttribute(block_topk_kernel<uint16_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        block_topk_kernel<uint16_t><<<grid, SEL_THREADS, smem, s>>>(d, (int)dbs, (int)nfull, (int)k_many, (int)k_few, (const uint16_t*)x, out);
    }
    MAB_CHECK_LAUNCH("block_topk");
    return MAB_OK;
}
