// Kernel B of the step: sparse window -> Adam-style update, weight decay, alpha error-feedback
// integration, parameter update, error-feedback shrink (micro_adam.py:234-235, 276-316), and the
// operator-level compute_microadam_update built on the same code.
//
// Two variants share the streaming epilogue:
//  * tile kernel (the normal case): one CTA of 256 threads per top-k block.  All window entries
//    of the block are staged in shared memory, the touched positions are numbered through a
//    bitmap + prefix popcount, the two moments are accumulated in compact arrays (one slot per
//    touched position, row after row so that the float sums are reproducible), turned into the
//    update, and the block is then streamed in chunks against a small dense copy of the update.
//    Shared memory per CTA is ~44 KB for m = 10, k = 1 %, so five CTAs share an SM and one CTA's
//    window phase overlaps the others' streaming.
//  * wide kernel (window too large for the compact arrays, e.g. m = 20 with k = 5 %): one CTA per
//    sub-range of a block with dense accumulators (window.cuh).
#include "common.cuh"
#include "window.cuh"
#include "fused.cuh"

namespace mab {

enum : int { MODE_WRITE_UPDATE = 0, MODE_STEP = 1 };

// 8 consecutive elements of a buffer as floats; vector access when `full`, else element-wise
// up to `n` (the tensor's last, short octet).
template <typename T> struct Octet;
template <> struct Octet<float> {
    __device__ __forceinline__ static void load(const float* p, float (&v)[8], bool full, int n) {
        if (full) {
            const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = (e < n) ? p[e] : 0.0f;
        }
    }
    __device__ __forceinline__ static void store(float* p, const float (&v)[8], bool full, int n) {
        if (full) {
            reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) if (e < n) p[e] = v[e];
        }
    }
};
template <> struct Octet<uint16_t> {
    __device__ __forceinline__ static void load(const uint16_t* p, float (&v)[8], bool full, int n) {
        if (full) {
            const uint4 a = reinterpret_cast<const uint4*>(p)[0];
            v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
            v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
            v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
            v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = (e < n) ? bf16_bits_to_f32(p[e]) : 0.0f;
        }
    }
    __device__ __forceinline__ static void store(uint16_t* p, const float (&v)[8], bool full, int n) {
        if (full) {
            uint4 a;
            a.x = f32_to_bf16_bits_rne(v[0]) | ((uint32_t)f32_to_bf16_bits_rne(v[1]) << 16);
            a.y = f32_to_bf16_bits_rne(v[2]) | ((uint32_t)f32_to_bf16_bits_rne(v[3]) << 16);
            a.z = f32_to_bf16_bits_rne(v[4]) | ((uint32_t)f32_to_bf16_bits_rne(v[5]) << 16);
            a.w = f32_to_bf16_bits_rne(v[6]) | ((uint32_t)f32_to_bf16_bits_rne(v[7]) << 16);
            reinterpret_cast<uint4*>(p)[0] = a;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) if (e < n) p[e] = f32_to_bf16_bits_rne(v[e]);
        }
    }
};

__device__ __forceinline__ float round_as(float v, bool bf16) {
    return bf16 ? bf16_bits_to_f32(f32_to_bf16_bits_rne(v)) : v;
}

// Streams tensor elements [e0, e0 + len) against the dense update u[0..len) in shared memory
// (already rounded to the gradient's element type).  e0 is a multiple of 8 (and of
// quant_block_size when alpha > 0).  NT threads, all of them must call.
template <typename TP, int MODE, int NT>
__device__ __forceinline__ void stream_range(const mab_tensor& T, const WindowArgs& a, const float* __restrict__ u_s,
                                             int64_t e0, int len) {
    TP* p = reinterpret_cast<TP*>(T.param) + e0;
    const bool vec = aligned16(p);                        // octets stay 16-byte aligned from here
    const int n_oct = (len + 7) >> 3;
    if (MODE == MODE_WRITE_UPDATE) {
        for (int o = threadIdx.x; o < n_oct; o += NT) {
            const int n = min(8, len - o * 8);
            float u[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) u[e] = u_s[o * 8 + e];
            Octet<TP>::store(p + o * 8, u, vec && n == 8, n);
        }
        return;
    }
    const float decay = T.decay_f32, neg_lr = T.neg_lr_f32;
    const bool do_decay = T.weight_decay > 0.0;
    if (a.alpha == 0.0f) {
        // two octets per thread and iteration so that two parameter loads are in flight
        for (int o = threadIdx.x; o < n_oct; o += 2 * NT) {
            const int o2 = o + NT;
            const int n1 = min(8, len - o * 8);
            const int n2 = (o2 < n_oct) ? min(8, len - o2 * 8) : 0;
            float pv1[8], pv2[8];
            Octet<TP>::load(p + o * 8, pv1, vec && n1 == 8, n1);
            if (n2 > 0) Octet<TP>::load(p + o2 * 8, pv2, vec && n2 == 8, n2);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float x = pv1[e];
                if (do_decay) x = Elem<TP>::round(__fmul_rn(x, decay));
                pv1[e] = fmaf(neg_lr, u_s[o * 8 + e], x);
            }
            Octet<TP>::store(p + o * 8, pv1, vec && n1 == 8, n1);
            if (n2 > 0) {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float x = pv2[e];
                    if (do_decay) x = Elem<TP>::round(__fmul_rn(x, decay));
                    pv2[e] = fmaf(neg_lr, u_s[o2 * 8 + e], x);
                }
                Octet<TP>::store(p + o2 * 8, pv2, vec && n2 == 8, n2);
            }
        }
        return;
    }
    // alpha > 0: u += alpha * Qinv(e); p update; e <- Q((1 - alpha) * Qinv(e)) with fresh statistics
    const bool g_bf16 = (T.grad_dtype == MAB_BF16);
    const int lanes = a.lanes_per_qb;
    const int n_oct_pad = (n_oct + 31) & ~31;
    for (int o = threadIdx.x; o < n_oct_pad; o += NT) {
        const int n = max(0, min(8, len - o * 8));
        const int64_t ge = e0 + (int64_t)o * 8;        // global element index of the octet
        float xs[8];
        float lo = INFINITY, hi = -INFINITY;
        int64_t qb = 0;
        if (n > 0) {
            qb = ge / a.qbs;
            const QParams q = qparams(T.min_vals[qb], T.max_vals[qb]);
            uint32_t codes = 0;
            const uint8_t* ef = T.error + (ge >> 1);
#pragma unroll
            for (int b = 0; b < 4; ++b) if (2 * b < n) codes |= (uint32_t)ef[b] << (8 * b);
            float pv[8];
            Octet<TP>::load(p + o * 8, pv, vec && n == 8, n);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t code = (codes >> (8 * (e >> 1) + ((e & 1) ? 0 : 4))) & 0xFu;
                const float x1 = qinv(code, q);
                const float u = round_as(__fadd_rn(u_s[o * 8 + e], __fmul_rn(a.alpha, x1)), g_bf16);
                float x = pv[e];
                if (do_decay) x = Elem<TP>::round(__fmul_rn(x, decay));
                pv[e] = fmaf(neg_lr, u, x);
                xs[e] = round_as(__fadd_rn(0.0f, __fmul_rn(a.one_minus_alpha, x1)), g_bf16);
                if (e < n) { lo = fminf(lo, xs[e]); hi = fmaxf(hi, xs[e]); }
            }
            Octet<TP>::store(p + o * 8, pv, vec && n == 8, n);
        }
        for (int off = 1; off < lanes; off <<= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, off));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, off));
        }
        if (n > 0) {
            const uint16_t mn_b = f32_to_bf16_bits_rne(lo), mx_b = f32_to_bf16_bits_rne(hi);
            if ((ge % a.qbs) == 0) { T.min_vals[qb] = mn_b; T.max_vals[qb] = mx_b; }
            const QParams q2 = qparams(mn_b, mx_b);
            uint8_t* ef = T.error + (ge >> 1);
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (2 * b < n) {
                    const uint32_t c0 = qcode_exact(xs[2 * b], q2);
                    const uint32_t c1 = (2 * b + 1 < n) ? qcode_exact(xs[2 * b + 1], q2) : 0u;
                    ef[b] = (uint8_t)((c0 << 4) | c1);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------ tile kernel

constexpr int WT_THREADS = 256;
constexpr int WT_CHUNK = 3712;            // positions per streaming chunk: 29 * 128
constexpr int WT_WORDS = 1024;            // bitmap words (32768 positions)
constexpr int WT_MAX_ENTRIES = 16384;     // window entries of one block the compact arrays may hold

__host__ __device__ constexpr int wt_smem_bytes(int entries) {
    const int e = (entries + 3) & ~3;
    const int staging = e > WT_CHUNK ? 4 * e : 4 * WT_CHUNK;
    return 8 * e + staging + 4 * WT_WORDS + 2 * WT_WORDS;
}

// Fast (not correctly rounded) form of m_hat / (sqrt(v_hat) + eps): the update is specified to
// a tolerance, and the approximations are deterministic.
__device__ __forceinline__ float adam_update_fast(float m, float v, float inv_bc1, float inv_bc2, float eps) {
    float s;
    asm("sqrt.approx.f32 %0, %1;" : "=f"(s) : "f"(v * inv_bc2));
    return __fdividef(m * inv_bc1, s + eps);
}

template <typename TP, int MODE>
__device__ __forceinline__ void window_tile_body(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units,
                                                 int max_entries, const WindowArgs& a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_first[WIN_MAX_TENSORS + 1];
    __shared__ int s_scan[36];
    const int ecap = (max_entries + 3) & ~3;
    float* m_acc = reinterpret_cast<float*>(smem_raw);
    float* v_acc = m_acc + ecap;
    uint32_t* ent = reinterpret_cast<uint32_t*>(v_acc + ecap);          // (bf16 value << 16) | position, later | slot
    float* dense = reinterpret_cast<float*>(ent);                        // aliases ent once the entries are consumed
    const int staging_words = max(ecap, WT_CHUNK);
    uint32_t* bitmap = ent + staging_words;
    uint16_t* prefix = reinterpret_cast<uint16_t*>(bitmap + WT_WORDS);
    const int t = threadIdx.x;

    for (int i = t; i < n_tensors; i += WT_THREADS) s_first[i] = tensors[i].first_unit_a;
    if (t == 0) s_first[n_tensors] = total_units;
    __syncthreads();
    const float inv_bc1 = 1.0f / a.bc1, inv_bc2 = 1.0f / a.bc2;

    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        const int ti = find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const int dbs = T.d_block_size, nfull = T.topk_full_blocks_count;
        const int64_t blk_base = (int64_t)blk * dbs;
        const int n_blk = (int)min((int64_t)dbs, T.d - blk_base);
        const int kcnt = (blk < nfull) ? T.k_block_size_many : T.k_block_size_few;
        const int64_t koff = (int64_t)blk * T.k_block_size_many;
        const int16_t* __restrict__ I_blk = T.I + koff;
        const uint16_t* __restrict__ V_blk = T.V + koff;
        const int64_t pitch = T.k;
        const int rows = a.rows;
        const int E = rows * kcnt;
        const bool g_bf16 = (T.grad_dtype == MAB_BF16);

        // 1. stage the window entries, clear the bitmap and the compact moments
        for (int r = 0; r < rows; ++r)
            for (int j = t; j < kcnt; j += WT_THREADS)
                ent[r * kcnt + j] = ((uint32_t)V_blk[r * pitch + j] << 16) | (uint32_t)(uint16_t)I_blk[r * pitch + j];
        for (int i = t; i < WT_WORDS; i += WT_THREADS) bitmap[i] = 0u;
        for (int i = t; i < E; i += WT_THREADS) { m_acc[i] = 0.0f; v_acc[i] = 0.0f; }
        __syncthreads();
        // 2. mark touched positions
        for (int i = t; i < E; i += WT_THREADS) {
            const uint32_t pos = ent[i] & 0xFFFFu;
            atomicOr(&bitmap[pos >> 5], 1u << (pos & 31));
        }
        __syncthreads();
        // 3. number them: prefix[w] = touched positions in words below w
        int cnt[WT_WORDS / WT_THREADS], local = 0;
#pragma unroll
        for (int i = 0; i < WT_WORDS / WT_THREADS; ++i) { cnt[i] = __popc(bitmap[t * (WT_WORDS / WT_THREADS) + i]); local += cnt[i]; }
        int touched;
        int run = block_exclusive_scan(local, s_scan, touched);
#pragma unroll
        for (int i = 0; i < WT_WORDS / WT_THREADS; ++i) { prefix[t * (WT_WORDS / WT_THREADS) + i] = (uint16_t)run; run += cnt[i]; }
        __syncthreads();
        // 4. replace positions by slots, then accumulate row after row
        for (int i = t; i < E; i += WT_THREADS) {
            const uint32_t e = ent[i];
            const uint32_t pos = e & 0xFFFFu;
            const uint32_t slot = prefix[pos >> 5] + __popc(bitmap[pos >> 5] & ((1u << (pos & 31)) - 1u));
            ent[i] = (e & 0xFFFF0000u) | slot;
        }
        __syncthreads();
        for (int r = 0; r < rows; ++r) {
            const float w1 = a.w1[r], w2 = a.w2[r];
            for (int j = t; j < kcnt; j += WT_THREADS) {
                const uint32_t e = ent[r * kcnt + j];
                const int slot = e & 0xFFFFu;
                const float val = __uint_as_float(e & 0xFFFF0000u);
                m_acc[slot] = __fadd_rn(m_acc[slot], __fmul_rn(val, w1));
                v_acc[slot] = __fadd_rn(v_acc[slot], __fmul_rn(__fmul_rn(val, val), w2));
            }
            __syncthreads();
        }
        // 5. moments -> update (rounded to the gradient's element type), slot by slot
        for (int s = t; s < touched; s += WT_THREADS)
            m_acc[s] = round_as(adam_update_fast(m_acc[s], v_acc[s], inv_bc1, inv_bc2, a.eps), g_bf16);
        // 6. stream the block in chunks against a dense copy of the update
        for (int c0 = 0; c0 < n_blk; c0 += WT_CHUNK) {
            const int len = min(WT_CHUNK, n_blk - c0);
            __syncthreads();                                   // ent / dense free, updates final
            for (int i = t; i < WT_CHUNK / 4; i += WT_THREADS) reinterpret_cast<float4*>(dense)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            __syncthreads();
            const int w0 = c0 >> 5, nw = (len + 31) >> 5;
            for (int w = t; w < nw; w += WT_THREADS) {
                uint32_t bits = bitmap[w0 + w];
                int slot = prefix[w0 + w];
                while (bits) {
                    const int b = __ffs(bits) - 1;
                    bits &= bits - 1;
                    dense[w * 32 + b] = m_acc[slot++];
                }
            }
            __syncthreads();
            stream_range<TP, MODE, WT_THREADS>(T, a, dense, blk_base + c0, len);
        }
        __syncthreads();                                       // everything is reused by the next unit
    }
}

template <typename TP, int MODE>
__global__ void __launch_bounds__(WT_THREADS)
window_tile_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int max_entries,
                   const __grid_constant__ WindowArgs a) {
    window_tile_body<TP, MODE>(tensors, n_tensors, total_units, max_entries, a);
}

// Single tensor whose descriptor travels as a kernel argument (operator-level entry point).
template <typename TP, int MODE>
__global__ void __launch_bounds__(WT_THREADS)
window_tile_single_kernel(const __grid_constant__ mab_tensor t, int total_units, int max_entries,
                          const __grid_constant__ WindowArgs a) {
    window_tile_body<TP, MODE>(&t, 1, total_units, max_entries, a);
}

// ------------------------------------------------------------------------------------ wide kernel

// TP: element type of `param` (MODE_STEP) or of the output buffer held in `param` (MODE_WRITE_UPDATE).
template <typename TP, int MODE>
__device__ __forceinline__ void window_wide_body(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units,
                                                 const WindowArgs& a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int s_first[WIN_MAX_TENSORS + 1];
    WindowSmem sm(smem_raw);
    for (int i = threadIdx.x; i < n_tensors; i += WIN_THREADS) s_first[i] = tensors[i].first_unit_b;
    if (threadIdx.x == 0) s_first[n_tensors] = total_units;
    __syncthreads();

    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        const int ti = find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        const int dbs = T.d_block_size, nfull = T.topk_full_blocks_count;
        const int subs_per_block = (dbs + WIN_SR - 1) / WIN_SR;
        const int local = unit - s_first[ti];
        int blk = local / subs_per_block, sub = local - blk * subs_per_block;
        if (blk > nfull) { sub += (blk - nfull) * subs_per_block; blk = nfull; }
        const int64_t blk_base = (int64_t)blk * dbs;
        const int n_blk = (int)min((int64_t)dbs, T.d - blk_base);
        const int kcnt = (blk < nfull) ? T.k_block_size_many : T.k_block_size_few;
        const int s0 = sub * WIN_SR;
        const int len = min(WIN_SR, n_blk - s0);
        const int64_t koff = (int64_t)blk * T.k_block_size_many;

        window_to_update(T.I + koff, T.V + koff, T.k, kcnt, s0, len, a, sm);
        if (T.grad_dtype == MAB_BF16) {
            for (int i = threadIdx.x; i < len; i += WIN_THREADS) sm.m_acc[i] = round_as(sm.m_acc[i], true);
            __syncthreads();
        }
        stream_range<TP, MODE, WIN_THREADS>(T, a, sm.m_acc, blk_base + s0, len);
        __syncthreads();   // shared accumulators are reused by the next unit
    }
}

template <typename TP, int MODE>
__global__ void __launch_bounds__(WIN_THREADS)
window_wide_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, const __grid_constant__ WindowArgs a) {
    window_wide_body<TP, MODE>(tensors, n_tensors, total_units, a);
}

template <typename TP, int MODE>
__global__ void __launch_bounds__(WIN_THREADS)
window_wide_single_kernel(const __grid_constant__ mab_tensor t, int total_units, const __grid_constant__ WindowArgs a) {
    window_wide_body<TP, MODE>(&t, 1, total_units, a);
}

// ------------------------------------------------------------------------------------ launch

// `single` != nullptr: one tensor passed by value; else n_tensors descriptors in device memory.
// units_tile / units_wide are the unit counts of the two variants; max_entries = rows * largest
// k_block_size of the launch decides which one runs.
template <typename TP, int MODE>
static int launch_window(const mab_tensor* dev_tensors, const mab_tensor* single, int n_tensors, int units_tile,
                         int units_wide, int max_entries, const WindowArgs& a, cudaStream_t s) {
    const int sms = device_sm_count();
    if (max_entries <= WT_MAX_ENTRIES) {
        const int smem = wt_smem_bytes(max_entries);
        const int per_sm = std::max(1, std::min(8, (227 * 1024) / (smem + 2048)));
        const int grid = (int)std::min<int64_t>(units_tile, (int64_t)sms * per_sm);
        if (single) {
            auto kern = window_tile_single_kernel<TP, MODE>;
            MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            kern<<<grid, WT_THREADS, smem, s>>>(*single, units_tile, max_entries, a);
        } else {
            auto kern = window_tile_kernel<TP, MODE>;
            MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            kern<<<grid, WT_THREADS, smem, s>>>(dev_tensors, n_tensors, units_tile, max_entries, a);
        }
    } else {
        const int grid = (int)std::min<int64_t>(units_wide, (int64_t)sms * 2);
        if (single) {
            auto kern = window_wide_single_kernel<TP, MODE>;
            MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WIN_SMEM_BYTES));
            kern<<<grid, WIN_THREADS, WIN_SMEM_BYTES, s>>>(*single, units_wide, a);
        } else {
            auto kern = window_wide_kernel<TP, MODE>;
            MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WIN_SMEM_BYTES));
            kern<<<grid, WIN_THREADS, WIN_SMEM_BYTES, s>>>(dev_tensors, n_tensors, units_wide, a);
        }
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "window kernel launch");
    return MAB_OK;
}

int fill_window_args(WindowArgs& a, int64_t steps, int m, double beta1, double beta2, double eps, float alpha, int qbs) {
    MAB_REQUIRE(steps >= 1, MAB_ERR_BAD_ARG, "steps must be >= 1 (got %lld)", (long long)steps);
    MAB_REQUIRE(m >= 1 && m <= MAB_MAX_WINDOW, MAB_ERR_LIMIT, "m=%d outside [1, %d]", m, MAB_MAX_WINDOW);
    a.rows = (int)std::min<int64_t>(steps, m);
    for (int r = 0; r < MAB_MAX_WINDOW; ++r) { a.w1[r] = 0.f; a.w2[r] = 0.f; }
    for (int r = 0; r < a.rows; ++r) {
        const int64_t age = ((steps - 1) - r) % m;
        a.w1[r] = (float)(pow(beta1, (double)age) * (1.0 - beta1));
        a.w2[r] = (float)(pow(beta2, (double)age) * (1.0 - beta2));
    }
    a.bc1 = (float)(1.0 - pow(beta1, (double)steps));
    a.bc2 = (float)(1.0 - pow(beta2, (double)steps));
    a.eps = (float)eps;
    a.alpha = alpha;
    a.one_minus_alpha = (float)(1.0 - (double)alpha);
    a.qbs = qbs;
    a.lanes_per_qb = qbs >= 8 ? qbs / 8 : 1;
    return MAB_OK;
}

int launch_window_step(const mab_tensor* dev_tensors, int n_tensors, int units_tile, int units_wide, int max_entries,
                       int param_dtype, const WindowArgs& a, cudaStream_t s) {
    if (param_dtype == MAB_F32)
        return launch_window<float, MODE_STEP>(dev_tensors, nullptr, n_tensors, units_tile, units_wide, max_entries, a, s);
    return launch_window<uint16_t, MODE_STEP>(dev_tensors, nullptr, n_tensors, units_tile, units_wide, max_entries, a, s);
}

int units_b_of(const mab_tensor& t) {
    const int subs = (t.d_block_size + WIN_SR - 1) / WIN_SR;
    const int64_t tail = t.d - (int64_t)t.topk_full_blocks_count * t.d_block_size;
    return t.topk_full_blocks_count * subs + (t.k_block_size_few > 0 ? (int)((tail + WIN_SR - 1) / WIN_SR) : 0);
}

}  // namespace mab

using namespace mab;

extern "C" int mab_compute_microadam_update(int blocks, int threads, int carveout, int64_t steps, double beta1, double beta2,
                                            double eps, int64_t dbs, int64_t kbs, int64_t d, int64_t m, int64_t k,
                                            const int16_t* I, const uint16_t* V, void* out, int out_dtype, void* stream) {
    (void)blocks; (void)threads; (void)carveout;
    MAB_REQUIRE(d >= 0 && k >= 0 && dbs > 0 && kbs > 0, MAB_ERR_BAD_ARG, "compute_microadam_update: bad sizes");
    if (d == 0) return MAB_OK;
    MAB_REQUIRE(I && V && out, MAB_ERR_BAD_ARG, "compute_microadam_update: null pointer");
    MAB_REQUIRE(out_dtype == MAB_F32 || out_dtype == MAB_BF16, MAB_ERR_UNSUPPORTED, "compute_microadam_update: dtype %d", out_dtype);
    MAB_REQUIRE(dbs <= 32768, MAB_ERR_LIMIT, "compute_microadam_update: d_block_size %lld exceeds 32768", (long long)dbs);
    MAB_REQUIRE(dbs % 8 == 0 || d <= dbs, MAB_ERR_UNSUPPORTED,
                "compute_microadam_update: d_block_size %lld is not a multiple of 8", (long long)dbs);
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    WindowArgs a;
    if (int rc = fill_window_args(a, steps, (int)m, beta1, beta2, eps, 0.0f, 8)) return rc;

    mab_tensor t = {};
    t.param = out; t.I = const_cast<int16_t*>(I); t.V = const_cast<uint16_t*>(V);
    t.d = d; t.k = k; t.d_block_size = (int)dbs;
    t.topk_full_blocks_count = (int)(d / dbs);
    const int64_t tail = d - (int64_t)t.topk_full_blocks_count * dbs;
    t.k_block_size_many = (int)kbs;
    t.k_block_size_few = (int)(k - (int64_t)t.topk_full_blocks_count * kbs);
    MAB_REQUIRE(t.k_block_size_few >= 0 && (tail > 0 || t.k_block_size_few == 0), MAB_ERR_BAD_ARG,
                "compute_microadam_update: k=%lld inconsistent with d=%lld, d_block_size=%lld, k_block_size=%lld",
                (long long)k, (long long)d, (long long)dbs, (long long)kbs);
    t.param_dtype = out_dtype; t.grad_dtype = out_dtype;
    const int units_wide = units_b_of(t);
    const int units_tile = t.topk_full_blocks_count + (t.k_block_size_few > 0 ? 1 : 0);
    if (units_tile == 0) return MAB_OK;
    const int64_t max_entries = (int64_t)a.rows * std::max(t.k_block_size_many, t.k_block_size_few);
    cudaStream_t s = (cudaStream_t)stream;
    const int me = (int)std::min<int64_t>(max_entries, INT32_MAX);
    if (out_dtype == MAB_F32) return launch_window<float, MODE_WRITE_UPDATE>(nullptr, &t, 1, units_tile, units_wide, me, a, s);
    return launch_window<uint16_t, MODE_WRITE_UPDATE>(nullptr, &t, 1, units_tile, units_wide, me, a, s);
}
