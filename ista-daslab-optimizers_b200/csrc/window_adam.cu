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
#include "async_copy.cuh"

namespace mab {

#ifdef MAB_STATS
// Development-only phase timers of the tile kernel (cycles of thread 0, summed over tiles); [15] = tiles.
__device__ unsigned long long g_stats_b[16];
#define MAB_BTICK(i) do { if (threadIdx.x == 0) { const long long _now = clock64(); atomicAdd(&g_stats_b[i], (unsigned long long)(_now - b_tick)); b_tick = _now; } } while (0)
#define MAB_BTICK_DECL long long b_tick = clock64();
#else
#define MAB_BTICK(i) do { } while (0)
#define MAB_BTICK_DECL
#endif

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
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(a.x) : "f"(v[1]), "f"(v[0]));
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(a.y) : "f"(v[3]), "f"(v[2]));
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(a.z) : "f"(v[5]), "f"(v[4]));
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(a.w) : "f"(v[7]), "f"(v[6]));
            reinterpret_cast<uint4*>(p)[0] = a;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) if (e < n) p[e] = f32_to_bf16_bits_rne(v[e]);
        }
    }
};

// Two floats -> two bf16 (round to nearest even) in one conversion; low half = first value.
__device__ __forceinline__ uint32_t cvt_bf16x2_rne(float a, float b) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
    return d;
}

// p <- round_p(round_p(p * decay) - lr * u) for 8 values, two per instruction (packed f32x2
// operations round each component like the scalar ones).
// HAS_U = false: only the decay (the caller updates the few touched elements afterwards).
template <typename TP, bool HAS_U = true>
__device__ __forceinline__ void update_octet(float (&pv)[8], const float (&u)[8], bool do_decay, float2 decay2, float2 neg_lr2) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        float2 x = make_float2(pv[2 * b], pv[2 * b + 1]);
        if (do_decay) {
            x = __fmul2_rn(x, decay2);
            if (sizeof(TP) == 2) {                       // the decayed value is stored as bf16 before the update reads it
                const uint32_t w = cvt_bf16x2_rne(x.x, x.y);
                x = make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
            }
        }
        if (HAS_U) x = __ffma2_rn(neg_lr2, make_float2(u[2 * b], u[2 * b + 1]), x);
        pv[2 * b] = x.x; pv[2 * b + 1] = x.y;
    }
}

// An octet as loaded (16-byte vectors), unpacked to floats only when it is used.
template <typename T> struct RawOctet;
template <> struct RawOctet<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = reinterpret_cast<const float4*>(p)[0]; b = reinterpret_cast<const float4*>(p)[1]; }
    __device__ __forceinline__ void unpack(float (&v)[8]) const {
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct RawOctet<uint16_t> {
    uint4 a;
    __device__ __forceinline__ void load(const uint16_t* p) { a = reinterpret_cast<const uint4*>(p)[0]; }
    __device__ __forceinline__ void unpack(float (&v)[8]) const {
        v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
        v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
        v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
        v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
    }
};

// Where the streaming loop gets the update of octet o (8 consecutive elements of the range) from.
struct NoU {                    // no update: the stream only applies the weight decay
    static constexpr bool has_u = false;
    __device__ __forceinline__ void load(int, float (&v)[8]) const {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.0f;
    }
};
struct DenseU {                 // a dense float array in shared memory, 16-byte aligned
    static constexpr bool has_u = true;
    const float* u;
    __device__ __forceinline__ void load(int o, float (&v)[8]) const {
        const float4 a = reinterpret_cast<const float4*>(u + o * 8)[0], b = reinterpret_cast<const float4*>(u + o * 8)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
struct SparseU {                // touched positions as a bitmap, their updates compact in slot order
    static constexpr bool has_u = true;
    const uint32_t* bitmap;     // bit i of the range set <=> position i touched
    const uint16_t* prefix;     // touched positions in lower bitmap words
    const float2* mv;           // .x = update of the slot
    __device__ __forceinline__ void load(int o, float (&v)[8]) const {
        const uint32_t word = bitmap[o >> 2];
        const uint32_t sh = 8u * (o & 3);
        const uint32_t byte = (word >> sh) & 0xFFu;
        int slot = prefix[o >> 2] + __popc(word & ((1u << sh) - 1u));
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const bool on = (byte >> e) & 1u;
            v[e] = on ? mv[slot].x : 0.0f;
            slot += on ? 1 : 0;
        }
    }
};

// Per-thread partial sums of the update's logging probes (micro_adam.py:306-308, 272-273); they live across the
// blocks a CTA works on and reach the probe buffer once, when the kernel ends.
struct UpdateProbe {
    float sum_u2 = 0.0f, sum_qe2 = 0.0f;
    int zeros_u = 0, zeros_qe = 0;
    __device__ __forceinline__ void flush(double* probe) {
        if (probe == nullptr) return;
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            sum_u2 += __shfl_xor_sync(0xffffffffu, sum_u2, o);
            sum_qe2 += __shfl_xor_sync(0xffffffffu, sum_qe2, o);
            zeros_u += __shfl_xor_sync(0xffffffffu, zeros_u, o);
            zeros_qe += __shfl_xor_sync(0xffffffffu, zeros_qe, o);
        }
        if (lane_id() == 0) {
            if (sum_u2 != 0.0f) atomicAdd(&probe[MAB_PROBE_NORM_U], (double)sum_u2);
            if (zeros_u != 0) atomicAdd(&probe[MAB_PROBE_ZEROS_U], (double)zeros_u);
            if (sum_qe2 != 0.0f) atomicAdd(&probe[MAB_PROBE_NORM_QE], (double)sum_qe2);
            if (zeros_qe != 0) atomicAdd(&probe[MAB_PROBE_ZEROS_QE], (double)zeros_qe);
        }
    }
};

__device__ __forceinline__ float round_as(float v, bool bf16) {
    return bf16 ? bf16_bits_to_f32(f32_to_bf16_bits_rne(v)) : v;
}

// Streams tensor elements [e0, e0 + len) against their updates (already rounded to the gradient's
// element type), which `src` delivers octet by octet.  e0 is a multiple of 8 (and of
// quant_block_size when alpha > 0).  NT threads, all of them must call.  ALPHA selects the form at
// compile time: 0 = no alpha term, 1 = alpha > 0 (it needs many more registers), 2 = alpha == -2.
template <typename TP, int MODE, int NT, int ALPHA, typename USrc>
__device__ __forceinline__ void stream_range(const mab_tensor& T, const WindowArgs& a, const USrc& src, int64_t e0, int len,
                                             UpdateProbe& pr) {
    const bool probing = MODE == MODE_STEP && a.probe != nullptr;
    TP* p = reinterpret_cast<TP*>(T.param) + e0;
    const bool vec = aligned16(p);                        // octets stay 16-byte aligned from here
    const int n_oct = (len + 7) >> 3;
    if (MODE == MODE_WRITE_UPDATE) {
        for (int o = threadIdx.x; o < n_oct; o += NT) {
            const int n = min(8, len - o * 8);
            float u[8];
            src.load(o, u);
            Octet<TP>::store(p + o * 8, u, vec && n == 8, n);
        }
        return;
    }
    const float decay = T.decay_f32, neg_lr = T.neg_lr_f32;
    const bool do_decay = T.weight_decay > 0.0;
    if (ALPHA == 0) {
        const float2 decay2 = make_float2(decay, decay), neg_lr2 = make_float2(neg_lr, neg_lr);
        constexpr int B = (sizeof(TP) == 2) ? 4 : 2;          // octets per thread and batch
        const int full_oct = vec ? (len >> 3) : 0;           // octets that can move as 16-byte vectors
        const int nbatch = (full_oct + B * NT - 1) / (B * NT);
        // software pipeline: the loads of batch i + 1 are in flight while batch i is computed and stored
        RawOctet<TP> cur[B], nxt[B];
#pragma unroll
        for (int i = 0; i < B; ++i) { const int o = threadIdx.x + i * NT; if (o < full_oct) cur[i].load(p + o * 8); }
        for (int bi = 0; bi < nbatch; ++bi) {
            const int o0 = bi * B * NT + threadIdx.x;
            if (bi + 1 < nbatch) {
#pragma unroll
                for (int i = 0; i < B; ++i) { const int o = o0 + (B + i) * NT; if (o < full_oct) nxt[i].load(p + o * 8); }
            }
#pragma unroll
            for (int i = 0; i < B; ++i) {
                const int o = o0 + i * NT;
                if (o < full_oct) {
                    float pv[8], u[8];
                    cur[i].unpack(pv);
                    src.load(o, u);
                    if (USrc::has_u && probing) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) { pr.sum_u2 = fmaf(u[e], u[e], pr.sum_u2); pr.zeros_u += (u[e] == 0.0f) ? 1 : 0; }
                    }
                    update_octet<TP, USrc::has_u>(pv, u, do_decay, decay2, neg_lr2);
                    Octet<TP>::store(p + o * 8, pv, true, 8);
                }
            }
#pragma unroll
            for (int i = 0; i < B; ++i) cur[i] = nxt[i];
        }
        // the ragged rest (a misaligned tensor, or the last, short octet): element-wise
        for (int o = full_oct + threadIdx.x; o < n_oct; o += NT) {
            const int n = min(8, len - o * 8);
            float pv[8], u[8];
            Octet<TP>::load(p + o * 8, pv, false, n);
            src.load(o, u);
            if (USrc::has_u && probing) {
#pragma unroll
                for (int e = 0; e < 8; ++e) if (e < n) { pr.sum_u2 = fmaf(u[e], u[e], pr.sum_u2); pr.zeros_u += (u[e] == 0.0f) ? 1 : 0; }
            }
            update_octet<TP, USrc::has_u>(pv, u, do_decay, decay2, neg_lr2);
            Octet<TP>::store(p + o * 8, pv, false, n);
        }
        return;
    }
    const bool g_bf16 = (T.grad_dtype == MAB_BF16);
    if (ALPHA == 2) {
        // alpha == -2 (micro_adam.py:238-273), with a = the residual kernel A left in quant_err and e = the new codes:
        //   p <- decay(p);  p <- p - a;  p <- p + Qinv(e);  quant_err <- a - Qinv(e);  then p <- p - lr * u
        TP* qe = reinterpret_cast<TP*>(T.quant_err) + e0;
        const bool vec_q = aligned16(qe);
        for (int o = threadIdx.x; o < n_oct; o += NT) {
            const int n = min(8, len - o * 8);
            const int64_t ge = e0 + (int64_t)o * 8;
            const int64_t qb = ge / a.qbs;
            const QParams q = qparams(T.min_vals[qb], T.max_vals[qb]);
            uint32_t codes = 0;
            const uint8_t* ef = T.error + (ge >> 1);
#pragma unroll
            for (int b = 0; b < 4; ++b) if (2 * b < n) codes |= (uint32_t)ef[b] << (8 * b);
            float pv[8], av[8], uo[8];
            Octet<TP>::load(p + o * 8, pv, vec && n == 8, n);
            Octet<TP>::load(qe + o * 8, av, vec_q && n == 8, n);
            src.load(o, uo);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t code = (codes >> (8 * (e >> 1) + ((e & 1) ? 0 : 4))) & 0xFu;
                const float x = round_as(__fadd_rn(0.0f, qinv(code, q)), g_bf16);             // grad.zero_(); grad += Qinv(e)
                float v = pv[e];
                if (do_decay) v = Elem<TP>::round(__fmul_rn(v, decay));
                v = Elem<TP>::round(__fsub_rn(v, av[e]));                                     // p.add_(grad, alpha=-1)
                v = Elem<TP>::round(__fadd_rn(v, x));                                         // p.add_(grad)
                av[e] = Elem<TP>::round(__fsub_rn(av[e], x));                                 // quant_err.sub_(grad)
                pv[e] = fmaf(neg_lr, uo[e], v);
                if (probing && e < n) {
                    pr.sum_u2 = fmaf(uo[e], uo[e], pr.sum_u2); pr.zeros_u += (uo[e] == 0.0f) ? 1 : 0;
                    pr.sum_qe2 = fmaf(av[e], av[e], pr.sum_qe2); pr.zeros_qe += (av[e] == 0.0f) ? 1 : 0;
                }
            }
            Octet<TP>::store(p + o * 8, pv, vec && n == 8, n);
            Octet<TP>::store(qe + o * 8, av, vec_q && n == 8, n);
        }
        return;
    }
    // alpha > 0: u += alpha * Qinv(e); p update; e <- Q((1 - alpha) * Qinv(e)) with fresh statistics
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
            float pv[8], uo[8];
            Octet<TP>::load(p + o * 8, pv, vec && n == 8, n);
            src.load(o, uo);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t code = (codes >> (8 * (e >> 1) + ((e & 1) ? 0 : 4))) & 0xFu;
                const float x1 = qinv(code, q);
                const float u = round_as(__fadd_rn(uo[e], __fmul_rn(a.alpha, x1)), g_bf16);
                if (probing && e < n) { pr.sum_u2 = fmaf(u, u, pr.sum_u2); pr.zeros_u += (u == 0.0f) ? 1 : 0; }
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

constexpr int WT_WORDS = 1024;            // bitmap words (32768 positions)
constexpr int WT_MAX_ENTRIES = 16384;     // window entries of one block the compact arrays may hold
constexpr int WT_KEEP = 6;                // window entries a thread keeps in registers between marking and numbering
constexpr int WT_NO_SLOT = 0xFFFF;        // slot of a window entry whose index lies outside the block (slots stay below 32768)

// Bytes one row's slice of I (or V) occupies in the raw staging area: the slice is copied from the
// 16-byte boundary below its first element, in whole 16-byte pieces.
__host__ __device__ constexpr int wt_row_stride(int max_k) { return ((max_k * 2 + 30) + 15) & ~15; }

__host__ __device__ constexpr int wt_smem_bytes(int rows, int max_k) {
    const int e = (rows * max_k + 3) & ~3;
    return 8 * e + rows * 2 * wt_row_stride(max_k) + 4 * WT_WORDS + 2 * WT_WORDS + 2 * e;
}

// Asks L2 for one unit's slices of the valid window rows: one thread per row slice of I or V.
// `who` = index of the calling thread among those that ask (the first 2 * rows of them do).
__device__ __forceinline__ void prefetch_window_rows(const mab_tensor& T, int blk, int rows, int who) {
    if (who < 2 * rows) {
        const int kcnt = (blk < T.topk_full_blocks_count) ? T.k_block_size_many : T.k_block_size_few;
        const int r = who >> 1;
        const int64_t off = (int64_t)blk * T.k_block_size_many + (int64_t)r * row_pitch_of(T);
        const uintptr_t base = (who & 1) ? reinterpret_cast<uintptr_t>(T.V + off) : reinterpret_cast<uintptr_t>(T.I + off);
        const uintptr_t end = base + 2u * kcnt;
        for (uintptr_t line = base & ~(uintptr_t)127; line < end; line += 128)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
    }
}

__device__ __forceinline__ void cp_async_16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src_gmem) : "memory");
}

// Shared-memory arrays of the window phases of one tile.
struct WindowTileSmem {
    float2*        mv;        // (first moment | update, second moment) per slot
    unsigned char* raw;       // rows x {I slice, V slice}, rstride bytes each
    uint32_t*      bitmap;    // touched positions
    uint16_t*      prefix;    // touched positions in lower bitmap words
    uint16_t*      spos;      // position of each slot
    int            rstride;
    __device__ WindowTileSmem(unsigned char* base, int rows, int max_k) {
        const int ecap = (rows * max_k + 3) & ~3;
        rstride = wt_row_stride(max_k);
        mv = reinterpret_cast<float2*>(base);
        raw = reinterpret_cast<unsigned char*>(mv + ecap);
        bitmap = reinterpret_cast<uint32_t*>(raw + rows * 2 * rstride);
        prefix = reinterpret_cast<uint16_t*>(bitmap + WT_WORDS);
        spos = prefix + WT_WORDS;
    }
};

// Phases 1-4 of a tile, by the NT threads of the CTA: stages the `rows` window rows of block `blk`, numbers
// the touched positions (slots, in ascending position) and accumulates both moments row after row into
// w.mv[slot].  Returns the number of touched positions.  Ends with a barrier.
template <int NT>
__device__ __forceinline__ int window_tile_moments(const mab_tensor& T, int blk, int n_blk, int kcnt, const WindowArgs& a,
                                                   const WindowTileSmem& w, int* s_scan, int* s_pos_off, int* s_val_off) {
    const int t = threadIdx.x;
    const int rows = a.rows;
    const int64_t koff = (int64_t)blk * T.k_block_size_many;
    const int64_t pitch = row_pitch_of(T);
    const uintptr_t I_blk = reinterpret_cast<uintptr_t>(T.I + koff), V_blk = reinterpret_cast<uintptr_t>(T.V + koff);
    const uintptr_t I_lo = reinterpret_cast<uintptr_t>(T.I), I_hi = reinterpret_cast<uintptr_t>(T.I + (int64_t)a.m * pitch);
    const uintptr_t V_lo = reinterpret_cast<uintptr_t>(T.V), V_hi = reinterpret_cast<uintptr_t>(T.V + (int64_t)a.m * pitch);
    const int E = rows * kcnt;
    const uint32_t div_kcnt = kcnt > 1 ? 0xFFFFFFFFu / (uint32_t)kcnt + 1u : 0u;   // i / kcnt == umulhi(i, div_kcnt) while i * kcnt < 2^32
    const int chunks_per_row = w.rstride >> 4;
    MAB_BTICK_DECL
    // 1. stage the window entries: every row's slice of I and of V is copied asynchronously in
    //    16-byte pieces from the 16-byte boundary below its first element; meanwhile clear the
    //    bitmap and the compact moments
    if (t < rows) {
        s_pos_off[t] = (2 * t) * w.rstride + (int)((I_blk + (uintptr_t)t * pitch * 2) & 15);
        s_val_off[t] = (2 * t + 1) * w.rstride + (int)((V_blk + (uintptr_t)t * pitch * 2) & 15);
    }
    for (int ra = t >> 6; ra < rows * 2; ra += NT >> 6) {                         // ra = 2 * row + array; 64 threads per slice
        const int r = ra >> 1;
        const bool isV = ra & 1;
        const uintptr_t seg = (isV ? V_blk : I_blk) + (uintptr_t)r * pitch * 2;
        const uintptr_t seg_end = seg + 2u * kcnt;
        const uintptr_t first = seg & ~(uintptr_t)15;
        const uintptr_t lo = isV ? V_lo : I_lo, hi = isV ? V_hi : I_hi;
        unsigned char* dst_row = w.raw + ra * w.rstride;
        for (int c = t & 63; c < chunks_per_row; c += 64) {
            const uintptr_t src = first + 16u * c;
            if (src < seg_end) {
                unsigned char* dst = dst_row + 16 * c;
                if (src >= lo && src + 16 <= hi) cp_async_16(dst, reinterpret_cast<const void*>(src));
                else                                         // a piece that sticks out of the array: element by element
                    for (int b = 0; b < 16; b += 2)
                        if (src + b >= lo && src + b + 2 <= hi)
                            *reinterpret_cast<uint16_t*>(dst + b) = *reinterpret_cast<const uint16_t*>(src + b);
            }
        }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int i = t; i < WT_WORDS; i += NT) w.bitmap[i] = 0u;
    for (int i = t; i < E; i += NT) w.mv[i] = make_float2(0.0f, 0.0f);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    MAB_BTICK(0);
    // entry i = (row r, column j): its position sits at raw + 2r * rstride + (address of the row's slice & 15) + 2j
    auto pos_ptr = [&](int i) -> uint16_t* {
        const int r = kcnt > 1 ? (int)__umulhi((uint32_t)i, div_kcnt) : i, j = i - r * kcnt;
        return reinterpret_cast<uint16_t*>(w.raw + s_pos_off[r]) + j;
    };
    // 2. mark touched positions (an index outside the block - only a damaged checkpoint can hold one - is
    //    ignored, here and below).  A thread's first entries stay in registers for step 4.
    constexpr int KEEP = NT >= 512 ? WT_KEEP : 1;             // (the 256-thread variants have no registers to spare)
    uint16_t* kept_ptr[KEEP];
    uint32_t kept_pos[KEEP];
#pragma unroll
    for (int it = 0; it < KEEP; ++it) {
        const int i = t + it * NT;
        kept_ptr[it] = pos_ptr(min(i, E - 1));
        kept_pos[it] = i < E ? (uint32_t)*kept_ptr[it] : 0xFFFFFFFFu;
    }
#pragma unroll
    for (int it = 0; it < KEEP; ++it)
        if (kept_pos[it] < (uint32_t)n_blk) atomicOr(&w.bitmap[kept_pos[it] >> 5], 1u << (kept_pos[it] & 31));
    for (int i = t + KEEP * NT; i < E; i += NT) {
        const uint32_t pos = *pos_ptr(i);
        if (pos < (uint32_t)n_blk) atomicOr(&w.bitmap[pos >> 5], 1u << (pos & 31));
    }
    __syncthreads();
    MAB_BTICK(1);
    // 3. number them: prefix[word] = touched positions in words below
    constexpr int WPT = WT_WORDS / NT;
    int cnt[WPT], local = 0;
#pragma unroll
    for (int i = 0; i < WPT; ++i) { cnt[i] = __popc(w.bitmap[t * WPT + i]); local += cnt[i]; }
    int touched;
    int run = block_exclusive_scan(local, s_scan, touched);
#pragma unroll
    for (int i = 0; i < WPT; ++i) { w.prefix[t * WPT + i] = (uint16_t)run; run += cnt[i]; }
    __syncthreads();
    MAB_BTICK(2);
    // 4. positions -> slots (in place), then accumulate row after row
    auto to_slot = [&](uint16_t* pp, uint32_t pos) {
        if (pos < (uint32_t)n_blk) {
            const uint32_t slot = w.prefix[pos >> 5] + __popc(w.bitmap[pos >> 5] & ((1u << (pos & 31)) - 1u));
            *pp = (uint16_t)slot;
            w.spos[slot] = (uint16_t)pos;                    // entries of one position write the same value
        } else {
            *pp = WT_NO_SLOT;
        }
    };
#pragma unroll
    for (int it = 0; it < KEEP; ++it)
        if (kept_pos[it] != 0xFFFFFFFFu) to_slot(kept_ptr[it], kept_pos[it]);
    for (int i = t + KEEP * NT; i < E; i += NT) {
        uint16_t* pp = pos_ptr(i);
        to_slot(pp, *pp);
    }
    __syncthreads();
    MAB_BTICK(3);
    if ((t & ~31) < kcnt) {                                   // whole warps decide, so that every warp meets the barriers in one piece
        if (kcnt <= NT) {
            // one entry per thread and row: the next row's slot and value are fetched before the barrier of the current one
            const bool on = t < kcnt;
            int slot = WT_NO_SLOT;
            uint32_t vbits = 0;
            if (on) {
                slot = reinterpret_cast<const uint16_t*>(w.raw + s_pos_off[0])[t];
                vbits = reinterpret_cast<const uint16_t*>(w.raw + s_val_off[0])[t];
            }
            for (int r = 0; r < rows; ++r) {
                int slot_n = WT_NO_SLOT;
                uint32_t vbits_n = 0;
                if (on && r + 1 < rows) {
                    slot_n = reinterpret_cast<const uint16_t*>(w.raw + s_pos_off[r + 1])[t];
                    vbits_n = reinterpret_cast<const uint16_t*>(w.raw + s_val_off[r + 1])[t];
                }
                if (slot != WT_NO_SLOT) {
                    const float val = __uint_as_float(vbits << 16);
                    float2 acc = w.mv[slot];
                    acc.x = __fadd_rn(acc.x, __fmul_rn(val, a.w1[r]));
                    acc.y = __fadd_rn(acc.y, __fmul_rn(__fmul_rn(val, val), a.w2[r]));
                    w.mv[slot] = acc;
                }
                __syncthreads();
                slot = slot_n; vbits = vbits_n;
            }
        } else {
            for (int r = 0; r < rows; ++r) {
                const uint16_t* slot_r = reinterpret_cast<const uint16_t*>(w.raw + s_pos_off[r]);
                const uint16_t* val_r = reinterpret_cast<const uint16_t*>(w.raw + s_val_off[r]);
                const float w1 = a.w1[r], w2 = a.w2[r];
                for (int j = t; j < kcnt; j += NT) {
                    const int slot = slot_r[j];
                    if (slot == WT_NO_SLOT) continue;
                    const float val = bf16_bits_to_f32(val_r[j]);
                    float2 acc = w.mv[slot];
                    acc.x = __fadd_rn(acc.x, __fmul_rn(val, w1));
                    acc.y = __fadd_rn(acc.y, __fmul_rn(__fmul_rn(val, val), w2));
                    w.mv[slot] = acc;
                }
                __syncthreads();
            }
        }
    } else {
        for (int r = 0; r < rows; ++r) __syncthreads();      // warps beyond the row length only keep the barriers company
    }
    MAB_BTICK(4);
    return touched;
}

template <typename TP, int MODE, int ALPHA, int NT>
__device__ __forceinline__ void window_tile_body(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units,
                                                 int max_k, const WindowArgs& a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_first[WIN_MAX_TENSORS + 1];
    __shared__ int s_scan[36];
    __shared__ int s_pos_off[MAB_MAX_WINDOW], s_val_off[MAB_MAX_WINDOW];   // byte offsets of each row's first position / value in raw
    const int rows = a.rows;
    const WindowTileSmem w(smem_raw, rows, max_k);
    const int t = threadIdx.x;

    for (int i = t; i < n_tensors; i += NT) s_first[i] = tensors[i].first_unit_a;
    if (t == 0) s_first[n_tensors] = total_units;
    __syncthreads();
    const float inv_bc1 = 1.0f / a.bc1, inv_bc2 = 1.0f / a.bc2;
    UpdateProbe pr;
    const bool probing = MODE == MODE_STEP && a.probe != nullptr;

    int ti = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        if (unit >= s_first[ti + 1]) ti = find_tensor(s_first, n_tensors, unit);   // (units ascend: mostly the same tensor as before)
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const int dbs = T.d_block_size, nfull = T.topk_full_blocks_count;
        const int64_t blk_base = (int64_t)blk * dbs;
        const int n_blk = (int)min((int64_t)dbs, T.d - blk_base);
        if (MODE == MODE_STEP) {
            // the next unit's window rows are small and are asked into L2 now
            if (unit + (int)gridDim.x < total_units && (int)threadIdx.x < 2 * rows) {
                const int nu = unit + gridDim.x;
                const int nti = nu < s_first[ti + 1] ? ti : find_tensor(s_first, n_tensors, nu);
                prefetch_window_rows(tensors[nti], nu - s_first[nti], rows, threadIdx.x);
            }
            // this block's parameters travel to L2 while the window is worked on
            prefetch_l2<NT>(reinterpret_cast<uintptr_t>(reinterpret_cast<TP*>(T.param) + blk_base), (int64_t)n_blk * sizeof(TP));
        }
        const int kcnt = (blk < nfull) ? T.k_block_size_many : T.k_block_size_few;
        const bool g_bf16 = (T.grad_dtype == MAB_BF16);

        MAB_BTICK_DECL
        const int touched = window_tile_moments<NT>(T, blk, n_blk, kcnt, a, w, s_scan, s_pos_off, s_val_off);
        MAB_BTICK(9);
        // 5. moments -> update (rounded to the gradient's element type), slot by slot
        for (int s = t; s < touched; s += NT) {
            const float2 acc = w.mv[s];
            const float u = round_as(adam_update_fast(acc.x, acc.y, inv_bc1, inv_bc2, a.eps), g_bf16);
            w.mv[s].x = u;
            if (probing && ALPHA == 0) { pr.sum_u2 = fmaf(u, u, pr.sum_u2); pr.zeros_u -= (u != 0.0f) ? 1 : 0; }   // (the other forms count in the stream)
        }
        if (probing && ALPHA == 0 && t == 0) pr.zeros_u += n_blk;       // every position without a non-zero update is a zero of u
        __syncthreads();
        MAB_BTICK(5);
        if (MODE == MODE_STEP && ALPHA == 0) {
            // 6. without the alpha term only the touched positions get an update: stream the block for the
            //    weight decay alone (nothing to stream without decay), then update the touched elements
            //    one by one; fma(-lr, 0, x) == x, so the untouched elements are already final
            if (T.weight_decay > 0.0) {
                stream_range<TP, MODE, NT, ALPHA>(T, a, NoU{}, blk_base, n_blk, pr);
                __syncthreads();                               // the decayed values are read back below
            }
            MAB_BTICK(6);
            TP* p = reinterpret_cast<TP*>(T.param) + blk_base;
            const float neg_lr = T.neg_lr_f32;
            for (int s2 = t; s2 < touched; s2 += NT) {
                const int pos = w.spos[s2];
                Elem<TP>::store(p, pos, __fmaf_rn(neg_lr, w.mv[s2].x, Elem<TP>::load(p, pos)));
            }
        } else {
            // 6. stream the whole block; each octet finds its updates through the bitmap
            const SparseU src{w.bitmap, w.prefix, w.mv};
            stream_range<TP, MODE, NT, ALPHA>(T, a, src, blk_base, n_blk, pr);
        }
        MAB_BTICK(7);
        __syncthreads();                                       // everything is reused by the next unit
        MAB_BTICK(8);
#ifdef MAB_STATS
        if (threadIdx.x == 0) atomicAdd(&g_stats_b[15], 1ull);
#endif
    }
    if (probing) pr.flush(a.probe);
}

// NT threads per CTA: 256 while four CTAs fit an SM; windows whose arrays leave room for two CTAs or one get 512 or
// 1024 threads instead, so that an SM always has 32 warps to hide the latency of the barrier-separated phases.
template <typename TP, int MODE, int ALPHA, int NT>
__global__ void __launch_bounds__(NT, ALPHA == 0 ? 1024 / NT : 1)
window_tile_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int max_k,
                   const __grid_constant__ WindowArgs a) {
    window_tile_body<TP, MODE, ALPHA, NT>(tensors, n_tensors, total_units, max_k, a);
}

// Single tensor whose descriptor travels as a kernel argument (operator-level entry point).
template <typename TP, int MODE, int ALPHA, int NT>
__global__ void __launch_bounds__(NT)
window_tile_single_kernel(const __grid_constant__ mab_tensor t, int total_units, int max_k,
                          const __grid_constant__ WindowArgs a) {
    window_tile_body<TP, MODE, ALPHA, NT>(&t, 1, total_units, max_k, a);
}

// ------------------------------------------------------------------------------------ resident-tile kernel
//
// The step without the alpha term on bf16 parameters: the block's parameters are walked once.  One
// bulk copy (the 1-D copy engine) brings them into shared memory while the window phases run; the
// weight decay and the updates of the touched positions are applied there, and one bulk copy writes
// the block back while the CTA already works on its next block.  512 threads, two CTAs per SM.
//
// round_bf16(p * decay) == p for every bf16 p when 0 <= 1 - decay <= 2^-10: the product differs from p
// by less than a quarter of the distance to the neighbouring bf16 value, for normal and subnormal p
// alike.  The decay pass is skipped for such a tensor (lr * weight_decay = 1e-4 is the usual case);
// the result is bit for bit the one the pass would produce.

constexpr int WR_THREADS = 512;

// Set when a wait on the copy engine gave up; read through mab_device_error() together with the other kernels' flags.
__device__ int g_copy_timeout_window;

__device__ __forceinline__ bool decay_is_identity_bf16(float decay) {
    return decay <= 1.0f && (1.0f - decay) <= 0.0009765625f;
}

__global__ void __launch_bounds__(WR_THREADS, 2)
window_resident_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int max_k, int tile_bytes,
                       const __grid_constant__ WindowArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];                 // [tile][window arrays]
    __shared__ int s_first[WIN_MAX_TENSORS + 1];
    __shared__ int s_scan[36];
    __shared__ int s_pos_off[MAB_MAX_WINDOW], s_val_off[MAB_MAX_WINDOW];
    __shared__ __align__(8) uint64_t s_bar;
    uint16_t* tile = reinterpret_cast<uint16_t*>(smem_raw);
    uint4* tile4 = reinterpret_cast<uint4*>(smem_raw);
    const int rows = a.rows;
    const WindowTileSmem w(smem_raw + tile_bytes, rows, max_k);
    const int t = threadIdx.x;

    for (int i = t; i < n_tensors; i += WR_THREADS) s_first[i] = tensors[i].first_unit_a;
    if (t == 0) { s_first[n_tensors] = total_units; mbar_init(&s_bar, 1); }
    __syncthreads();
    const float inv_bc1 = 1.0f / a.bc1, inv_bc2 = 1.0f / a.bc2;
    uint32_t parity = 0;
    bool store_in_flight = false;                                               // thread 0 only
    UpdateProbe pr;
    const bool probing = a.probe != nullptr;

    int ti = 0;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        if (unit >= s_first[ti + 1]) ti = find_tensor(s_first, n_tensors, unit);   // (units ascend: mostly the same tensor as before)
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const int dbs = T.d_block_size, nfull = T.topk_full_blocks_count;
        const int64_t blk_base = (int64_t)blk * dbs;
        const int n_blk = (int)min((int64_t)dbs, T.d - blk_base);
        uint16_t* p = reinterpret_cast<uint16_t*>(T.param) + blk_base;
        const bool bulk = (n_blk & 7) == 0 && aligned16(p);                     // the copy engine moves whole 16-byte pieces
        const int n_oct = (n_blk + 7) >> 3;

        MAB_BTICK_DECL
        // the block's parameters start travelling; the previous block's store must have left the tile first
        if (t == 0) {
            if (store_in_flight) { bulk_wait_read(); store_in_flight = false; }
            if (bulk) {
                fence_async_smem();
                mbar_arrive_expect_tx(&s_bar, (uint32_t)n_blk * 2u);
                bulk_g2s(tile, p, (uint32_t)n_blk * 2u, &s_bar);
            }
        }
        if (unit + (int)gridDim.x < total_units && t < 2 * rows) {              // the next unit's window rows: into L2
            const int nu = unit + gridDim.x;
            const int nti = nu < s_first[ti + 1] ? ti : find_tensor(s_first, n_tensors, nu);
            prefetch_window_rows(tensors[nti], nu - s_first[nti], rows, threadIdx.x);
        }
        const int kcnt = (blk < nfull) ? T.k_block_size_many : T.k_block_size_few;
        const bool g_bf16 = (T.grad_dtype == MAB_BF16);
        const int touched = window_tile_moments<WR_THREADS>(T, blk, n_blk, kcnt, a, w, s_scan, s_pos_off, s_val_off);
        MAB_BTICK(9);

        // the tile: wait for the bulk copy, or fetch a ragged block (a tensor's last one, an unaligned slice) with plain loads
        if (bulk) {
            const bool ok = mbar_wait(&s_bar, parity);
            parity ^= 1u;
            if (__syncthreads_or(!ok)) {
                if (t == 0) atomicExch(&g_copy_timeout_window, 1);
                return;
            }
        } else {
            if (t == 0 && store_in_flight) { bulk_wait_read(); store_in_flight = false; }
            __syncthreads();
            for (int i = t; i < n_blk; i += WR_THREADS) tile[i] = p[i];
            __syncthreads();
        }
        MAB_BTICK(5);
        // weight decay over the whole tile, in shared memory
        const float decay = T.decay_f32;
        if (T.weight_decay > 0.0 && !decay_is_identity_bf16(decay)) {
            const float2 decay2 = make_float2(decay, decay);
            for (int o = t; o < n_oct; o += WR_THREADS) {
                const uint4 v = tile4[o];
                const uint32_t in[4] = {v.x, v.y, v.z, v.w};
                uint32_t out[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const float2 x = __fmul2_rn(make_float2(__uint_as_float(in[b] << 16), __uint_as_float(in[b] & 0xFFFF0000u)), decay2);
                    out[b] = cvt_bf16x2_rne(x.x, x.y);
                }
                tile4[o] = make_uint4(out[0], out[1], out[2], out[3]);         // (positions past n_blk of a ragged tile are never stored)
            }
            __syncthreads();
        }
        MAB_BTICK(6);
        // moments -> update (rounded to the gradient's element type) -> parameter, touched positions only:
        // fma(-lr, 0, x) == x, so the untouched elements are already final
        const float neg_lr = T.neg_lr_f32;
        for (int s = t; s < touched; s += WR_THREADS) {
            const float2 acc = w.mv[s];
            const float u = round_as(adam_update_fast(acc.x, acc.y, inv_bc1, inv_bc2, a.eps), g_bf16);
            const int pos = w.spos[s];
            tile[pos] = f32_to_bf16_bits_rne(__fmaf_rn(neg_lr, u, bf16_bits_to_f32(tile[pos])));
            if (probing) { pr.sum_u2 = fmaf(u, u, pr.sum_u2); pr.zeros_u -= (u != 0.0f) ? 1 : 0; }
        }
        if (probing && t == 0) pr.zeros_u += n_blk;                             // every position without a non-zero update is a zero of u
        MAB_BTICK(7);
        // the tile goes back
        if (bulk) {
            fence_async_smem();                                                 // this thread's writes, before the copy engine reads them
            __syncthreads();
            if (t == 0) { bulk_s2g(p, tile, (uint32_t)n_blk * 2u); store_in_flight = true; }
        } else {
            __syncthreads();
            for (int i = t; i < n_blk; i += WR_THREADS) p[i] = tile[i];
            __syncthreads();
        }
        MAB_BTICK(8);
#ifdef MAB_STATS
        if (threadIdx.x == 0) atomicAdd(&g_stats_b[15], 1ull);
#endif
    }
    if (t == 0 && store_in_flight) bulk_wait_all();                            // shared memory must outlive the copy engine's reads
    if (probing) pr.flush(a.probe);
}

// ------------------------------------------------------------------------------------ wide kernel

// TP: element type of `param` (MODE_STEP) or of the output buffer held in `param` (MODE_WRITE_UPDATE).
template <typename TP, int MODE, int ALPHA>
__device__ __forceinline__ void window_wide_body(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units,
                                                 const WindowArgs& a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_first[WIN_MAX_TENSORS + 1];
    WindowSmem sm(smem_raw);
    for (int i = threadIdx.x; i < n_tensors; i += WIN_THREADS) s_first[i] = tensors[i].first_unit_b;
    if (threadIdx.x == 0) s_first[n_tensors] = total_units;
    __syncthreads();
    UpdateProbe pr;

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

        window_to_update(T.I + koff, T.V + koff, row_pitch_of(T), kcnt, s0, len, a, sm);
        if (T.grad_dtype == MAB_BF16) {
            for (int i = threadIdx.x; i < len; i += WIN_THREADS) sm.m_acc[i] = round_as(sm.m_acc[i], true);
            __syncthreads();
        }
        stream_range<TP, MODE, WIN_THREADS, ALPHA>(T, a, DenseU{sm.m_acc}, blk_base + s0, len, pr);
        __syncthreads();   // shared accumulators are reused by the next unit
    }
    if (MODE == MODE_STEP) pr.flush(a.probe);
}

template <typename TP, int MODE, int ALPHA>
__global__ void __launch_bounds__(WIN_THREADS, 2)
window_wide_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, const __grid_constant__ WindowArgs a) {
    window_wide_body<TP, MODE, ALPHA>(tensors, n_tensors, total_units, a);
}

template <typename TP, int MODE, int ALPHA>
__global__ void __launch_bounds__(WIN_THREADS)
window_wide_single_kernel(const __grid_constant__ mab_tensor t, int total_units, const __grid_constant__ WindowArgs a) {
    window_wide_body<TP, MODE, ALPHA>(&t, 1, total_units, a);
}

// ------------------------------------------------------------------------------------ launch

// `single` != nullptr: one tensor passed by value; else n_tensors descriptors in device memory.
// units_tile / units_wide are the unit counts of the two variants; rows * max_k (the largest
// k_block_size of the launch) decides which one runs.
template <typename TP, int MODE, int ALPHA>
static int launch_window_impl(const mab_tensor* dev_tensors, const mab_tensor* single, int n_tensors, int units_tile,
                              int units_wide, int max_k, const WindowArgs& a, cudaStream_t s) {
    const int sms = device_sm_count();
    // the tile variant while its compact arrays fit one CTA's shared memory (next to the kernel's static arrays)
    const int smem_tile = (int64_t)a.rows * max_k <= WT_MAX_ENTRIES ? wt_smem_bytes(a.rows, max_k) : 0;
    if (smem_tile > 0 && smem_tile + 4096 <= device_max_optin_smem()) {
        const int smem = smem_tile;
        const int per_sm = std::max(1, std::min(8, (227 * 1024) / (smem + 3072)));
        const int grid = (int)std::min<int64_t>(units_tile, (int64_t)sms * per_sm);
        // fewer resident CTAs (large windows) get more threads each; the forms with the alpha term keep 256
        const int nt = (ALPHA != 0 || per_sm >= 4) ? 256 : per_sm >= 2 ? 512 : 1024;
        auto run = [&](auto kern_single, auto kern_multi, int threads) -> int {
            if (single) {
                MAB_CUDA_TRY(cudaFuncSetAttribute(kern_single, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
                kern_single<<<grid, threads, smem, s>>>(*single, units_tile, max_k, a);
            } else {
                MAB_CUDA_TRY(cudaFuncSetAttribute(kern_multi, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
                kern_multi<<<grid, threads, smem, s>>>(dev_tensors, n_tensors, units_tile, max_k, a);
            }
            return MAB_OK;
        };
        int rc;
        if constexpr (ALPHA == 0) {
            if (nt == 1024) rc = run(window_tile_single_kernel<TP, MODE, 0, 1024>, window_tile_kernel<TP, MODE, 0, 1024>, 1024);
            else if (nt == 512) rc = run(window_tile_single_kernel<TP, MODE, 0, 512>, window_tile_kernel<TP, MODE, 0, 512>, 512);
            else rc = run(window_tile_single_kernel<TP, MODE, 0, 256>, window_tile_kernel<TP, MODE, 0, 256>, 256);
        } else {
            rc = run(window_tile_single_kernel<TP, MODE, ALPHA, 256>, window_tile_kernel<TP, MODE, ALPHA, 256>, 256);
        }
        if (rc) return rc;
    } else {
        const int grid = (int)std::min<int64_t>(units_wide, (int64_t)sms * 2);
        if (single) {
            auto kern = window_wide_single_kernel<TP, MODE, ALPHA>;
            MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WIN_SMEM_BYTES));
            kern<<<grid, WIN_THREADS, WIN_SMEM_BYTES, s>>>(*single, units_wide, a);
        } else {
            auto kern = window_wide_kernel<TP, MODE, ALPHA>;
            MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, WIN_SMEM_BYTES));
            kern<<<grid, WIN_THREADS, WIN_SMEM_BYTES, s>>>(dev_tensors, n_tensors, units_wide, a);
        }
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "window kernel launch");
    return MAB_OK;
}

// `single` != nullptr: one tensor passed by value; else n_tensors descriptors in device memory.
// units_tile / units_wide are the unit counts of the two variants; rows * max_k (the largest
// k_block_size of the launch) decides which one runs.
template <typename TP, int MODE>
static int launch_window(const mab_tensor* dev_tensors, const mab_tensor* single, int n_tensors, int units_tile,
                         int units_wide, int max_k, const WindowArgs& a, cudaStream_t s) {
    if (MODE == MODE_STEP && a.alpha == -2.0f)
        return launch_window_impl<TP, MODE, 2>(dev_tensors, single, n_tensors, units_tile, units_wide, max_k, a, s);
    if (MODE == MODE_STEP && a.alpha != 0.0f)
        return launch_window_impl<TP, MODE, 1>(dev_tensors, single, n_tensors, units_tile, units_wide, max_k, a, s);
    return launch_window_impl<TP, MODE, 0>(dev_tensors, single, n_tensors, units_tile, units_wide, max_k, a, s);
}

int fill_window_args(WindowArgs& a, int64_t steps, int m, double beta1, double beta2, double eps, float alpha, int qbs) {
    MAB_REQUIRE(steps >= 1, MAB_ERR_BAD_ARG, "steps must be >= 1 (got %lld)", (long long)steps);
    MAB_REQUIRE(m >= 1 && m <= MAB_MAX_WINDOW, MAB_ERR_LIMIT, "m=%d outside [1, %d]", m, MAB_MAX_WINDOW);
    a.rows = (int)std::min<int64_t>(steps, m);
    a.m = m;
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
    a.probe = nullptr;
    return MAB_OK;
}

// Shared memory of one CTA of the resident-tile kernel, or 0 when two such CTAs do not fit an SM.
static int resident_smem_bytes(int rows, int max_k, int max_dbs, int* tile_bytes) {
    *tile_bytes = (max_dbs * 2 + 127) & ~127;
    if ((int64_t)rows * max_k > WT_MAX_ENTRIES) return 0;
    const int smem = *tile_bytes + wt_smem_bytes(rows, max_k);
    const int static_and_reserved = 6 * 1024;                 // the kernel's static arrays + the per-CTA reservation
    return 2 * (smem + static_and_reserved) <= device_max_optin_smem() + 1024 ? smem : 0;
}

int launch_window_step(const mab_tensor* dev_tensors, int n_tensors, int units_tile, int units_wide, int max_k, int max_dbs,
                       int param_dtype, const WindowArgs& a, cudaStream_t s) {
    if (param_dtype == MAB_F32)
        return launch_window<float, MODE_STEP>(dev_tensors, nullptr, n_tensors, units_tile, units_wide, max_k, a, s);
    int tile_bytes = 0;
    const int smem = (a.alpha == 0.0f) ? resident_smem_bytes(a.rows, max_k, max_dbs, &tile_bytes) : 0;
    if (smem > 0) {
        const int grid = (int)std::min<int64_t>(units_tile, (int64_t)device_sm_count() * 2);
        MAB_CUDA_TRY(cudaFuncSetAttribute(window_resident_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        window_resident_kernel<<<grid, WR_THREADS, smem, s>>>(dev_tensors, n_tensors, units_tile, max_k, tile_bytes, a);
        count_launch();
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "window_resident_kernel launch");
        return MAB_OK;
    }
    return launch_window<uint16_t, MODE_STEP>(dev_tensors, nullptr, n_tensors, units_tile, units_wide, max_k, a, s);
}

// The give-up path of the bounded waits, exercised without any fault: the barrier is told to expect
// 16 bytes that no copy delivers, the wait runs out after `probe_limit` probes, and the kernel reports
// it through the same flag and the same early return the step kernels use.
__global__ void wait_selftest_kernel(int probe_limit) {
    __shared__ __align__(8) uint64_t s_bar;
    if (threadIdx.x == 0) mbar_init(&s_bar, 1);
    __syncthreads();
    if (threadIdx.x == 0) mbar_arrive_expect_tx(&s_bar, 16u);
    const bool ok = mbar_wait(&s_bar, 0u, probe_limit);
    if (__syncthreads_or(!ok)) {
        if (threadIdx.x == 0) atomicExch(&g_copy_timeout_window, 1);
        return;
    }
}

int launch_wait_selftest(int probe_limit, cudaStream_t s) {
    wait_selftest_kernel<<<1, 64, 0, s>>>(probe_limit);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "wait_selftest_kernel launch");
}

int copy_timeout_window(int* out, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_copy_timeout_window, sizeof(int));
    if (e == cudaSuccess && clear) { const int z = 0; e = cudaMemcpyToSymbol(g_copy_timeout_window, &z, sizeof(int)); }
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "mab_device_error");
}

int units_b_of(const mab_tensor& t) {
    const int subs = (t.d_block_size + WIN_SR - 1) / WIN_SR;
    const int64_t tail = t.d - (int64_t)t.topk_full_blocks_count * t.d_block_size;
    return t.topk_full_blocks_count * subs + (t.k_block_size_few > 0 ? (int)((tail + WIN_SR - 1) / WIN_SR) : 0);
}

}  // namespace mab

using namespace mab;

#ifdef MAB_STATS
extern "C" int mab_debug_stats_b(unsigned long long* out16, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out16, mab::g_stats_b, sizeof(mab::g_stats_b));
    if (e == cudaSuccess && reset) { unsigned long long z[16] = {0}; e = cudaMemcpyToSymbol(mab::g_stats_b, z, sizeof(z)); }
    return e == cudaSuccess ? 0 : -3;
}
#endif

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
    const int max_k = std::max(t.k_block_size_many, t.k_block_size_few);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == MAB_F32) return launch_window<float, MODE_WRITE_UPDATE>(nullptr, &t, 1, units_tile, units_wide, max_k, a, s);
    return launch_window<uint16_t, MODE_WRITE_UPDATE>(nullptr, &t, 1, units_tile, units_wide, max_k, a, s);
}
