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
#include "async_copy.cuh"
#include "fused.cuh"

namespace mab {

constexpr int A_MAX_TENSORS = WIN_MAX_TENSORS;   // one limit for every kernel of a fused launch

// a = round_to_grad_dtype(g + x) for an octet.
__device__ __forceinline__ void add_round(const float (&g)[8], const float (&x)[8], float (&a)[8], const float*) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float2 s = __fadd2_rn(make_float2(g[2 * b], g[2 * b + 1]), make_float2(x[2 * b], x[2 * b + 1]));
        a[2 * b] = s.x; a[2 * b + 1] = s.y;
    }
}
__device__ __forceinline__ void add_round(const float (&g)[8], const float (&x)[8], float (&a)[8], const uint16_t*) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float2 s = __fadd2_rn(make_float2(g[2 * b], g[2 * b + 1]), make_float2(x[2 * b], x[2 * b + 1]));
        const uint32_t w = pack_bf16x2_rne(s.x, s.y);
        a[2 * b] = __uint_as_float(w << 16); a[2 * b + 1] = __uint_as_float(w & 0xFFFF0000u);
    }
}

// 8 staged elements in shared memory (16-byte aligned) as floats.
__device__ __forceinline__ void staged_octet(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void staged_octet(const uint16_t* p, float (&v)[8]) {
    const uint4 a = reinterpret_cast<const uint4*>(p)[0];
    v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
    v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
    v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
    v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
}

// 8 elements of the gradient in global memory (read-only path) as floats.
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

// Set when a wait on the copy engine gave up (no launch spins for ever); read by mab_device_error().
__device__ int g_copy_timeout;

// Where a tile lives and whether the copy engine can stage it: whole octets and quantisation
// blocks only, sources aligned for 16-byte bulk copies (4 bytes for the statistics).
template <typename TG>
struct TileRef {
    const TG* g; const uint8_t* ef; const uint16_t* mn; const uint16_t* mx;   // first element / byte / statistic of the tile
    int n, k; bool staged; int stat_skip;                                      // stat_skip: 0/1 entries copied before the tile's first
};

template <typename TG>
__device__ __forceinline__ TileRef<TG> tile_ref(const mab_tensor& T, int blk, int qshift) {
    TileRef<TG> r;
    const int dbs = T.d_block_size;
    const int64_t base = (int64_t)blk * dbs;
    r.n = (int)min((int64_t)dbs, T.d - base);
    r.k = (blk < T.topk_full_blocks_count) ? T.k_block_size_many : T.k_block_size_few;
    r.g = reinterpret_cast<const TG*>(T.grad) + base;
    r.ef = T.error + (base >> 1);
    const int64_t qb0 = base >> qshift;
    r.mn = T.min_vals + qb0;
    r.mx = T.max_vals + qb0;
    r.stat_skip = (int)(qb0 & 1);
    r.staged = (r.n & 31) == 0 && (r.n & ((1 << qshift) - 1)) == 0 && aligned16(r.g) && aligned16(r.ef) &&
               ((reinterpret_cast<uintptr_t>(T.min_vals) | reinterpret_cast<uintptr_t>(T.max_vals)) & 3) == 0;
    return r;
}

// Shared-memory staging area of one tile, carved from the dynamic allocation.
template <typename TG>
struct Stage {
    TG* g; uint32_t* ef; uint16_t* mn; uint16_t* mx;
    __device__ Stage(unsigned char* raw, int stage_elems, int qshift) {
        const int g_bytes = (stage_elems * (int)sizeof(TG) + 127) & ~127;
        const int ef_bytes = ((stage_elems >> 1) + 127) & ~127;
        const int st_bytes = ((((stage_elems >> qshift) + 4) * 2) + 15) & ~15;
        g = reinterpret_cast<TG*>(raw);
        ef = reinterpret_cast<uint32_t*>(raw + g_bytes);
        mn = reinterpret_cast<uint16_t*>(raw + g_bytes + ef_bytes);
        mx = reinterpret_cast<uint16_t*>(raw + g_bytes + ef_bytes + st_bytes);
    }
    __host__ __device__ static int bytes(int stage_elems, int qshift) {
        const int g_bytes = (stage_elems * (int)sizeof(TG) + 127) & ~127;
        const int ef_bytes = ((stage_elems >> 1) + 127) & ~127;
        const int st_bytes = ((((stage_elems >> qshift) + 4) * 2) + 15) & ~15;
        return g_bytes + ef_bytes + 2 * st_bytes;
    }
};

// Starts the copies of a staged tile: one thread arms the barrier and issues the bulk copies of the
// gradient and the codes (one copy each); the statistics (a few hundred bf16) go through cp.async.
template <typename TG, bool WITH_STATS = true>
__device__ __forceinline__ void stage_issue(const TileRef<TG>& r, const Stage<TG>& st, uint64_t* bar, int qshift) {
    if (threadIdx.x == SEL_THREADS - 32) {           // first lane of the last warp: warp 0 has serial work of its own
        const uint32_t gb = (uint32_t)r.n * (uint32_t)sizeof(TG), eb = (uint32_t)r.n >> 1;
        mbar_arrive_expect_tx(bar, gb + eb);
        bulk_g2s(st.g, r.g, gb, bar);
        bulk_g2s(st.ef, r.ef, eb, bar);
    }
    if (!WITH_STATS) return;
    const int words = (((r.n >> qshift) + r.stat_skip) + 1) >> 1;      // 4-byte words covering the tile's statistics
    const uint32_t* mn_src = reinterpret_cast<const uint32_t*>(r.mn - r.stat_skip);
    const uint32_t* mx_src = reinterpret_cast<const uint32_t*>(r.mx - r.stat_skip);
    for (int i = threadIdx.x; i < words; i += SEL_THREADS) {
        cp_async_4(reinterpret_cast<uint32_t*>(st.mn) + i, mn_src + i);
        cp_async_4(reinterpret_cast<uint32_t*>(st.mx) + i, mx_src + i);
    }
    cp_async_commit();
}

// ---- quantisation blocks of any size ("loose": they ignore the borders of the top-k blocks, micro_adam.py:217-231) ----
//
// A quantisation block may then span several tiles, so a tile cannot requantise its residual by itself.  The
// kernel below runs in a second form for that case: the old statistics are read per octet from global memory,
// and instead of statistics + codes it leaves (1) the residual, in the gradient buffer (which the reference
// overwrites in the same step too) and (2) per quantisation block the minimum and maximum of the residual in
// two scratch arrays, as order-preserving unsigned keys merged with atomicMin / atomicMax.  A second kernel
// (requant_loose_kernel) then reads the residual once, rounds the merged statistics to bf16 and writes codes
// and statistics.  Octets never straddle a quantisation block: quant_block_size is a multiple of 8.

template <typename TG>
__device__ __forceinline__ TileRef<TG> tile_ref_loose(const mab_tensor& T, int blk) {
    TileRef<TG> r;
    const int dbs = T.d_block_size;
    const int64_t base = (int64_t)blk * dbs;
    r.n = (int)min((int64_t)dbs, T.d - base);
    r.k = (blk < T.topk_full_blocks_count) ? T.k_block_size_many : T.k_block_size_few;
    r.g = reinterpret_cast<const TG*>(T.grad) + base;
    r.ef = T.error + (base >> 1);
    r.mn = T.min_vals; r.mx = T.max_vals; r.stat_skip = 0;       // statistics are indexed per octet, from the tensor's first
    r.staged = (r.n & 31) == 0 && aligned16(r.g) && aligned16(r.ef);
    return r;
}

template <typename TG>
__device__ __forceinline__ void store_residual_octet(TG* dst, const float (&a)[8], bool vec, int cnt);
template <>
__device__ __forceinline__ void store_residual_octet<float>(float* dst, const float (&a)[8], bool vec, int cnt) {
    if (vec && cnt >= 8) {
        reinterpret_cast<float4*>(dst)[0] = make_float4(a[0], a[1], a[2], a[3]);
        reinterpret_cast<float4*>(dst)[1] = make_float4(a[4], a[5], a[6], a[7]);
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) if (e < cnt) dst[e] = a[e];
    }
}
template <>
__device__ __forceinline__ void store_residual_octet<uint16_t>(uint16_t* dst, const float (&a)[8], bool vec, int cnt) {
    if (vec && cnt >= 8) {                              // the values are bf16 already: the high halves are exact
        uint4 w;
        w.x = (__float_as_uint(a[0]) >> 16) | (__float_as_uint(a[1]) & 0xFFFF0000u);
        w.y = (__float_as_uint(a[2]) >> 16) | (__float_as_uint(a[3]) & 0xFFFF0000u);
        w.z = (__float_as_uint(a[4]) >> 16) | (__float_as_uint(a[5]) & 0xFFFF0000u);
        w.w = (__float_as_uint(a[6]) >> 16) | (__float_as_uint(a[7]) & 0xFFFF0000u);
        *reinterpret_cast<uint4*>(dst) = w;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) if (e < cnt) dst[e] = (uint16_t)(__float_as_uint(a[e]) >> 16);
    }
}

template <typename TG, bool LOOSE>
__global__ void __launch_bounds__(SEL_THREADS, 1)
ef_topk_quant_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int qshift, int stage_elems,
                     LooseArgs la) {
    extern __shared__ __align__(128) unsigned char stage_raw[];      // [staging area | SelectSmem | FastSelSmem]
    SelectSmem& sm = *reinterpret_cast<SelectSmem*>(stage_raw + Stage<TG>::bytes(stage_elems, qshift));
    FastSelSmem& fs = *reinterpret_cast<FastSelSmem*>(stage_raw + Stage<TG>::bytes(stage_elems, qshift) + sizeof(SelectSmem));
    __shared__ int s_first[A_MAX_TENSORS + 1];
    __shared__ __align__(8) uint64_t s_bar;
    __shared__ uint32_t s_qlo[LOOSE ? LOOSE_MAX_QB : 1], s_qhi[LOOSE ? LOOSE_MAX_QB : 1];   // loose: the tile's part of the block statistics
    const bool big_qb = LOOSE && la.qbs >= SEL_MAX_TILE;        // a tile then touches at most two quantisation blocks
    const Stage<TG> st(stage_raw, stage_elems, qshift);
    int guess = 0;                                  // lower bound found for the previous tile, as key bits
    for (int i = threadIdx.x; i < n_tensors; i += SEL_THREADS) s_first[i] = tensors[i].first_unit_a;
    if (threadIdx.x == 0) { s_first[n_tensors] = total_units; mbar_init(&s_bar, 1); }
    __syncthreads();
    const int oshift = qshift - 3;                  // octets per quantisation block, as a shift
    const int lanes_per_qb = 1 << oshift;
    uint32_t parity = 0;

    // prologue: start staging the first tile
    bool cur_staged = false;
    if ((int)blockIdx.x < total_units) {
        const int ti = find_tensor(s_first, n_tensors, blockIdx.x);
        const TileRef<TG> r = LOOSE ? tile_ref_loose<TG>(tensors[ti], blockIdx.x - s_first[ti])
                                    : tile_ref<TG>(tensors[ti], blockIdx.x - s_first[ti], qshift);
        cur_staged = r.staged && r.n <= stage_elems;
        if (cur_staged) stage_issue<TG, !LOOSE>(r, st, &s_bar, qshift);
    }

    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        const int ti = find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const TileRef<TG> tr = LOOSE ? tile_ref_loose<TG>(T, blk) : tile_ref<TG>(T, blk, qshift);
        const int n = tr.n, k = tr.k;
        const int64_t base = (int64_t)blk * T.d_block_size;
        const bool vec_e = (reinterpret_cast<uintptr_t>(tr.ef) & 3) == 0;
        // loose: the tile's first quantisation block and where the tile starts inside it
        const int64_t lqb0 = LOOSE ? base / la.qbs : 0;
        const int lrem0 = LOOSE ? (int)(base - lqb0 * la.qbs) : 0;
        if (LOOSE) {
            for (int i = threadIdx.x; i < LOOSE_MAX_QB; i += SEL_THREADS) { s_qlo[i] = 0xFFFFFFFFu; s_qhi[i] = 0u; }
        }

        MAB_TICK_DECL
        // ---- a = g + Qinv(e), rounded to the gradient's element type ------------------------
        float a[SEL_OCTETS][8];
        float omax[SEL_OCTETS];
        if (cur_staged) {
            cp_async_wait_all();
            const bool ok = mbar_wait(&s_bar, parity);
            parity ^= 1u;
            if (__syncthreads_or(!ok)) {            // the copy engine never delivered: flag it and stop
                if (threadIdx.x == 0) atomicExch(&g_copy_timeout, 1);
                return;
            }
            const int n_oct = n >> 3;
            const uint16_t* s_mn = st.mn + tr.stat_skip;
            const uint16_t* s_mx = st.mx + tr.stat_skip;
#pragma unroll
            for (int j = 0; j < SEL_OCTETS; ++j) {
                const int o = j * SEL_THREADS + (int)threadIdx.x;
                omax[j] = 0.0f;
                if (o < n_oct) {
                    QParams q;
                    if (LOOSE) {
                        const int64_t qb = lqb0 + loose_block(lrem0 + o * 8, la.qbs, big_qb);
                        q = qparams(__ldg(tr.mn + qb), __ldg(tr.mx + qb));
                    } else {
                        q = qparams(s_mn[o >> oshift], s_mx[o >> oshift]);
                    }
                    float gv[8], x[8];
                    staged_octet(st.g + o * 8, gv);
                    decode_octet(st.ef[o], q, x);
                    add_round(gv, x, a[j], static_cast<const TG*>(nullptr));
#pragma unroll
                    for (int e = 0; e < 8; ++e) omax[j] = fmaxf(omax[j], fabsf(a[j][e]));
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[j][e] = 0.0f;
                }
            }
        } else {
            const bool vec_g = aligned16(tr.g);
#pragma unroll
            for (int j = 0; j < SEL_OCTETS; ++j) {
                const int o = j * SEL_THREADS + (int)threadIdx.x;
                const int cnt = n - o * 8;               // >= 8: full octet, 1..7: the tensor's last, <= 0: none
                omax[j] = 0.0f;
                if (cnt > 0) {
                    const int64_t qb = LOOSE ? lqb0 + loose_block(lrem0 + o * 8, la.qbs, big_qb) : (int64_t)(o >> oshift);
                    const QParams q = qparams(tr.mn[qb], tr.mx[qb]);
                    uint32_t w = 0;
                    if (vec_e && cnt >= 8) w = __ldg(reinterpret_cast<const uint32_t*>(tr.ef + o * 4));
                    else {
#pragma unroll
                        for (int b = 0; b < 4; ++b) if (2 * b < cnt) w |= (uint32_t)tr.ef[o * 4 + b] << (8 * b);
                    }
                    float gv[8], x[8];
                    GradOctet<TG>::load(tr.g + o * 8, gv, vec_g && cnt >= 8, cnt);
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
        }
        MAB_TICK(10);
        // the staging area is free again: start on the tile this CTA handles next
        __syncthreads();
        cur_staged = false;
        if (unit + (int)gridDim.x < total_units) {
            const int nu = unit + gridDim.x;
            const int nti = find_tensor(s_first, n_tensors, nu);
            const TileRef<TG> nr = LOOSE ? tile_ref_loose<TG>(tensors[nti], nu - s_first[nti])
                                         : tile_ref<TG>(tensors[nti], nu - s_first[nti], qshift);
            cur_staged = nr.staged && nr.n <= stage_elems;
            if (cur_staged) stage_issue<TG, !LOOSE>(nr, st, &s_bar, qshift);
        }

        MAB_TICK(11);
        // ---- exact top-k ---------------------------------------------------------------------
        const int64_t row_off = (int64_t)T.ring_index * row_pitch_of(T) + (int64_t)blk * T.k_block_size_many;
        uint16_t* v_out = T.V + row_off;
        int n_cand = 0;
        int oct_slot[SEL_OCTETS];
        bool compact_octets;
        const bool fast = fast_select(a, omax, n, k, guess, sm, fs, n_cand, oct_slot, compact_octets, sizeof(TG) == 2 ? 16 : 0);
        if (!fast) {
            int need;
            const int T_key = block_kth_key_bisect(a, k, sm, need);
            publish_masks(a, T_key, sm);
            resolve_selection(need, sm);
        }
        MAB_TICK(12);
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

        MAB_TICK(13);
        // ---- a[I] = 0 (slow path: also V[row]); statistics; e = Q(a) ------------------------------
        uint8_t* ef_out = T.error + (base >> 1);
        uint16_t* mn_out = T.min_vals + (base >> qshift);
        uint16_t* mx_out = T.max_vals + (base >> qshift);
        const uint8_t* sel_bytes = reinterpret_cast<const uint8_t*>(sm.sel_bm);
        int l_cur = -1;                                   // loose: the block whose extremes the thread is collecting
        uint32_t l_lo = 0xFFFFFFFFu, l_hi = 0u;
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            const int o = j * SEL_THREADS + (int)threadIdx.x;
            const int cnt = n - o * 8;
            const uint32_t sel = sel_bytes[o];
            if (fast && compact_octets) {
                if (oct_slot[j] >= 0) {                   // the copy already has the selected elements zeroed
                    const float4 lo4 = reinterpret_cast<const float4*>(fs.oct_val[oct_slot[j]])[0];
                    const float4 hi4 = reinterpret_cast<const float4*>(fs.oct_val[oct_slot[j]])[1];
                    a[j][0] = lo4.x; a[j][1] = lo4.y; a[j][2] = lo4.z; a[j][3] = lo4.w;
                    a[j][4] = hi4.x; a[j][5] = hi4.y; a[j][6] = hi4.z; a[j][7] = hi4.w;
                }
            } else if (fast) {
#pragma unroll
                for (int e = 0; e < 8; ++e) a[j][e] = (sel & (1u << e)) ? 0.0f : a[j][e];
            } else if (sel) {
                const int word = o >> 2;
                int p = sm.sel_before[word] + __popc(sm.sel_bm[word] & ((1u << (8 * (o & 3))) - 1u));
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (sel & (1u << e)) { v_out[p++] = f32_to_bf16_bits_rne(a[j][e]); a[j][e] = 0.0f; }
            }
            if (T.quant_err != nullptr && cnt > 0) {      // alpha == -2: the residual a also goes to the caller's buffer
                TG* qe = reinterpret_cast<TG*>(T.quant_err) + base + o * 8;
                for (int e = 0; e < min(cnt, 8); ++e) Elem<TG>::store(qe, e, a[j][e]);
            }
            float lo = INFINITY, hi = -INFINITY;
            if (cnt >= 8) {
                octet_min_max(a[j], lo, hi);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) if (e < cnt) { lo = fminf(lo, a[j][e]); hi = fmaxf(hi, a[j][e]); }
            }
            if (LOOSE) {
                // the residual goes back to the gradient buffer, its extremes to the tile's entries of the block statistics
                if (cnt > 0) store_residual_octet<TG>(const_cast<TG*>(tr.g) + o * 8, a[j], aligned16(tr.g), cnt);
                if (cnt > 0) {
                    const int qi = loose_block(lrem0 + o * 8, la.qbs, big_qb);
                    if (qi != l_cur) {                                   // hand the collected extremes over when the block changes (blocks longer than a tile: at most once)
                        if (l_cur >= 0) { atomicMin(&s_qlo[l_cur], l_lo); atomicMax(&s_qhi[l_cur], l_hi); }
                        l_cur = qi; l_lo = 0xFFFFFFFFu; l_hi = 0u;
                    }
                    l_lo = min(l_lo, ord_key(lo));
                    l_hi = max(l_hi, ord_key(hi));
                }
                continue;
            }
            // bf16 rounding is monotone and odd, so the block statistics are the lane-wise maximum of the
            // rounded (-min, max) pairs: one packed value and one packed max per shuffle step
            uint32_t st_b = pack_bf16x2_rne(-lo, hi);
            for (int off = 1; off < lanes_per_qb; off <<= 1) st_b = max_bf16x2(st_b, __shfl_xor_sync(0xffffffffu, st_b, off));
            if (cnt > 0) {
                const uint16_t mn_b = (uint16_t)((st_b & 0xFFFFu) ^ 0x8000u), mx_b = (uint16_t)(st_b >> 16);
                if ((o & (lanes_per_qb - 1)) == 0) { mn_out[o >> oshift] = mn_b; mx_out[o >> oshift] = mx_b; }
                const QParams q2 = qparams(mn_b, mx_b);
                if (cnt >= 8) {
                    // the defining form without division instructions (values can lie outside statistics that were
                    // rounded to bf16: the clamped form); the scalar definition where the step is out of its range
                    const uint32_t w = (q2.u >= CODEC_U_MIN && q2.u <= CODEC_U_MAX) ? encode_octet_div_f32<true>(a[j], div_consts(q2))
                                                                                    : encode_octet_exact(a[j], q2, 8);
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
        if (LOOSE) {
            const int c_first = __shfl_sync(0xffffffffu, l_cur, 0);
            if (__all_sync(0xffffffffu, l_cur == c_first)) {             // the whole warp ended in one block (or holds nothing)
                l_lo = __reduce_min_sync(0xffffffffu, l_lo);
                l_hi = __reduce_max_sync(0xffffffffu, l_hi);
                if (lane_id() == 0 && l_cur >= 0) { atomicMin(&s_qlo[l_cur], l_lo); atomicMax(&s_qhi[l_cur], l_hi); }
            } else if (l_cur >= 0) {
                atomicMin(&s_qlo[l_cur], l_lo); atomicMax(&s_qhi[l_cur], l_hi);
            }
        }
        MAB_TICK(14);
        __syncthreads();   // selection scratch is reused by the next unit
        if (LOOSE) {
            const int n_qb = loose_block(lrem0 + n - 1, la.qbs, false) + 1;      // blocks the tile touches
            const int64_t at = la.qb_first[ti] + lqb0;
            for (int i = threadIdx.x; i < n_qb; i += SEL_THREADS) {
                atomicMin(la.st_min + at + i, s_qlo[i]);
                atomicMax(la.st_max + at + i, s_qhi[i]);
            }
            __syncthreads();   // the entries are reset at the start of the next unit
        }
        MAB_TICK(15);
    }
}

int units_a_of(const mab_tensor& t) { return t.topk_full_blocks_count + (t.k_block_size_few > 0 ? 1 : 0); }

int launch_ef_topk_quant(const mab_tensor* dev_tensors, int n_tensors, int total_units, int grad_dtype,
                         int qbs, int max_dbs, cudaStream_t s, const LooseArgs* loose) {
    if (grad_dtype == MAB_BF16) {          // bf16 tiles are small enough for two shared-memory resident CTAs per SM
        const int rc = launch_ef_topk_quant_bf16(dev_tensors, n_tensors, total_units, qbs, max_dbs, s, loose);
        if (rc <= 0) return rc;
    }
    const int grid = (int)std::min<int64_t>(total_units, (int64_t)device_sm_count());
    int qshift = 0;
    if (loose == nullptr) while ((1 << qshift) < qbs) ++qshift;
    else qshift = 6;                                    // only sizes the (unused) statistics area of the staging buffer
    LooseArgs la = {0, nullptr, nullptr, nullptr};
    if (loose) la = *loose;
    // stage whole tiles when they fit beside the kernel's static shared memory, else load directly
    const int scratch = (int)(sizeof(SelectSmem) + sizeof(FastSelSmem));
    const int limit = device_max_optin_smem() - 4 * 1024 - scratch - (loose ? 2 * LOOSE_MAX_QB * 4 : 0);
    auto run = [&](auto kern, int stage_bytes_full) -> int {
        const int stage_elems = stage_bytes_full > limit ? 0 : max_dbs;
        const int smem = (stage_elems ? stage_bytes_full : 0) + scratch;
        MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kern<<<grid, SEL_THREADS, smem, s>>>(dev_tensors, n_tensors, total_units, qshift, stage_elems, la);
        return MAB_OK;
    };
    int rc;
    if (grad_dtype == MAB_F32) {
        const int full = Stage<float>::bytes(max_dbs, qshift);
        rc = loose ? run(ef_topk_quant_kernel<float, true>, full) : run(ef_topk_quant_kernel<float, false>, full);
    } else {
        const int full = Stage<uint16_t>::bytes(max_dbs, qshift);
        rc = loose ? run(ef_topk_quant_kernel<uint16_t, true>, full) : run(ef_topk_quant_kernel<uint16_t, false>, full);
    }
    if (rc) return rc;
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "ef_topk_quant_kernel launch");
    return MAB_OK;
}

int copy_timeout_f32(int* out, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_copy_timeout, sizeof(int));
    if (e == cudaSuccess && clear) { const int z = 0; e = cudaMemcpyToSymbol(g_copy_timeout, &z, sizeof(int)); }
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "mab_device_error");
}

}  // namespace mab

#ifdef MAB_STATS
extern "C" int mab_debug_stats(unsigned long long* out32, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out32, mab::g_stats, sizeof(mab::g_stats));
    if (e == cudaSuccess && reset) { unsigned long long z[32] = {0}; e = cudaMemcpyToSymbol(mab::g_stats, z, sizeof(z)); }
    return e == cudaSuccess ? 0 : -3;
}
#endif
