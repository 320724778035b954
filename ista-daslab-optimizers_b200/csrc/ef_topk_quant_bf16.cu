// Kernel A for bf16 gradients: the tile lives in shared memory, two CTAs per SM.
//
// A bf16 tile (29 056 values) is 58 KB, so two tiles fit one SM.  The tile is staged by the bulk
// copy engine, turned into a = g + Qinv(e) in place, searched, zeroed at the selected positions and
// re-quantised, all in shared memory; registers hold nothing across phases, so a CTA needs only 512
// threads with 64 registers and two CTAs run per SM: one tile's barrier-bound selection overlaps the
// other tile's arithmetic.  A thread owns whole quantisation blocks (64 consecutive values for
// quant_block_size 64), so block statistics need no shuffles and the decode / encode constants are
// computed once per block instead of once per 8 values.
//
// Results are bit-identical to the register-resident kernel in ef_topk_quant.cu (same arithmetic,
// same tie rule); that kernel keeps serving fp32 gradients, whose 116 KB tiles allow one CTA per SM.
#include "common.cuh"
#include "select.cuh"
#include "codec_fast.cuh"
#include "async_copy.cuh"
#include "fused.cuh"

namespace mab {

constexpr int S_NT = 512;
constexpr int S_WPT = SEL_WORDS / S_NT;     // bitmap words per thread
constexpr int S_CAND_CAP = 2048;
constexpr int S_OCT_CAP = 1024;
constexpr int S_MAX_TENSORS = 512;

#ifdef MAB_STATS
__device__ unsigned long long g_stats_c[16];
#define MAB_CTICK(i) do { if (threadIdx.x == 0) { const long long _now = clock64(); atomicAdd(&g_stats_c[i], (unsigned long long)(_now - c_tick)); c_tick = _now; } } while (0)
#define MAB_CTICK_DECL long long c_tick = clock64();
#else
#define MAB_CTICK(i) do { } while (0)
#define MAB_CTICK_DECL
#endif

// Set when a wait on the copy engine gave up; read through mab_device_error() together with the other kernel's flag.
__device__ int g_copy_timeout_bf16;

struct __align__(16) SmemSel {
    uint32_t gt_bm[SEL_WORDS], tie_bm[SEL_WORDS], sel_bm[SEL_WORDS];
    int      sel_before[SEL_WORDS];
    uint32_t cand[S_CAND_CAP];           // candidates as (|value| bits << 16) | (0xFFFF - position): larger is better, all distinct
    uint16_t oct_list[S_OCT_CAP];        // octets that hold a candidate
    int      hist[256];
    uint32_t member[32];
    int      rot[64];
    int      counters[40];
    int      ctrl[8];
    int      scan[36];
    int      n_list, n_cand, kmax;
};

struct BfStage {
    uint16_t* tile; uint32_t* ef; uint16_t* mn; uint16_t* mx;
    __host__ __device__ static int tile_bytes(int elems) { return (elems * 2 + 127) & ~127; }
    __host__ __device__ static int ef_bytes(int elems) { return ((elems >> 1) + 127) & ~127; }
    __host__ __device__ static int st_bytes(int elems, int qshift) { return ((((elems >> qshift) + 4) * 2) + 15) & ~15; }
    __host__ __device__ static int bytes(int elems, int qshift) { return tile_bytes(elems) + ef_bytes(elems) + 2 * st_bytes(elems, qshift); }
    __device__ BfStage(unsigned char* raw, int elems, int qshift) {
        tile = reinterpret_cast<uint16_t*>(raw);
        ef = reinterpret_cast<uint32_t*>(raw + tile_bytes(elems));
        mn = reinterpret_cast<uint16_t*>(raw + tile_bytes(elems) + ef_bytes(elems));
        mx = reinterpret_cast<uint16_t*>(raw + tile_bytes(elems) + ef_bytes(elems) + st_bytes(elems, qshift));
    }
};

__device__ __forceinline__ void unpack8(const uint4& a, float (&v)[8]) {
    v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
    v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
    v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
    v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
}

__device__ __forceinline__ int key_of_bits(uint16_t b) { return (int)(b & 0x7FFFu) << 16; }   // |value| as float key bits

// Number of tile elements with key >= thr (key bits), every thread of the CTA calling.
__device__ __forceinline__ int tile_count_ge(const uint16_t* tile, int n_oct, int thr, int* counter) {
    const float thr_f = __int_as_float(thr);
    int c = 0;
    for (int o = threadIdx.x; o < n_oct; o += S_NT) {
        float v[8];
        unpack8(reinterpret_cast<const uint4*>(tile)[o], v);
#pragma unroll
        for (int e = 0; e < 8; ++e) c += (fabsf(v[e]) >= thr_f) ? 1 : 0;
    }
    c = __reduce_add_sync(0xffffffffu, c);
    if (lane_id() == 0 && c) atomicAdd(counter, c);
    __syncthreads();
    return *reinterpret_cast<volatile int*>(counter);
}

// From gt_bm / tie_bm: sel_bm = gt | (the need_ties lowest tie positions), sel_before = prefix popcount.
// Every thread owns S_WPT consecutive bitmap words.  Starts and ends with a barrier.
__device__ __forceinline__ void resolve_selection_smem(int need_ties, SmemSel& ss) {
    __syncthreads();
    const int w0 = threadIdx.x * S_WPT;
    uint32_t sel[S_WPT];
    int total;
#pragma unroll
    for (int i = 0; i < S_WPT; ++i) sel[i] = ss.gt_bm[w0 + i];
    if (need_ties > 0) {
        uint32_t tw[S_WPT];
        int cnt = 0;
#pragma unroll
        for (int i = 0; i < S_WPT; ++i) { tw[i] = ss.tie_bm[w0 + i]; cnt += __popc(tw[i]); }
        int before = block_exclusive_scan(cnt, ss.scan, total);
#pragma unroll
        for (int i = 0; i < S_WPT; ++i) {
            const int keep = need_ties - before;
            before += __popc(tw[i]);
            if (keep <= 0) tw[i] = 0;
            else while (__popc(tw[i]) > keep) tw[i] &= ~(0x80000000u >> __clz(tw[i]));
            sel[i] |= tw[i];
        }
        __syncthreads();
    }
    int cnt = 0;
#pragma unroll
    for (int i = 0; i < S_WPT; ++i) cnt += __popc(sel[i]);
    int before = block_exclusive_scan(cnt, ss.scan, total);
#pragma unroll
    for (int i = 0; i < S_WPT; ++i) { ss.sel_bm[w0 + i] = sel[i]; ss.sel_before[w0 + i] = before; before += __popc(sel[i]); }
    __syncthreads();
}

// Reserves `cnt` consecutive slots behind *counter for every lane (one atomic per warp); returns the
// lane's first slot.  All 32 lanes must call.
__device__ __forceinline__ int warp_alloc(int cnt, int* counter) {
    int inc = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const int v = __shfl_up_sync(0xffffffffu, inc, d); if (lane_id() >= d) inc += v; }
    int base = 0;
    if (lane_id() == 31 && inc) base = atomicAdd(counter, inc);
    base = __shfl_sync(0xffffffffu, base, 31);
    return base + inc - cnt;
}

// One octet of a = bf16(g + Qinv(e)) in place; returns the largest |a| of the octet.
template <bool FAST>
__device__ __forceinline__ float dequant_octet(uint4* tile4, const uint32_t* ef, int o, const QParams& q, const DecodeConsts& dc) {
    float gv[8], x[8];
    unpack8(tile4[o], gv);
    if (FAST) decode_octet_fast(ef[o], dc, x);
    else decode_octet_exact(ef[o], q, x);
    uint4 out;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float2 s = __fadd2_rn(make_float2(gv[2 * p], gv[2 * p + 1]), make_float2(x[2 * p], x[2 * p + 1]));
        ow[p] = pack_bf16x2_rne(s.x, s.y);
    }
    tile4[o] = out;
    const uint32_t m2 = maxabs_bf16x2(maxabs_bf16x2(ow[0], ow[1]), maxabs_bf16x2(ow[2], ow[3]));
    return fmaxf(fabsf(__uint_as_float(m2 << 16)), fabsf(__uint_as_float(m2 & 0xFFFF0000u)));
}

// QB64: quant_block_size is 64, so a thread's quantisation block is 8 octets and the loops over
// them unroll; tiles that are not whole (a tensor's last block) or not aligned take the general code.
template <bool QB64>
__global__ void __launch_bounds__(S_NT, 2)
ef_topk_quant_bf16_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int qshift, int stage_elems) {
    extern __shared__ __align__(128) unsigned char smem_raw[];       // [staging: tile | codes | statistics][SmemSel]
    __shared__ int s_first[S_MAX_TENSORS + 1];
    __shared__ __align__(8) uint64_t s_bar;
    const BfStage st(smem_raw, stage_elems, qshift);
    SmemSel& ss = *reinterpret_cast<SmemSel*>(smem_raw + BfStage::bytes(stage_elems, qshift));
    const int t = threadIdx.x, lane = lane_id(), warp = warp_id();
    for (int i = t; i < n_tensors; i += S_NT) s_first[i] = tensors[i].first_unit_a;
    if (t == 0) { s_first[n_tensors] = total_units; mbar_init(&s_bar, 1); }
    __syncthreads();
    const int cshift = qshift - 3;              // octets per quantisation block, as a shift
    const int cpq = 1 << cshift;
    uint32_t parity = 0;
    int guess = 0;

    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        const int ti = find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const int dbs = T.d_block_size;
        const int64_t base = (int64_t)blk * dbs;
        const int n = (int)min((int64_t)dbs, T.d - base);
        const int k = (blk < T.topk_full_blocks_count) ? T.k_block_size_many : T.k_block_size_few;
        const uint16_t* g = reinterpret_cast<const uint16_t*>(T.grad) + base;
        const uint8_t* ef_g = T.error + (base >> 1);
        const int64_t qb0 = base >> qshift;
        const int n_oct = (n + 7) >> 3, n_qb = (n + (1 << qshift) - 1) >> qshift;
        const int skip = (int)(qb0 & 1);
        const bool staged = (n & 31) == 0 && (n & ((1 << qshift) - 1)) == 0 && aligned16(g) && aligned16(ef_g) &&
                            ((reinterpret_cast<uintptr_t>(T.min_vals) | reinterpret_cast<uintptr_t>(T.max_vals)) & 3) == 0;

        MAB_CTICK_DECL
        // ---- bring the tile in -------------------------------------------------------------------
        // (selection scratch is cleared here: the barrier that ends the load publishes it)
        if (t == 0) { ss.kmax = 0; ss.n_list = 0; ss.n_cand = 0; }
        if (t < 64) ss.rot[t] = 0;
        if (t < 256) ss.hist[t] = 0;
        for (int w = t; w < SEL_WORDS; w += S_NT) { ss.gt_bm[w] = 0u; ss.tie_bm[w] = 0u; }
        if (staged) {
            if (t == 0) {
                bulk_wait_read();                                     // the previous tile's codes have left shared memory
                fence_async_smem();
                mbar_arrive_expect_tx(&s_bar, (uint32_t)n * 2u + ((uint32_t)n >> 1));
                bulk_g2s(st.tile, g, (uint32_t)n * 2u, &s_bar);
                bulk_g2s(st.ef, ef_g, (uint32_t)n >> 1, &s_bar);
            }
            const int words = ((n_qb + skip) + 1) >> 1;
            const uint32_t* mn_src = reinterpret_cast<const uint32_t*>(T.min_vals + qb0 - skip);
            const uint32_t* mx_src = reinterpret_cast<const uint32_t*>(T.max_vals + qb0 - skip);
            for (int i = t; i < words; i += S_NT) {
                cp_async_4(reinterpret_cast<uint32_t*>(st.mn) + i, mn_src + i);
                cp_async_4(reinterpret_cast<uint32_t*>(st.mx) + i, mx_src + i);
            }
            cp_async_commit();
            cp_async_wait_all();
            const bool ok = mbar_wait(&s_bar, parity);
            parity ^= 1u;
            if (__syncthreads_or(!ok)) {
                if (t == 0) { atomicExch(&g_copy_timeout_bf16, 1); bulk_wait_all(); }
                return;
            }
        } else {
            // ragged tile (a tensor's last block, or unaligned buffers): plain loads, zero padded to whole octets
            if (t == 0) bulk_wait_read();                             // the previous tile's codes have left shared memory
            __syncthreads();
            for (int i = t; i < n_oct * 8; i += S_NT) st.tile[i] = (i < n) ? g[i] : (uint16_t)0;
            for (int i = t; i < n_oct; i += S_NT) {
                uint32_t w = 0;
                for (int b = 0; b < 4; ++b) if ((i * 8 + 2 * b) < n) w |= (uint32_t)ef_g[i * 4 + b] << (8 * b);
                st.ef[i] = w;
            }
            for (int i = t; i < n_qb; i += S_NT) { st.mn[i + skip] = T.min_vals[qb0 + i]; st.mx[i + skip] = T.max_vals[qb0 + i]; }
            __syncthreads();
        }
        MAB_CTICK(0);
        if (unit + (int)gridDim.x < total_units) {           // the tile after this one: into L2 while this one is worked on
            const int nu = unit + gridDim.x;
            const int nti = find_tensor(s_first, n_tensors, nu);
            const mab_tensor& N = tensors[nti];
            const int64_t nbase = (int64_t)(nu - s_first[nti]) * N.d_block_size;
            const int64_t nn = min((int64_t)N.d_block_size, N.d - nbase);
            prefetch_l2<S_NT>(reinterpret_cast<uintptr_t>(reinterpret_cast<const uint16_t*>(N.grad) + nbase), nn * 2);
            prefetch_l2<S_NT>(reinterpret_cast<uintptr_t>(N.error + (nbase >> 1)), (nn + 1) >> 1);
        }
        const uint16_t* s_mn = st.mn + skip;
        const uint16_t* s_mx = st.mx + skip;
        uint4* tile4 = reinterpret_cast<uint4*>(st.tile);

        // ---- a = bf16(g + Qinv(e)) in place; per-octet maxima stay in registers ------------------------
        // register slot i of a thread: block t + (i >> cshift) * S_NT, chunk (i + lane) mod cpq of that block
        float omax[8];
        if (QB64 && staged) {
#pragma unroll
            for (int i = 0; i < 8; ++i) omax[i] = 0.0f;
            if (t < n_qb) {
                const QParams q = qparams(s_mn[t], s_mx[t]);
                const DecodeConsts dc = decode_consts(q);
                if (dc.fast) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) omax[i] = dequant_octet<true>(tile4, st.ef, (t << 3) + ((i + lane) & 7), q, dc);
                } else {
#pragma unroll 1
                    for (int i = 0; i < 8; ++i) {
                        const float m = dequant_octet<false>(tile4, st.ef, (t << 3) + ((i + lane) & 7), q, dc);
#pragma unroll
                        for (int j = 0; j < 8; ++j) if (j == i) omax[j] = m;
                    }
                }
            }
        } else {
            QParams q = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                omax[i] = 0.0f;
                const int b = t + (i >> cshift) * S_NT;
                if (b < n_qb) {
                    if ((i & (cpq - 1)) == 0) q = qparams(s_mn[b], s_mx[b]);
                    const int o = (b << cshift) + ((i + lane) & (cpq - 1));
                    if (o < n_oct) {
                        float gv[8], x[8];
                        unpack8(tile4[o], gv);
                        decode_octet(st.ef[o], q, x);
                        uint4 out;
                        uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
                        uint32_t m2 = 0u;                                     // packed running max of |a|
#pragma unroll
                        for (int p = 0; p < 4; ++p) {
                            const float2 s = __fadd2_rn(make_float2(gv[2 * p], gv[2 * p + 1]), make_float2(x[2 * p], x[2 * p + 1]));
                            uint32_t w = pack_bf16x2_rne(s.x, s.y);
                            if (!staged) {                                    // padding of a ragged tile stays zero
                                const int e0 = o * 8 + 2 * p;
                                if (e0 + 1 >= n) w = (e0 >= n) ? 0u : (w & 0xFFFFu);
                            }
                            ow[p] = w;
                            m2 = max_bf16x2(m2, abs_bf16x2(w));
                        }
                        const float m = fmaxf(__uint_as_float(m2 << 16), __uint_as_float(m2 & 0xFFFF0000u));
                        tile4[o] = out;
                        omax[i] = m;
                    }
                }
            }
        }

        MAB_CTICK(1);
        // ---- exact top-k ---------------------------------------------------------------------------
        {
            float tm = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) tm = fmaxf(tm, omax[i]);
            const int wm = __reduce_max_sync(0xffffffffu, __float_as_int(tm));
            if (lane == 0 && wm) atomicMax(&ss.kmax, wm);
        }
        __syncthreads();
        const int kmax = ss.kmax;
        bool done = false;
        int C = 0;
        uint32_t Tc_sel = 0;
        if (kmax == 0) {
            // every key is zero: the k lowest positions win the ties
            for (int w = t; w < SEL_WORDS; w += S_NT) {
                const int lo = w * 32;
                ss.gt_bm[w] = (lo + 32 <= k) ? 0xFFFFFFFFu : (lo < k ? ((1u << (k - lo)) - 1u) : 0u);
                ss.tie_bm[w] = 0u;
            }
            resolve_selection_smem(0, ss);
            done = true;
            C = -1;                                          // values (all zero) are taken from the tile below
        }
        if (!done && kmax < 0x7f800000 && k <= n_oct) {
            // lower bound of the k-th key on octet maxima: at least k octets reach it, at most ~1.5 k
            const int accept = k + (k >> 1) + 8;
            int lo = 0, hi = kmax + 1, step = 1 << 20;
            int gq = (guess > 0 && guess <= kmax) ? guess : max(1, kmax - (2 << 23));
            bool have_lo = false, have_hi = false;
            for (int it = 0; it < 64; ++it) {
                int mine = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) mine += (__float_as_int(omax[i]) >= gq) ? 1 : 0;
                mine = __reduce_add_sync(0xffffffffu, mine);
                if (lane == 0 && mine) atomicAdd(&ss.rot[it], mine);
                __syncthreads();
                const int c = *reinterpret_cast<volatile int*>(&ss.rot[it]);
                if (c >= k) { lo = gq; have_lo = true; if (c <= accept) break; }
                else { hi = gq; have_hi = true; }
                if (hi - lo <= 1) break;
                if (have_lo && have_hi) gq = lo + ((hi - lo) >> 1);
                else if (have_lo) { gq = (int)min((int64_t)lo + step, (int64_t)hi - 1); step <<= 1; }
                else { gq = (int)max((int64_t)hi - step, (int64_t)1); step <<= 1; }
            }
            guess = lo;
            const int T_lo = have_lo ? lo : 0;
            if (T_lo > 0) {
                const float T_lo_f = __int_as_float(T_lo);
                const uint32_t T16 = ((uint32_t)T_lo + 0xFFFFu) >> 16;          // the bound as a bf16 magnitude
                // 1. octets whose maximum reaches the bound -> list (any order)
                int mine = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) mine += (omax[i] >= T_lo_f) ? 1 : 0;
                int at = warp_alloc(mine, &ss.n_list);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (omax[i] >= T_lo_f) {
                        if (at < S_OCT_CAP) ss.oct_list[at] = (uint16_t)(((t + (i >> cshift) * S_NT) << cshift) + ((i + lane) & (cpq - 1)));
                        ++at;
                    }
                __syncthreads();
                const int n_list = ss.n_list;
                if (n_list <= S_OCT_CAP) {
                    // 2. their values that reach the bound -> candidates (any order)
                    for (int i0 = 0; i0 < n_list; i0 += S_NT) {
                        const int i = i0 + t;
                        uint32_t o = 0, mask = 0;
                        if (i < n_list) {
                            o = ss.oct_list[i];
                            const uint4 v = tile4[o];
                            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                mask |= ((w[p] & 0x7FFFu) >= T16) ? (1u << (2 * p)) : 0u;
                                mask |= (((w[p] >> 16) & 0x7FFFu) >= T16) ? (2u << (2 * p)) : 0u;
                            }
                        }
                        int slot = warp_alloc(__popc(mask), &ss.n_cand);
                        while (mask) {
                            const uint32_t pos = (o << 3) + (__ffs(mask) - 1);
                            mask &= mask - 1;
                            if (slot < S_CAND_CAP) ss.cand[slot] = ((uint32_t)(st.tile[pos] & 0x7FFFu) << 16) | (0xFFFFu - pos);
                            ++slot;
                        }
                    }
                    __syncthreads();
                    C = ss.n_cand;
                    if (C <= S_CAND_CAP) {
                        // 3. one warp finds the k-th largest candidate (the composite values are distinct, so
                        //    there are no ties left to break): 256-bin radix levels over the live range, the
                        //    last <= 32 members ranked directly
                        if (warp == S_NT / 32 - 1) {
                            uint32_t lo_c = T16 << 16, hi_c = ((uint32_t)kmax & 0xFFFF0000u) | 0xFFFFu, Tc = 0;
                            int k_rem = k;
                            for (int level = 0; level < 6; ++level) {
                                const uint32_t W1 = hi_c - lo_c;
                                const int sh = W1 < 256u ? 0 : (32 - __clz(W1)) - 8;
                                if (level > 0) {
#pragma unroll
                                    for (int j = 0; j < 8; ++j) ss.hist[lane * 8 + j] = 0;
                                    __syncwarp();
                                }
                                for (int i = lane; i < C; i += 32) {
                                    const uint32_t c = ss.cand[i];
                                    if (c >= lo_c && c <= hi_c) atomicAdd(&ss.hist[(c - lo_c) >> sh], 1);
                                }
                                __syncwarp();
                                int h[8], sum = 0;
#pragma unroll
                                for (int j = 0; j < 8; ++j) { h[j] = ss.hist[lane * 8 + j]; sum += h[j]; }
                                int suf = sum;
#pragma unroll
                                for (int d = 1; d < 32; d <<= 1) { const int v = __shfl_down_sync(0xffffffffu, suf, d); if (lane + d < 32) suf += v; }
                                const unsigned okm = __ballot_sync(0xffffffffu, suf >= k_rem);
                                const int owner = 31 - __clz(okm);
                                int above = suf - sum, bsel = 7;
#pragma unroll
                                for (int j = 7; j >= 0; --j) if (bsel == j && above + h[j] < k_rem) { above += h[j]; bsel = j - 1; }
                                int hb = 0;
#pragma unroll
                                for (int j = 0; j < 8; ++j) if (j == bsel) hb = h[j];
                                const int b_star = __shfl_sync(0xffffffffu, lane * 8 + bsel, owner);
                                k_rem -= __shfl_sync(0xffffffffu, above, owner);
                                hb = __shfl_sync(0xffffffffu, hb, owner);
                                lo_c += (uint32_t)b_star << sh;
                                hi_c = min(hi_c, lo_c + ((1u << sh) - 1u));
                                if (sh == 0) { Tc = lo_c; break; }
                                if (hb <= 32) {
                                    int base = 0;
                                    for (int i0 = 0; i0 < C; i0 += 32) {
                                        const int i = i0 + lane;
                                        const uint32_t c = i < C ? ss.cand[i] : 0u;
                                        const bool in = c >= lo_c && c <= hi_c;
                                        const unsigned bal = __ballot_sync(0xffffffffu, in);
                                        if (in) ss.member[base + __popc(bal & ((1u << lane) - 1u))] = c;
                                        base += __popc(bal);
                                    }
                                    __syncwarp();
                                    const uint32_t me = lane < base ? ss.member[lane] : 0u;
                                    int greater = 0;
                                    for (int j = 0; j < base; ++j) greater += (__shfl_sync(0xffffffffu, me, j) > me) ? 1 : 0;
                                    const unsigned hit = __ballot_sync(0xffffffffu, lane < base && greater == k_rem - 1);
                                    Tc = __shfl_sync(0xffffffffu, me, __ffs(hit) - 1);
                                    break;
                                }
                            }
                            if (lane == 0) ss.ctrl[3] = (int)Tc;
                        }
                        __syncthreads();
                        Tc_sel = (uint32_t)ss.ctrl[3];
                        // 4. selected positions -> bitmap -> ranks
                        for (int i = t; i < C; i += S_NT) {
                            const uint32_t c = ss.cand[i];
                            if (c >= Tc_sel) { const uint32_t pos = 0xFFFFu - (c & 0xFFFFu); atomicOr(&ss.gt_bm[pos >> 5], 1u << (pos & 31)); }
                        }
                        resolve_selection_smem(0, ss);
                        done = true;
                    }
                }
            }
        }
        MAB_CTICK(2);
        const int64_t row_off = (int64_t)T.ring_index * T.k + (int64_t)blk * T.k_block_size_many;
        int16_t* i_out = T.I + row_off;
        uint16_t* v_out = T.V + row_off;
        if (!done) {
            // general path: bisection on the key bits over the tile in shared memory (data-independent cost)
            C = -1;
            done = true;
            if (t < 40) ss.counters[t] = 0;
            __syncthreads();
            int Tk = 0;
            for (int bit = 30; bit >= 16; --bit) {          // bf16 keys have 16 zero bits below
                const int cand = Tk | (1 << bit);
                if (tile_count_ge(st.tile, n_oct, cand, &ss.counters[bit]) >= k) Tk = cand;
            }
            const int n_gt = tile_count_ge(st.tile, n_oct, Tk + 0x10000, &ss.counters[32]);
            const int need = k - n_gt;
            const float Tf = __int_as_float(Tk);
            uint8_t* gtb = reinterpret_cast<uint8_t*>(ss.gt_bm);
            uint8_t* tieb = reinterpret_cast<uint8_t*>(ss.tie_bm);
            for (int o = t; o < SEL_WORDS * 4; o += S_NT) {
                uint32_t gm = 0, tm = 0;
                if (o < n_oct) {
                    float v[8];
                    unpack8(tile4[o], v);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const bool valid = o * 8 + e < n;     // padding never competes, whatever the threshold
                        gm |= (valid && fabsf(v[e]) > Tf) ? (1u << e) : 0u;
                        tm |= (valid && fabsf(v[e]) == Tf) ? (1u << e) : 0u;
                    }
                }
                gtb[o] = (uint8_t)gm; tieb[o] = (uint8_t)tm;
            }
            resolve_selection_smem(need, ss);
        }

        MAB_CTICK(3);
        // ---- I[row], V[row]; selected positions become 0 in the tile ------------------------------------
        if (C >= 0) {
            for (int i = t; i < C; i += S_NT) {
                const uint32_t c = ss.cand[i];
                if (c >= Tc_sel) {
                    const uint32_t q = 0xFFFFu - (c & 0xFFFFu), w = q >> 5;
                    const int rank = ss.sel_before[w] + __popc(ss.sel_bm[w] & ((1u << (q & 31)) - 1u));
                    i_out[rank] = (int16_t)q;
                    v_out[rank] = st.tile[q];
                    st.tile[q] = 0;
                }
            }
        } else {
            const int w0 = t * S_WPT;
#pragma unroll
            for (int i = 0; i < S_WPT; ++i) {
                uint32_t sel = ss.sel_bm[w0 + i];
                int p = ss.sel_before[w0 + i];
                while (sel) {
                    const int b = __ffs(sel) - 1;
                    sel &= sel - 1;
                    const int q = (w0 + i) * 32 + b;
                    i_out[p] = (int16_t)q;
                    v_out[p++] = st.tile[q];
                    st.tile[q] = 0;
                }
            }
        }
        __syncthreads();

        MAB_CTICK(4);
        // ---- statistics and codes of the residual, one thread per quantisation block --------------------
        uint16_t* mn_out = T.min_vals + qb0;
        uint16_t* mx_out = T.max_vals + qb0;
        if (QB64 && staged) {
            if (t < n_qb) {
                uint32_t hi2 = 0xFF80FF80u, lo2 = 0x7F807F80u;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = tile4[(t << 3) + ((c + lane) & 7)];
                    hi2 = max_bf16x2(max_bf16x2(hi2, v.x), max_bf16x2(max_bf16x2(v.y, v.z), v.w));
                    lo2 = min_bf16x2(min_bf16x2(lo2, v.x), min_bf16x2(min_bf16x2(v.y, v.z), v.w));
                }
                hi2 = max_bf16x2(hi2, hi2 >> 16);
                lo2 = min_bf16x2(lo2, lo2 >> 16);
                const uint16_t mn_b = (uint16_t)(lo2 & 0xFFFFu), mx_b = (uint16_t)(hi2 & 0xFFFFu);
                mn_out[t] = mn_b; mx_out[t] = mx_b;
                const QParams q2 = qparams(mn_b, mx_b);
                const EncodeConsts ec = encode_consts(q2);
                if (ec.fast) {
                    uint32_t redo = 0u;                                   // octets with a value too close to a code boundary
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        const int o = (t << 3) + ((c + lane) & 7);
                        float r[8], worst;
                        unpack8(tile4[o], r);
                        st.ef[o] = encode_octet_speculative<false>(r, ec, worst);   // exact statistics of bf16 values: no clamp needed
                        redo |= (worst > CODEC_SAFE_FRAC) ? (1u << c) : 0u;
                    }
                    while (redo) {
                        const int c = __ffs(redo) - 1;
                        redo &= redo - 1;
                        const int o = (t << 3) + ((c + lane) & 7);
                        float r[8];
                        unpack8(tile4[o], r);
                        st.ef[o] = encode_octet_fast<false>(r, q2, ec);
                    }
                } else {
#pragma unroll 1
                    for (int c = 0; c < 8; ++c) {
                        const int o = (t << 3) + ((c + lane) & 7);
                        float r[8];
                        unpack8(tile4[o], r);
                        st.ef[o] = encode_octet_exact(r, q2, 8);
                    }
                }
            }
        } else
        for (int b = t; b < n_qb; b += S_NT) {
            uint32_t hi2 = 0xFF80FF80u, lo2 = 0x7F807F80u;  // running packed max (from -inf) and min (from +inf)
            const int o_first = b << cshift;
            for (int c = 0; c < cpq; ++c) {
                const int o = o_first + ((c + lane) & (cpq - 1));
                if (o < n_oct) {
                    const uint4 v = tile4[o];
                    const int cnt = n - o * 8;
                    if (cnt >= 8) {
                        hi2 = max_bf16x2(max_bf16x2(hi2, v.x), max_bf16x2(max_bf16x2(v.y, v.z), v.w));
                        lo2 = min_bf16x2(min_bf16x2(lo2, v.x), min_bf16x2(min_bf16x2(v.y, v.z), v.w));
                    } else {                                   // the tensor's last, short octet: valid elements only
                        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                        for (int e = 0; e < cnt; ++e) {
                            const uint32_t x = (w[e >> 1] >> (16 * (e & 1))) & 0xFFFFu;
                            hi2 = max_bf16x2(hi2, x | (x << 16));
                            lo2 = min_bf16x2(lo2, x | (x << 16));
                        }
                    }
                }
            }
            hi2 = max_bf16x2(hi2, hi2 >> 16 | hi2 << 16);
            lo2 = min_bf16x2(lo2, lo2 >> 16 | lo2 << 16);
            const uint16_t mn_b = (uint16_t)(lo2 & 0xFFFFu), mx_b = (uint16_t)(hi2 & 0xFFFFu);
            mn_out[b] = mn_b; mx_out[b] = mx_b;
            const QParams q2 = qparams(mn_b, mx_b);
            for (int c = 0; c < cpq; ++c) {
                const int o = o_first + ((c + lane) & (cpq - 1));
                if (o < n_oct) {
                    float r[8];
                    unpack8(tile4[o], r);
                    const int cnt = n - o * 8;
                    // bf16 values: the statistics are their exact minimum and maximum, no clamp needed
                    st.ef[o] = cnt >= 8 ? encode_octet<false>(r, q2) : encode_octet_exact(r, q2, cnt);
                }
            }
        }
        uint8_t* ef_out = T.error + (base >> 1);
        if (staged) {
            // codes out through the copy engine; the wait sits before the next tile's load
            fence_async_smem();
            __syncthreads();
            MAB_CTICK(5);
            if (t == 0) bulk_s2g(ef_out, st.ef, (uint32_t)n >> 1);
            MAB_CTICK(6);
#ifdef MAB_STATS
            if (threadIdx.x == 0) atomicAdd(&g_stats_c[15], 1ull);
#endif
            continue;
        }
        __syncthreads();
        MAB_CTICK(5);
        // codes out: whole words coalesced, the ragged end byte by byte
        const int full_words = ((reinterpret_cast<uintptr_t>(ef_out) & 3) == 0) ? (n >> 3) : 0;
        for (int i = t; i < full_words; i += S_NT) reinterpret_cast<uint32_t*>(ef_out)[i] = st.ef[i];
        for (int i = full_words + t; i < n_oct; i += S_NT) {
            const uint32_t w = st.ef[i];
            for (int b = 0; b < 4; ++b) if (i * 8 + 2 * b < n) ef_out[i * 4 + b] = (uint8_t)(w >> (8 * b));
        }
        __syncthreads();                                     // the staging area is overwritten by the next tile
        MAB_CTICK(6);
#ifdef MAB_STATS
        if (threadIdx.x == 0) atomicAdd(&g_stats_c[15], 1ull);
#endif
    }
    if (t == 0) bulk_wait_all();
}

int launch_ef_topk_quant_bf16(const mab_tensor* dev_tensors, int n_tensors, int total_units, int qbs, int max_dbs, cudaStream_t s) {
    int qshift = 0;
    while ((1 << qshift) < qbs) ++qshift;
    const int smem = BfStage::bytes(max_dbs, qshift) + (int)sizeof(SmemSel);
    if (2 * (smem + 3 * 1024) > device_max_optin_smem() + 1024) return 1;       // two CTAs per SM do not fit: caller uses the other kernel
    const int grid = (int)std::min<int64_t>(total_units, (int64_t)device_sm_count() * 2);
    if (qshift == 6) {
        MAB_CUDA_TRY(cudaFuncSetAttribute(ef_topk_quant_bf16_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        ef_topk_quant_bf16_kernel<true><<<grid, S_NT, smem, s>>>(dev_tensors, n_tensors, total_units, qshift, max_dbs);
    } else {
        MAB_CUDA_TRY(cudaFuncSetAttribute(ef_topk_quant_bf16_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        ef_topk_quant_bf16_kernel<false><<<grid, S_NT, smem, s>>>(dev_tensors, n_tensors, total_units, qshift, max_dbs);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "ef_topk_quant_bf16_kernel launch");
    return MAB_OK;
}

#ifdef MAB_STATS
}  // namespace mab
extern "C" int mab_debug_stats_c(unsigned long long* out16, int reset) {
    cudaError_t e = cudaMemcpyFromSymbol(out16, mab::g_stats_c, sizeof(mab::g_stats_c));
    if (e == cudaSuccess && reset) { unsigned long long z[16] = {0}; e = cudaMemcpyToSymbol(mab::g_stats_c, z, sizeof(z)); }
    return e == cudaSuccess ? 0 : -3;
}
namespace mab {
#endif

int read_copy_timeout_bf16(int* out) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_copy_timeout_bf16, sizeof(int));
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "mab_device_error");
}

}  // namespace mab
