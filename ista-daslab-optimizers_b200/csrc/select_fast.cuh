// Fast exact top-k for a tile held in registers (layout of select.cuh).
//
// The bisection in select.cuh costs 32 passes over all 32 values of every thread.  Here the
// full-width work is two passes:
//   1. a lower bound T_lo of the k-th largest key is found on per-thread (or per-octet) maxima
//      only: if at least k groups have a maximum >= T_lo, at least k elements do.  The search
//      walks T_lo up until between k and ~1.5 k groups qualify, one barrier per probe, starting
//      from the previous tile's bound;
//   2. the elements >= T_lo ("candidates", typically 1.2-2 k of them) are compacted into shared
//      memory with one block scan.
// The exact k-th key is then found among the candidates alone by a 256-bin radix histogram over
// [T_lo, max], refined until the bin holding the k-th key has at most 32 members, which one warp
// ranks (key descending, position ascending), or until the bin is a single key value, whose
// members are ties resolved by position through the bitmap scan of select.cuh.
// The result is delivered exactly like the slow path's: sel_bm / sel_before in SelectSmem.
// Any tile that does not fit (too many candidates, k larger than the number of groups, ...)
// returns false with no side effect the slow path cares about, and the caller bisects.
#pragma once
#include "common.cuh"
#include "select.cuh"

namespace mab {

#ifdef MAB_STATS
// Development-only tile statistics (compiled in with -DMAB_STATS): [0] fast tiles, [1..6] tiles sent
// to the slow path by reason, [7] lower-bound probes, [8] candidates, [9] histogram levels.
static __device__ unsigned long long g_stats[32];
#define MAB_STAT(i, v) do { if (threadIdx.x == 0) atomicAdd(&g_stats[i], (unsigned long long)(v)); } while (0)
// phase timer: adds the cycles since the previous mark to slot i (thread 0's clock)
#define MAB_TICK(i) do { if (threadIdx.x == 0) { const long long _now = clock64(); atomicAdd(&g_stats[i], (unsigned long long)(_now - g_tick)); g_tick = _now; } } while (0)
#define MAB_TICK_DECL long long g_tick = clock64();
#else
#define MAB_STAT(i, v) do { } while (0)
#define MAB_TICK(i) do { } while (0)
#define MAB_TICK_DECL
#endif

constexpr int FS_CAND_CAP = 4096;
constexpr int FS_OCT_CAP = 1024;          // octets holding a candidate that the compact copy can take
constexpr int FS_OCTET_LEVEL_K = 384;     // above this k the bound is searched on octet maxima

struct __align__(16) FastSelSmem {
    float    oct_val[FS_OCT_CAP][8];      // compact copy of the octets that hold a candidate (k <= FS_OCTET_LEVEL_K)
    float    cand_val[FS_CAND_CAP];       // signed value
    uint16_t cand_pos[FS_CAND_CAP];       // position in the tile; bit 15 set once selected
    uint16_t cand_ref[FS_CAND_CAP];       // 8 * (index in oct_val) + element, when the compact copy is in use
    uint16_t oct_id[FS_OCT_CAP];          // tile octet of each compact octet
    int      n_oct, n_cand;               // compact octets / candidates handed out so far
    int      hist[256];
    int      member[32];                  // candidate indices of the members of the final bin
    int      rot[64];                     // rotating counters of the octet-level probes
    int      ctrl[8];                     // broadcast slots
    int      n_member;
    int      kmax;
};

__device__ __forceinline__ int fs_key(float v) { return __float_as_int(fabsf(v)); }

// Probes on group maxima until count(groups with max >= T_lo) lies in [k, ~1.5 k].  Returns the
// bound as key bits (0 = none found).  `guess` carries the bound of the previous tile.
__device__ __forceinline__ int fs_lower_bound(const float (&omax)[SEL_OCTETS], float tmax, int k, bool octets, int kmax,
                                              int& guess, FastSelSmem& fs) {
    const int ti = __float_as_int(tmax);
    int oi[SEL_OCTETS];
#pragma unroll
    for (int j = 0; j < SEL_OCTETS; ++j) oi[j] = __float_as_int(omax[j]);
    if (octets) {
        if (threadIdx.x < 64) fs.rot[threadIdx.x] = 0;
        __syncthreads();
    }
    const int accept = k + (k >> 1) + 8;
    int lo = 0, hi = kmax + 1;                              // count(lo) >= k (trivially), count(hi) = 0 < k
    int g = (guess > 0 && guess <= kmax) ? guess : max(1, kmax - (2 << 23));
    int step = 1 << 20;
    bool have_lo = false, have_hi = false;
    for (int it = 0; it < 64; ++it) {
        int c;
        if (!octets) {
            c = __syncthreads_count(ti >= g);
        } else {
            int mine = 0;
#pragma unroll
            for (int j = 0; j < SEL_OCTETS; ++j) mine += (oi[j] >= g) ? 1 : 0;
            mine = __reduce_add_sync(0xffffffffu, mine);
            if (lane_id() == 0 && mine) atomicAdd(&fs.rot[it], mine);
            __syncthreads();
            c = *reinterpret_cast<volatile int*>(&fs.rot[it]);
        }
        MAB_STAT(7, 1);
        if (c >= k) { lo = g; have_lo = true; if (c <= accept) break; }
        else { hi = g; have_hi = true; }
        if (hi - lo <= 1) break;
        if (have_lo && have_hi) g = lo + ((hi - lo) >> 1);
        else if (have_lo) { g = (int)min((int64_t)lo + step, (int64_t)hi - 1); step <<= 1; }
        else { g = (int)max((int64_t)hi - step, (int64_t)1); step <<= 1; }
    }
    guess = lo;
    return have_lo ? lo : 0;
}

// Exact selection of the k largest keys among the tile's elements.  On success (true) sm.sel_bm /
// sm.sel_before hold the result, candidates flagged with bit 15 of cand_pos are the selected
// ones, n_cand their number.  Uniform: every thread gets the same return value.
//
// For small k the candidates are gathered in two steps that keep the per-element work off the
// 1024-thread path: octets whose maximum reaches the bound (about one in eight) are copied to a
// compact array in shared memory, one warp-aggregated atomic per warp and octet row, and the
// per-element test then runs over that array only.  In that case `oct_slot[j]` tells the owner of
// octet j where its copy is (-1: none), and on return the selected elements of the copies are
// already zero: the owner reloads its octets from there instead of testing selection bits.
// key_zero_bits = number of low key bits that are always zero (16 when the values are bf16): a
// histogram bin no wider than that holds a single key value, so its members are exact ties.
__device__ __forceinline__ bool fast_select(const float (&a)[SEL_OCTETS][8], const float (&omax)[SEL_OCTETS], int n, int k,
                                            int& guess, SelectSmem& sm, FastSelSmem& fs, int& n_cand,
                                            int (&oct_slot)[SEL_OCTETS], bool& compact_octets, int key_zero_bits) {
    MAB_TICK_DECL
    const int t = threadIdx.x, lane = lane_id(), warp = warp_id();
    float tmax = fmaxf(fmaxf(omax[0], omax[1]), fmaxf(omax[2], omax[3]));

    compact_octets = false;
#pragma unroll
    for (int j = 0; j < SEL_OCTETS; ++j) oct_slot[j] = -1;
    // block maximum key
    if (t == 0) { fs.kmax = 0; fs.n_oct = 0; fs.n_cand = 0; }
    __syncthreads();
    {
        const int wm = __reduce_max_sync(0xffffffffu, __float_as_int(tmax));
        if (lane == 0 && wm) atomicMax(&fs.kmax, wm);
    }
    __syncthreads();
    const int kmax = fs.kmax;
    MAB_TICK(16);
    if (kmax == 0 || kmax >= 0x7f800000) { MAB_STAT(1, 1); return false; }   // all zero, or non-finite values: slow path

    const bool octets = k > FS_OCTET_LEVEL_K;
    const int groups = octets ? (n + 7) / 8 : min(SEL_THREADS, (n + 7) / 8);
    if (k > groups) { MAB_STAT(2, 1); return false; }
    const int T_lo = fs_lower_bound(omax, tmax, k, octets, kmax, guess, fs);
    if (T_lo <= 0) { MAB_STAT(3, 1); return false; }
    const float T_lo_f = __int_as_float(T_lo);
    MAB_TICK(17);

    // ---- compact the candidates --------------------------------------------------------------
    int C = 0;
    bool by_octets = !octets;                                  // small k: through the compact octet copy
    if (by_octets) {
        // slots of the compact copy: one shared-memory atomic per warp reserves a run for its octets (the order of
        // the copy does not matter: everything downstream goes by the positions the entries carry)
        unsigned ball[SEL_OCTETS];
        int tot = 0;
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            ball[j] = __ballot_sync(0xffffffffu, omax[j] >= T_lo_f);
            tot += __popc(ball[j]);
        }
        int run = 0;
        if (lane == 0 && tot) run = atomicAdd(&fs.n_oct, tot);
        run = __shfl_sync(0xffffffffu, run, 0);
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j) {
            if ((ball[j] >> lane) & 1u) {
                const int slot = run + __popc(ball[j] & ((1u << lane) - 1u));
                if (slot < FS_OCT_CAP) {
                    reinterpret_cast<float4*>(fs.oct_val[slot])[0] = make_float4(a[j][0], a[j][1], a[j][2], a[j][3]);
                    reinterpret_cast<float4*>(fs.oct_val[slot])[1] = make_float4(a[j][4], a[j][5], a[j][6], a[j][7]);
                    fs.oct_id[slot] = (uint16_t)(j * SEL_THREADS + t);
                    oct_slot[j] = slot;
                }
            }
            run += __popc(ball[j]);
        }
        __syncthreads();
        const int n_oct = fs.n_oct;
        if (n_oct > FS_OCT_CAP) {                              // uniform: too clustered for the copy, use the registers
            by_octets = false;
#pragma unroll
            for (int j = 0; j < SEL_OCTETS; ++j) oct_slot[j] = -1;
        } else {
            // one compact octet per thread (FS_OCT_CAP <= SEL_THREADS); candidate slots again by one atomic per warp
            uint32_t mask = 0u;
            if (t < n_oct) {
#pragma unroll
                for (int e = 0; e < 8; ++e) mask |= (fabsf(fs.oct_val[t][e]) >= T_lo_f) ? (1u << e) : 0u;
            }
            const int mine = __popc(mask);
            int incl = mine;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += v; }
            int base = 0;
            if (lane == 31 && incl) base = atomicAdd(&fs.n_cand, incl);
            base = __shfl_sync(0xffffffffu, base, 31);
            int at = base + incl - mine;
            if (mine) {
                const uint32_t o = fs.oct_id[t];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    if (mask & (1u << e)) {
                        if (at < FS_CAND_CAP) {
                            fs.cand_val[at] = fs.oct_val[t][e];
                            fs.cand_pos[at] = (uint16_t)((o << 3) | e);
                            fs.cand_ref[at] = (uint16_t)((t << 3) | e);
                        }
                        ++at;
                    }
                }
            }
            __syncthreads();
            C = fs.n_cand;
            if (C > FS_CAND_CAP) { MAB_STAT(4, 1); return false; }
        }
    }
    if (!by_octets) {
        int mine = 0;
#pragma unroll
        for (int j = 0; j < SEL_OCTETS; ++j)
#pragma unroll
            for (int e = 0; e < 8; ++e) mine += (fabsf(a[j][e]) >= T_lo_f) ? 1 : 0;
        int at = block_exclusive_scan(mine, sm.scan, C);
        if (C > FS_CAND_CAP) { MAB_STAT(4, 1); return false; }   // uniform: C is a block-wide value
        if (mine) {
#pragma unroll
            for (int j = 0; j < SEL_OCTETS; ++j)
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (fabsf(a[j][e]) >= T_lo_f) {
                        fs.cand_val[at] = a[j][e];
                        fs.cand_pos[at] = (uint16_t)(((j * SEL_THREADS + t) << 3) | e);
                        ++at;
                    }
        }
    }
    compact_octets = by_octets;
    n_cand = C;
    MAB_TICK(18);
    MAB_STAT(8, C);

    // ---- exact k-th key among the candidates: radix histogram levels ---------------------------
    int r_lo = T_lo, r_hi = kmax, k_rem = k, R = C, sh = 31;
    for (int level = 0; level < 5; ++level) {
        const unsigned W1 = (unsigned)(r_hi - r_lo);          // width - 1
        sh = W1 < 256 ? 0 : (32 - __clz(W1)) - 8;
        if (t < 256) fs.hist[t] = 0;
        __syncthreads();                                       // also orders the candidate writes above
        for (int i = t; i < C; i += SEL_THREADS) {
            const int key = fs_key(fs.cand_val[i]);
            if (key >= r_lo && key <= r_hi) atomicAdd(&fs.hist[(key - r_lo) >> sh], 1);
        }
        __syncthreads();
        if (warp == 0) {
            // suffix sums from the top bin: lane l owns bins [8 l, 8 l + 8)
            int h[8], s = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) { h[i] = fs.hist[lane * 8 + i]; s += h[i]; }
            int suf = s;                                       // inclusive suffix over lanes >= lane
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_down_sync(0xffffffffu, suf, o);
                if (lane + o < 32) suf += v;
            }
            const unsigned ok = __ballot_sync(0xffffffffu, suf >= k_rem);
            const int owner = 31 - __clz(ok);                  // highest lane whose suffix reaches k_rem (ok != 0: total >= k_rem)
            if (lane == owner) {
                int above = suf - s;                           // candidates in bins above this lane's
                int b = 7;
                while (above + h[b] < k_rem) { above += h[b]; --b; }
                fs.ctrl[0] = lane * 8 + b;                     // bin holding the k_rem-th largest
                fs.ctrl[1] = k_rem - above;                    // how many of its members are selected
                fs.ctrl[2] = h[b];
            }
        }
        __syncthreads();
        const int b_star = fs.ctrl[0];
        k_rem = fs.ctrl[1];
        R = fs.ctrl[2];
        const int n_lo = r_lo + (b_star << sh);
        r_hi = (int)min((int64_t)r_hi, (int64_t)n_lo + ((int64_t)1 << sh) - 1);
        r_lo = n_lo;
        MAB_STAT(9, 1);
        if (R <= 32 || sh <= key_zero_bits) break;
    }
    MAB_TICK(19);
    if (R > 32 && sh > key_zero_bits) { MAB_STAT(5, 1); return false; } // cannot happen within 5 levels of 8 bits; stay safe

    // ---- members of the final bin: rank them (<= 32) or treat them as ties of one key -------------
    const bool by_rank = R <= 32;
    if (t == 0) fs.n_member = 0;
    sm.gt_bm[t] = 0u;
    sm.tie_bm[t] = 0u;
    __syncthreads();
    for (int i = t; i < C; i += SEL_THREADS) {
        const int key = fs_key(fs.cand_val[i]);
        const uint32_t pos = fs.cand_pos[i];
        if (key > r_hi) {
            fs.cand_pos[i] = (uint16_t)(pos | 0x8000u);
            atomicOr(&sm.gt_bm[pos >> 5], 1u << (pos & 31));
        } else if (key >= r_lo) {
            if (by_rank) fs.member[atomicAdd(&fs.n_member, 1)] = i;
            else atomicOr(&sm.tie_bm[pos >> 5], 1u << (pos & 31));
        }
    }
    __syncthreads();
    int need_ties = 0;
    if (by_rank) {
        // member w is ranked by warp w: lane l holds member l, one ballot counts who beats member w
        const int nm = fs.n_member;                            // == R <= 32
        if (warp < nm) {
            const int mine_idx = fs.member[warp];
            const int my_key = fs_key(fs.cand_val[mine_idx]);
            const int my_pos = (int)(fs.cand_pos[mine_idx] & 0x7FFFu);   // other warps may set the flag bit meanwhile
            const int idx = lane < nm ? fs.member[lane] : -1;
            const int key = idx >= 0 ? fs_key(fs.cand_val[idx]) : -1;
            const int pos = idx >= 0 ? (int)(fs.cand_pos[idx] & 0x7FFFu) : 0x7fffffff;
            const unsigned beats = __ballot_sync(0xffffffffu, key > my_key || (key == my_key && pos < my_pos));
            if (lane == 0 && __popc(beats) < k_rem) {
                fs.cand_pos[mine_idx] = (uint16_t)(my_pos | 0x8000);
                atomicOr(&sm.gt_bm[my_pos >> 5], 1u << (my_pos & 31));
            }
        }
    } else {
        need_ties = k_rem;                                     // the bin holds one key value: every member has the k-th key
    }
    MAB_TICK(20);
    resolve_selection(need_ties, sm);                          // starts with a barrier
    MAB_TICK(21);
    if (!by_rank) {
        // flag the ties that made it
        for (int i = t; i < C; i += SEL_THREADS) {
            const uint32_t pos = fs.cand_pos[i];
            const int key = fs_key(fs.cand_val[i]);
            if (!(pos & 0x8000u) && key >= r_lo && key <= r_hi && (sm.sel_bm[pos >> 5] >> (pos & 31)) & 1u)
                fs.cand_pos[i] = (uint16_t)(pos | 0x8000u);
        }
        __syncthreads();
    }
    if (by_octets) {
        // the residual of the copied octets: selected elements become 0 (their values stay in cand_val)
        for (int i = t; i < C; i += SEL_THREADS)
            if (fs.cand_pos[i] & 0x8000u) { const uint32_t ref = fs.cand_ref[i]; fs.oct_val[ref >> 3][ref & 7] = 0.0f; }
        __syncthreads();
    }
    MAB_STAT(0, 1);
    if (!by_rank) MAB_STAT(6, 1);
    return true;
}

}  // namespace mab
