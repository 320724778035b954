// Block-wide exact top-k selection over a tile held in registers.
//
// A tile (one top-k block, at most 32768 elements) is spread over the 1024 threads of a CTA in
// "octets": octet o = j * 1024 + t (j < 4) covers tile elements [8 o, 8 o + 8) and belongs to
// thread t.  The key of an element is its absolute value; key "bits" are the bit pattern of that
// absolute value read as a non-negative int (larger int <=> larger magnitude).  Positions past
// the end of the tile hold 0.0: they are the highest positions, so among equal keys they are
// taken last and, because k never exceeds the tile length, never selected.
//
// The contract is rule 5 of the step: the k largest keys, ties to the lower position, result
// in ascending position.  The k-th largest key T is found exactly; the outcome is delivered as
// a bitmap of the selected positions plus, per 32-position word, the number of selected
// positions before it, from which every consumer derives its ordered output slot.
#pragma once
#include "common.cuh"

namespace mab {

constexpr int SEL_THREADS = 1024;
constexpr int SEL_OCTETS  = 4;
constexpr int SEL_MAX_TILE = SEL_THREADS * SEL_OCTETS * 8;   // 32768 positions
constexpr int SEL_WORDS   = SEL_MAX_TILE / 32;               // 1024 bitmap words, one per thread

struct SelectSmem {
    int      counters[40];            // [0..31] bisection counters, [32] count of keys > T
    int      scan[36];
    uint32_t gt_bm[SEL_WORDS];        // key >  T
    uint32_t tie_bm[SEL_WORDS];       // key == T
    uint32_t sel_bm[SEL_WORDS];       // selected positions
    int      sel_before[SEL_WORDS];   // selected positions in lower words
};

// Number of keys >= thr (key bits) over the whole tile.  `counter` must be zero on entry and is
// left dirty.  A threshold above the bit pattern of infinity compares false everywhere.
__device__ __forceinline__ int block_count_ge(const float (&a)[SEL_OCTETS][8], int thr, int* counter) {
    const float thr_f = __int_as_float(thr);
    int c = 0;
#pragma unroll
    for (int j = 0; j < SEL_OCTETS; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) c += (fabsf(a[j][e]) >= thr_f) ? 1 : 0;
    c = __reduce_add_sync(0xffffffffu, c);
    if (lane_id() == 0 && c) atomicAdd(counter, c);
    __syncthreads();
    return *reinterpret_cast<volatile int*>(counter);
}

// Exact k-th largest key by bisection on the 31 key bits (cost independent of the data).
// Returns T; need_ties = how many keys equal to T are selected.  1 <= k <= tile length.
__device__ __forceinline__ int block_kth_key_bisect(const float (&key)[SEL_OCTETS][8], int k, SelectSmem& sm,
                                                    int& need_ties) {
    if (threadIdx.x < 40) sm.counters[threadIdx.x] = 0;
    __syncthreads();
    int T = 0;
    for (int bit = 30; bit >= 0; --bit) {
        int cand = T | (1 << bit);
        if (block_count_ge(key, cand, &sm.counters[bit]) >= k) T = cand;
    }
    const int n_gt = block_count_ge(key, T + 1, &sm.counters[32]);
    need_ties = k - n_gt;
    return T;
}

// Publishes, for the thread's octets, which positions have key > T and key == T.
__device__ __forceinline__ void publish_masks(const float (&key)[SEL_OCTETS][8], int T, SelectSmem& sm) {
    const float T_f = __int_as_float(T);
    uint8_t* gt = reinterpret_cast<uint8_t*>(sm.gt_bm);
    uint8_t* tie = reinterpret_cast<uint8_t*>(sm.tie_bm);
#pragma unroll
    for (int j = 0; j < SEL_OCTETS; ++j) {
        uint32_t g = 0, q = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            g |= (fabsf(key[j][e]) > T_f) ? (1u << e) : 0u;
            q |= (fabsf(key[j][e]) == T_f) ? (1u << e) : 0u;
        }
        const int o = j * SEL_THREADS + threadIdx.x;
        gt[o] = static_cast<uint8_t>(g);
        tie[o] = static_cast<uint8_t>(q);
    }
}

// From the published masks, builds sel_bm (all keys > T plus the need_ties lowest positions with
// key == T) and sel_before.  Every thread of the 1024 takes part.  Ends with a barrier.
__device__ __forceinline__ void resolve_selection(int need_ties, SelectSmem& sm) {
    __syncthreads();
    const int w = threadIdx.x;
    const uint32_t gw = sm.gt_bm[w];
    int total;
    uint32_t sel = gw;
    if (need_ties > 0) {                                    // uniform: no tie scan when no tie is needed
        uint32_t tw = sm.tie_bm[w];
        const int ties_before = block_exclusive_scan(__popc(tw), sm.scan, total);
        int keep = need_ties - ties_before;
        if (keep <= 0) tw = 0;
        else while (__popc(tw) > keep) tw &= ~(0x80000000u >> __clz(tw));   // drop the highest position
        sel |= tw;
        __syncthreads();
    }
    const int before = block_exclusive_scan(__popc(sel), sm.scan, total);
    sm.sel_bm[w] = sel;
    sm.sel_before[w] = before;
    __syncthreads();
}

// Writes the ascending in-block positions of the selection (int16) to out[0..k).
__device__ __forceinline__ void emit_indices(const SelectSmem& sm, int16_t* out) {
    const int w = threadIdx.x;
    uint32_t sel = sm.sel_bm[w];
    int p = sm.sel_before[w];
    while (sel) {
        const int b = __ffs(sel) - 1;
        sel &= sel - 1;
        out[p++] = static_cast<int16_t>(w * 32 + b);
    }
}

}  // namespace mab
