// Kernel A for bf16 gradients: the tile lives in shared memory, three CTAs per SM.
//
// A bf16 tile (29 056 values) is 58 KB.  Only the tile and 16 KB of selection scratch sit in shared
// memory (codes and statistics are read from and written to global memory directly, coalesced), so
// three CTAs of 256 threads fit one SM and one tile's latency-bound selection overlaps the other
// tiles' arithmetic.  The tile is staged by the bulk copy engine, turned into a = g + Qinv(e) in
// place, searched, zeroed at the selected positions and re-quantised.
//
// Work is mapped two ways.  Decode and encode walk the tile octet by octet (thread t owns octets
// t, t + 256, ...: consecutive lanes touch consecutive 16-byte pieces of the tile and consecutive
// code words in global memory) and fetch the constants of an octet's quantisation block from a
// small table in shared memory.  Statistics walk it block by block (thread t owns quantisation
// blocks t, t + 256; no shuffles).  For quant_block_size 64 the block tables fit the scratch; other
// block sizes take general per-block code in the same kernel.
//
// Regular tiles (whole blocks of 64, every thread with 14 whole octets, all blocks with a finite
// positive step) take a leaner route: the decode writes a into the tile with the octets of every
// 128-byte row (= one quantisation block) permuted by the row number (octet o sits at o ^ ((o >> 3) & 7)),
// so that afterwards a thread can own whole blocks - consecutive lanes own consecutive blocks and read
// different banks - and computes a block's statistics, its constants and its 32 code bytes from
// registers, with no tables and no shuffles.  The selection addresses the tile through the same
// permutation.  Everything else (other block sizes, ragged tiles, degenerate blocks) keeps the
// linear layout and the general code.
//
// Results are bit-identical to the register-resident kernel in ef_topk_quant.cu (same arithmetic,
// same tie rule); that kernel keeps serving fp32 gradients.
#include "common.cuh"
#include "select.cuh"
#include "codec_fast.cuh"
#include "async_copy.cuh"
#include "fused.cuh"

namespace mab {

constexpr int S_NT = 256;
constexpr int S_CTAS = 3;                    // resident CTAs per SM the shared memory is sized for
constexpr int S_SLOTS = SEL_MAX_TILE / 8 / S_NT;   // octets per thread: 16
constexpr int S_WPT = SEL_WORDS / S_NT;      // bitmap words per thread: 4
constexpr int S_CAND_CAP = 1536;
constexpr int S_WLIST = 128;                 // octets with a candidate, per warp
constexpr int S_QTAB = 512;                  // quantisation blocks whose constants fit the tables
constexpr int S_MAX_TENSORS = WIN_MAX_TENSORS;   // one limit for every kernel of a fused launch
static_assert(S_WPT == 4, "a thread owns four consecutive bitmap words");
static_assert(S_QTAB == 2 * S_NT, "a thread builds the constants of two quantisation blocks");

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
    union {
        uint32_t cand[S_CAND_CAP];       // candidates as (|value| bits << 16) | (0xFFFF - position): larger is better, all distinct
        struct {                         // before and after the selection: constants of each quantisation block
            float2 mu[S_QTAB];           //   (min, u)
            float  r0[S_QTAB];           //   1/u for the encoder, 0 where the defining form must run
        } qt;
    };
    uint32_t sel_bm[SEL_WORDS];          // selected positions
    uint16_t sel_before[SEL_WORDS];      // selected positions in lower words
    uint16_t oct_list[(S_NT / 32) * S_WLIST];
    int      hist[256];
    uint32_t member[32];
    int      rot[64];
    int      counters[40];
    int      ctrl[8];
    int      scan[36];
    int      n_member, n_cand, kmax, pad;
};

__device__ __forceinline__ void unpack8(const uint4& a, float (&v)[8]) {
    v[0] = __uint_as_float(a.x << 16); v[1] = __uint_as_float(a.x & 0xFFFF0000u);
    v[2] = __uint_as_float(a.y << 16); v[3] = __uint_as_float(a.y & 0xFFFF0000u);
    v[4] = __uint_as_float(a.z << 16); v[5] = __uint_as_float(a.z & 0xFFFF0000u);
    v[6] = __uint_as_float(a.w << 16); v[7] = __uint_as_float(a.w & 0xFFFF0000u);
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

// sel_bm = gt | (the need_ties lowest positions of tie), sel_before = prefix popcount, from the
// thread's own four words of both masks.  Starts and ends with a barrier.
__device__ __forceinline__ void resolve_selection_regs(const uint32_t (&gt)[S_WPT], uint32_t (&tw)[S_WPT], int need_ties, SmemSel& ss) {
    __syncthreads();
    const int w0 = threadIdx.x * S_WPT;
    uint32_t sel[S_WPT];
    int total;
#pragma unroll
    for (int i = 0; i < S_WPT; ++i) sel[i] = gt[i];
    if (need_ties > 0) {
        int cnt = 0;
#pragma unroll
        for (int i = 0; i < S_WPT; ++i) cnt += __popc(tw[i]);
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
    for (int i = 0; i < S_WPT; ++i) { ss.sel_bm[w0 + i] = sel[i]; ss.sel_before[w0 + i] = (uint16_t)before; before += __popc(sel[i]); }
    __syncthreads();
}

// The four code bytes of octet o (elements [8 o, 8 o + 8) of a tile of n elements), missing bytes as 0.
__device__ __forceinline__ uint32_t load_code_word(const uint8_t* ef_g, bool aligned4, int o, int n) {
    if (aligned4 && o * 8 + 8 <= n) return reinterpret_cast<const uint32_t*>(ef_g)[o];
    uint32_t w = 0;
    for (int b = 0; b < 4; ++b) if (o * 8 + 2 * b < n) w |= (uint32_t)ef_g[o * 4 + b] << (8 * b);
    return w;
}

__device__ __forceinline__ void store_code_word(uint8_t* ef_g, bool aligned4, int o, int n, uint32_t w) {
    if (aligned4 && o * 8 + 8 <= n) { reinterpret_cast<uint32_t*>(ef_g)[o] = w; return; }
    for (int b = 0; b < 4; ++b) if (o * 8 + 2 * b < n) ef_g[o * 4 + b] = (uint8_t)(w >> (8 * b));
}

// Where octet o of the tile sits: rows of 8 octets are permuted by the row number on regular tiles.
__device__ __forceinline__ int phys_oct(int o, bool swz) { return swz ? (o ^ ((o >> 3) & 7)) : o; }
__device__ __forceinline__ int phys_pos(int pos, bool swz) { return (phys_oct(pos >> 3, swz) << 3) | (pos & 7); }

// Codes of one octet of bf16 values r (statistics = their exact block minimum and maximum, u in
// [2^-100, 2^100]): the defining floor(RN(RN((r - mn) / u) + 0.5)) itself, two elements per instruction and
// without the division and conversion instructions.  The IEEE quotient comes from the correctly rounded
// reciprocal r0 = RN(1 / u): q = RN(d * r0) is within 1.5 ulp of d / u, one residual correction
// q <- RN(q + RN(d - q * u) * r0) (the residual is exact in an FMA) makes it faithful, and a second one
// makes it the correctly rounded quotient (Markstein's theorem on the final step of a division).  Values far
// below half a step, where the residual could underflow, get code 0 from any quotient below 0.5.
// floor: adding 2^23 with rounding down leaves the integer in the low mantissa bits.
__device__ __forceinline__ uint32_t encode_octet_div(const uint4& v, float2 nmn2, float2 r02, float2 nu2) {
    const float2 half2 = make_float2(0.5f, 0.5f), magic2 = make_float2(8388608.0f, 8388608.0f);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t y[8];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float2 r = make_float2(__uint_as_float(w[p] << 16), __uint_as_float(w[p] & 0xFFFF0000u));
        const float2 d = __fadd2_rn(r, nmn2);                               // r - mn
        float2 q = __fmul2_rn(d, r02);
        q = __ffma2_rn(__ffma2_rn(q, nu2, d), r02, q);
        q = __ffma2_rn(__ffma2_rn(q, nu2, d), r02, q);                      // RN(d / u)
        const float2 f = __fadd2_rd(__fadd2_rn(q, half2), magic2);          // 2^23 + floor(q + 0.5)
        y[2 * p] = __float_as_uint(f.x); y[2 * p + 1] = __float_as_uint(f.y);
    }
    // byte 0 of every float is the code; even elements go to the high nibbles
    const uint32_t ev = __byte_perm(__byte_perm(y[0], y[2], 0x0040), __byte_perm(y[4], y[6], 0x0040), 0x5410);
    const uint32_t od = __byte_perm(__byte_perm(y[1], y[3], 0x0040), __byte_perm(y[5], y[7], 0x0040), 0x5410);
    return (ev << 4) | od;
}

constexpr int S_GROUP = 2;                   // octets whose instructions the compiler may interleave (register pressure)
constexpr int S_FULL = 14;                   // 29 056 values = 3632 octets: every thread has 14 whole octets, some a 15th

// One octet of a = bf16(g + Qinv(e)) in place (positions >= n of a ragged tile stay zero); returns the
// largest |a| of the octet.
// RAGGED = false promises a whole octet; `commit` = false computes but leaves the tile as it is.
// The result goes to octet o_out of the tile (o itself, or its permuted place on a regular tile).
template <bool FAST, bool RAGGED>
__device__ __forceinline__ float dequant_octet(uint4* tile4, int o, int o_out, int n, uint32_t codes, const QParams& q, const DecodeConsts& dc, bool commit) {
    float gv[8], x[8];
    unpack8(tile4[o], gv);
    if (FAST) decode_octet_fast(codes, dc, x);
    else decode_octet_exact(codes, q, x);
    uint4 out;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float2 s = __fadd2_rn(make_float2(gv[2 * p], gv[2 * p + 1]), make_float2(x[2 * p], x[2 * p + 1]));
        ow[p] = pack_bf16x2_rne(s.x, s.y);
    }
    if (RAGGED && o * 8 + 8 > n) {                           // the tile's last, short octet
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int e0 = o * 8 + 2 * p;
            if (e0 + 1 >= n) ow[p] = (e0 >= n) ? 0u : (ow[p] & 0xFFFFu);
        }
    }
    if (commit) tile4[o_out] = out;
    const uint32_t m2 = maxabs_bf16x2(maxabs_bf16x2(ow[0], ow[1]), maxabs_bf16x2(ow[2], ow[3]));
    return fmaxf(fabsf(__uint_as_float(m2 << 16)), fabsf(__uint_as_float(m2 & 0xFFFF0000u)));
}

// a = bf16(g + Qinv(e)) in place for the thread's octets t, t + S_NT, ...; per-octet maxima to omax.
// The first FS octets of every thread are promised to exist, to be whole and to find their block in
// the table, so their code is one branch-free block whose octets the compiler can interleave.
// loose_qbs != 0: quantisation blocks of that many elements that ignore the tile's borders; the tile starts
// lrem0 elements into the block mn_g / mx_g point at.
template <int FS>
__device__ __forceinline__ void dequant_phase(uint4* tile4, const SmemSel& ss, bool tables, const uint16_t* mn_g, const uint16_t* mx_g,
                                              int cshift, int n, int n_oct, const uint32_t (&cw)[S_SLOTS], float (&omax)[S_SLOTS],
                                              int loose_qbs = 0, int lrem0 = 0) {
    const int t = threadIdx.x;
    const bool big = loose_qbs >= SEL_MAX_TILE;
    auto block_of = [&](int o) { return loose_qbs ? loose_block(lrem0 + o * 8, loose_qbs, big) : (o >> cshift); };
    uint32_t slow = 0u;                                      // octets whose block needs the defining decode
#pragma unroll
    for (int j = 0; j < S_SLOTS; ++j) {
        omax[j] = 0.0f;
        const int o = t + j * S_NT;
        if (j < FS) {
            if (j % S_GROUP == 0) asm volatile("" ::: "memory");   // octets are interleaved within a group only (register pressure)
            const float2 c = ss.qt.mu[block_of(o)];
            const QParams q = {c.x, c.y};
            const DecodeConsts dc = decode_consts(q);
            const float m = dequant_octet<true, false>(tile4, o, o, n, cw[j], q, dc, dc.fast);
            omax[j] = dc.fast ? m : 0.0f;
            slow |= dc.fast ? 0u : (1u << j);
        } else if (o < n_oct) {
            QParams q;
            const int b = block_of(o);
            if (tables) { const float2 c = ss.qt.mu[b]; q.mn = c.x; q.u = c.y; }
            else q = qparams(mn_g[b], mx_g[b]);
            const DecodeConsts dc = decode_consts(q);
            if (!dc.fast) slow |= 1u << j;
            else omax[j] = dequant_octet<true, true>(tile4, o, o, n, cw[j], q, dc, true);
        }
    }
    if (slow) {
#pragma unroll
        for (int j = 0; j < S_SLOTS; ++j) {
            if ((slow >> j) & 1u) {
                const int o = t + j * S_NT;
                const int b = block_of(o);
                const QParams q = qparams(mn_g[b], mx_g[b]);
                omax[j] = dequant_octet<false, true>(tile4, o, o, n, cw[j], q, decode_consts(q), true);
            }
        }
    }
}

// The same on a regular tile (see the head of the file): every block's decode is the fast one, the
// first S_FULL octets of every thread exist, and octet o is written to its permuted place.  The 8
// lanes that hold a 128-byte row read it in one instruction and write it in a later one, so the
// permutation inside the row happens in place.
__device__ __forceinline__ void dequant_phase_regular(uint4* tile4, const SmemSel& ss, int n_oct, const uint32_t (&cw)[S_SLOTS], float (&omax)[S_SLOTS]) {
    const int t = threadIdx.x;
    const int t_out = t ^ ((t >> 3) & 7);                   // phys_oct(t + j * S_NT) = t_out + j * S_NT
#pragma unroll
    for (int j = 0; j < S_SLOTS; ++j) {
        omax[j] = 0.0f;
        const int o = t + j * S_NT;
        if (j < S_FULL || o < n_oct) {
            if (j < S_FULL && j % S_GROUP == 0) asm volatile("" ::: "memory");
            const float2 c = ss.qt.mu[o >> 3];
            const QParams q = {c.x, c.y};
            omax[j] = dequant_octet<true, false>(tile4, o, t_out + j * S_NT, 0, cw[j], q, decode_consts(q), true);
        }
    }
}

// Codes of one block of a regular tile with the scalar form of the quantiser: the rare blocks whose step is
// zero (all values equal), subnormal or infinite.  Kept out of line so that the common path stays small.
__device__ __noinline__ void encode_block_exact(const uint4* row, int key, uint16_t mn_b, uint16_t mx_b, uint8_t* dst) {
    const QParams q2 = qparams(mn_b, mx_b);
    for (int c = 0; c < 8; ++c) {
        float r[8];
        unpack8(row[c ^ key], r);
        reinterpret_cast<uint32_t*>(dst)[c] = encode_octet_exact(r, q2, 8);
    }
}

// Statistics and codes of the residual on a regular tile: thread t owns blocks t, t + S_NT, ...; a
// block is one 128-byte row of the tile whose octet c sits at c ^ (row & 7), and row & 7 = t & 7.
// Writes the block's bf16 minimum / maximum and its 32 code bytes (ef_out is 4-byte aligned).
__device__ __forceinline__ void stats_encode_regular(const uint4* tile4, int n_qb, uint16_t* mn_out, uint16_t* mx_out, uint8_t* ef_out, bool ef_al16) {
    const int t = threadIdx.x;
    const int key = t & 7;
    for (int b = t; b < n_qb; b += S_NT) {
        const uint4* row = tile4 + (b << 3);
        uint32_t hi2 = 0xFF80FF80u, lo2 = 0x7F807F80u;      // running packed max (from -inf) and min (from +inf)
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint4 v = row[c ^ key];
            hi2 = max_bf16x2(max_bf16x2(hi2, v.x), max_bf16x2(max_bf16x2(v.y, v.z), v.w));
            lo2 = min_bf16x2(min_bf16x2(lo2, v.x), min_bf16x2(min_bf16x2(v.y, v.z), v.w));
        }
        hi2 = max_bf16x2(hi2, hi2 >> 16);
        lo2 = min_bf16x2(lo2, lo2 >> 16);
        const uint16_t mn_b = (uint16_t)(lo2 & 0xFFFFu), mx_b = (uint16_t)(hi2 & 0xFFFFu);
        mn_out[b] = mn_b; mx_out[b] = mx_b;
        const QParams q2 = qparams(mn_b, mx_b);
        uint8_t* dst = ef_out + ((size_t)b << 5);
        if (!(q2.u >= CODEC_U_MIN && q2.u <= CODEC_U_MAX)) {   // all-equal block (u == 0), subnormal or infinite step
            encode_block_exact(row, key, mn_b, mx_b, dst);
            continue;
        }
        const float r0 = rcp_rn_normal(q2.u);
        const float2 nmn2 = make_float2(-q2.mn, -q2.mn), r02 = make_float2(r0, r0), nu2 = make_float2(-q2.u, -q2.u);
        uint4 lo4, hi4;
        lo4.x = encode_octet_div(row[0 ^ key], nmn2, r02, nu2);
        lo4.y = encode_octet_div(row[1 ^ key], nmn2, r02, nu2);
        lo4.z = encode_octet_div(row[2 ^ key], nmn2, r02, nu2);
        lo4.w = encode_octet_div(row[3 ^ key], nmn2, r02, nu2);
        hi4.x = encode_octet_div(row[4 ^ key], nmn2, r02, nu2);
        hi4.y = encode_octet_div(row[5 ^ key], nmn2, r02, nu2);
        hi4.z = encode_octet_div(row[6 ^ key], nmn2, r02, nu2);
        hi4.w = encode_octet_div(row[7 ^ key], nmn2, r02, nu2);
        if (ef_al16) {
            reinterpret_cast<uint4*>(dst)[0] = lo4;
            reinterpret_cast<uint4*>(dst)[1] = hi4;
        } else {
            uint32_t* d32 = reinterpret_cast<uint32_t*>(dst);
            d32[0] = lo4.x; d32[1] = lo4.y; d32[2] = lo4.z; d32[3] = lo4.w;
            d32[4] = hi4.x; d32[5] = hi4.y; d32[6] = hi4.z; d32[7] = hi4.w;
        }
    }
}

// Codes of the thread's octets from the block tables, written to global memory; octets that came too
// close to a code boundary (or whose block is degenerate) are left to the caller in `redo`.  The
// first FS octets of every thread are promised to exist, to be whole and their code words aligned.
template <int FS>
__device__ __forceinline__ void encode_phase(const uint4* tile4, const SmemSel& ss, uint8_t* ef_out, bool ef_al4, int n, int n_oct, uint32_t& redo) {
    const int t = threadIdx.x;
#pragma unroll
    for (int j = 0; j < S_SLOTS; ++j) {
        const int o = t + j * S_NT;
        if (j < FS || o < n_oct) {
            if (j < FS && j % S_GROUP == 0) asm volatile("" ::: "memory");
            const float2 mu = ss.qt.mu[o >> 3];
            const float r0 = ss.qt.r0[o >> 3];
            EncodeConsts ec;
            ec.nmn2 = make_float2(-mu.x, -mu.x); ec.r02 = make_float2(r0, r0); ec.fast = true;
            float r[8], worst;
            unpack8(tile4[o], r);
            const uint32_t w = encode_octet_speculative<false>(r, ec, worst);   // exact statistics of bf16 values: no clamp needed
            const bool ok = worst <= CODEC_SAFE_FRAC && r0 != 0.0f;
            if (j < FS) { if (ok) reinterpret_cast<uint32_t*>(ef_out)[o] = w; }
            else if (ok) store_code_word(ef_out, ef_al4, o, n, w);
            redo |= ok ? 0u : (1u << j);
        }
    }
}

// QB64: quant_block_size is 64: the per-block constants fit the shared-memory tables and the loops
// over a block's 8 octets unroll.
// LOOSE: quantisation blocks of la.qbs elements that ignore the borders of the top-k blocks; the kernel then ends
// a tile with the residual written back to the gradient buffer and the extremes of every block it touches merged
// into la.st_min / la.st_max (requant_loose.cu finishes the job), instead of statistics and codes.
template <bool QB64, bool LOOSE>
__global__ void __launch_bounds__(S_NT, S_CTAS)
ef_topk_quant_bf16_kernel(const mab_tensor* __restrict__ tensors, int n_tensors, int total_units, int qshift, int stage_elems,
                          LooseArgs la) {
    extern __shared__ __align__(128) unsigned char smem_raw[];       // [tile][SmemSel]
    __shared__ int s_first[S_MAX_TENSORS + 1];
    __shared__ __align__(8) uint64_t s_bar;
    uint16_t* tile = reinterpret_cast<uint16_t*>(smem_raw);
    uint4* tile4 = reinterpret_cast<uint4*>(smem_raw);
    SmemSel& ss = *reinterpret_cast<SmemSel*>(smem_raw + ((stage_elems * 2 + 127) & ~127));
    const int t = threadIdx.x, lane = lane_id(), warp = warp_id();
    for (int i = t; i < n_tensors; i += S_NT) s_first[i] = tensors[i].first_unit_a;
    if (t == 0) { s_first[n_tensors] = total_units; mbar_init(&s_bar, 1); ss.ctrl[5] = 0; ss.ctrl[6] = 0; }
    __syncthreads();
    const int cshift = qshift - 3;              // octets per quantisation block, as a shift
    const int cpq = 1 << cshift;
    uint32_t parity = 0;
    int guess = 0;
    int tile_no = 0;                            // tiles this CTA has worked on: selects one of two "a block needs the slow decode" flags
    int ti_next = -1;                           // tensor of the next unit, found while prefetching it
    const uint16_t* g_next = nullptr;           // ... and its gradient tile, so that its copy can start before its descriptor is read again
    int n_next = 0;

    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        bool issued = false;
        if (t == 0 && g_next != nullptr && (n_next & 7) == 0 && aligned16(g_next)) {   // same test as `staged` below
            fence_async_smem();
            mbar_arrive_expect_tx(&s_bar, (uint32_t)n_next * 2u);
            bulk_g2s(smem_raw, g_next, (uint32_t)n_next * 2u, &s_bar);
            issued = true;
        }
        const int ti = ti_next >= 0 ? ti_next : find_tensor(s_first, n_tensors, unit);
        const mab_tensor& T = tensors[ti];
        const int blk = unit - s_first[ti];
        const int dbs = T.d_block_size;
        const int64_t base = (int64_t)blk * dbs;
        const int n = (int)min((int64_t)dbs, T.d - base);
        const int k = (blk < T.topk_full_blocks_count) ? T.k_block_size_many : T.k_block_size_few;
        const uint16_t* g = reinterpret_cast<const uint16_t*>(T.grad) + base;
        const uint8_t* ef_in = T.error + (base >> 1);
        uint8_t* ef_out = T.error + (base >> 1);
        const int64_t qb0 = LOOSE ? base / la.qbs : base >> qshift;
        const int lrem0 = LOOSE ? (int)(base - qb0 * la.qbs) : 0;   // loose: where the tile starts inside its first block
        // quantisation blocks of the tile; loose ones are at least 72 elements long, so the tables hold those a tile touches
        const int n_oct = (n + 7) >> 3;
        const int n_qb = LOOSE ? loose_block(lrem0 + n - 1, la.qbs, false) + 1 : (n + (1 << qshift) - 1) >> qshift;
        const bool staged = (n & 7) == 0 && aligned16(g);            // the bulk copy moves whole 16-byte pieces
        const bool ef_al4 = (reinterpret_cast<uintptr_t>(ef_in) & 3) == 0;
        const bool tables = (QB64 || LOOSE) && n_qb <= S_QTAB;
        const uint16_t* mn_g = T.min_vals + qb0;
        const uint16_t* mx_g = T.max_vals + qb0;
        const int64_t row_off = (int64_t)T.ring_index * row_pitch_of(T) + (int64_t)blk * T.k_block_size_many;
        int16_t* i_out = T.I + row_off;                      // (read here, with the rest of the descriptor, not after the selection)
        uint16_t* v_out = T.V + row_off;

        MAB_CTICK_DECL
        // ---- bring the tile in; meanwhile codes -> registers, decode constants -> table ---------------------
        // (selection scratch is cleared here: the barrier that ends the load publishes it)
        const int slow_slot = 5 + (tile_no & 1);             // set during this tile's load; the other one is cleared for the next tile
        ++tile_no;
        if (t == 0) { ss.kmax = 0; ss.n_member = 0; ss.n_cand = 0; ss.ctrl[4] = 0; ss.ctrl[slow_slot ^ 3] = 0; }
        if (t < 64) ss.rot[t] = 0;
        ss.hist[t] = 0;
        reinterpret_cast<uint4*>(ss.sel_bm)[t] = make_uint4(0u, 0u, 0u, 0u);
        if (staged) {
            if (t == 0 && !issued) {
                fence_async_smem();
                mbar_arrive_expect_tx(&s_bar, (uint32_t)n * 2u);
                bulk_g2s(tile, g, (uint32_t)n * 2u, &s_bar);
            }
        } else {
            // ragged tile (a tensor's last block, or an unaligned buffer): plain loads, zero padded to whole octets
            for (int i = t; i < n_oct * 8; i += S_NT) tile[i] = (i < n) ? g[i] : (uint16_t)0;
        }
        uint32_t cw[S_SLOTS];
        if (ef_al4 && (n & 7) == 0 && n_oct >= S_FULL * S_NT) {  // a full tile: the first S_FULL words of every thread exist and are whole
#pragma unroll
            for (int j = 0; j < S_SLOTS; ++j) {
                const int o = t + j * S_NT;
                cw[j] = (j < S_FULL || o < n_oct) ? reinterpret_cast<const uint32_t*>(ef_in)[o] : 0u;
            }
        } else {
#pragma unroll
            for (int j = 0; j < S_SLOTS; ++j) {
                const int o = t + j * S_NT;
                cw[j] = (o < n_oct) ? load_code_word(ef_in, ef_al4, o, n) : 0u;
            }
        }
        if (tables) {                                        // S_QTAB = 2 * S_NT: a thread's two blocks, their loads issued together
            const int b0 = t, b1 = t + S_NT;
            const uint16_t mn0 = b0 < n_qb ? mn_g[b0] : (uint16_t)0, mx0 = b0 < n_qb ? mx_g[b0] : (uint16_t)0;
            const uint16_t mn1 = b1 < n_qb ? mn_g[b1] : (uint16_t)0, mx1 = b1 < n_qb ? mx_g[b1] : (uint16_t)0;
            bool slow = false;
            if (b0 < n_qb) { const QParams q = qparams(mn0, mx0); ss.qt.mu[b0] = make_float2(q.mn, q.u); slow |= !decode_consts(q).fast; }
            if (b1 < n_qb) { const QParams q = qparams(mn1, mx1); ss.qt.mu[b1] = make_float2(q.mn, q.u); slow |= !decode_consts(q).fast; }
            if (slow) ss.ctrl[slow_slot] = 1;
        }
        if (staged) {
            const bool ok = mbar_wait(&s_bar, parity);
            parity ^= 1u;
            if (__syncthreads_or(!ok)) {
                if (t == 0) atomicExch(&g_copy_timeout_bf16, 1);
                return;
            }
        } else {
            __syncthreads();
        }
        MAB_CTICK(0);
        if (unit + (int)gridDim.x < total_units) {           // the tile after this one: into L2 while this one is worked on
            const int nu = unit + gridDim.x;
            const int nti = find_tensor(s_first, n_tensors, nu);
            ti_next = nti;
            const mab_tensor& N = tensors[nti];
            const int64_t nbase = (int64_t)(nu - s_first[nti]) * N.d_block_size;
            const int64_t nn = min((int64_t)N.d_block_size, N.d - nbase);
            g_next = reinterpret_cast<const uint16_t*>(N.grad) + nbase;
            n_next = (int)nn;
            // gradients: 128-byte lines over all threads; codes and statistics: a warp each (they are 4 and 64 times smaller)
            prefetch_l2<S_NT>(reinterpret_cast<uintptr_t>(reinterpret_cast<const uint16_t*>(N.grad) + nbase), nn * 2);
            if (warp < (LOOSE ? 1 : 3)) {
                const uintptr_t pb = warp == 0 ? reinterpret_cast<uintptr_t>(N.error + (nbase >> 1))
                                   : reinterpret_cast<uintptr_t>((warp == 1 ? N.min_vals : N.max_vals) + (nbase >> qshift));
                const int64_t bytes = warp == 0 ? (nn + 1) >> 1 : ((nn >> qshift) + 1) * 2;
                const uintptr_t first = pb & ~(uintptr_t)127;
                const int lines = (int)((pb + bytes - first + 127) >> 7);
                for (int i = lane; i < lines; i += 32) asm volatile("prefetch.global.L2 [%0];" ::"l"(first + ((uintptr_t)i << 7)));
            }
        }

        // ---- a = bf16(g + Qinv(e)) in place; per-octet maxima stay in registers ------------------------
        float omax[S_SLOTS];
        // regular tile: whole blocks of 64, 14 whole octets per thread, aligned codes, every block with the fast decode
        const bool swz = !LOOSE && tables && (n & 63) == 0 && n_oct >= S_FULL * S_NT && ef_al4 && ss.ctrl[slow_slot] == 0 && T.quant_err == nullptr;
        if (swz) dequant_phase_regular(tile4, ss, n_oct, cw, omax);
        else if (LOOSE && tables && (n & 7) == 0 && n_oct >= S_FULL * S_NT && ef_al4)   // a full tile: branch-free first octets
            dequant_phase<S_FULL>(tile4, ss, tables, mn_g, mx_g, cshift, n, n_oct, cw, omax, la.qbs, lrem0);
        else dequant_phase<0>(tile4, ss, tables, mn_g, mx_g, cshift, n, n_oct, cw, omax, LOOSE ? la.qbs : 0, lrem0);

        MAB_CTICK(1);
        // ---- exact top-k ---------------------------------------------------------------------------
        {
            float tm = 0.0f;
#pragma unroll
            for (int j = 0; j < S_SLOTS; ++j) tm = fmaxf(tm, omax[j]);
            const int wm = __reduce_max_sync(0xffffffffu, __float_as_int(tm));
            if (lane == 0 && wm) atomicMax(&ss.kmax, wm);
        }
        __syncthreads();
        const int kmax = ss.kmax;
        bool done = false;
        int C = -1;                                          // >= 0: the selection is described by the candidate list
        uint32_t Tc_sel = 0;
        if (kmax == 0) {
            // every key is zero: the k lowest positions win the ties
            uint32_t gt[S_WPT], tw[S_WPT];
#pragma unroll
            for (int i = 0; i < S_WPT; ++i) {
                const int lo = (t * S_WPT + i) * 32;
                gt[i] = (lo + 32 <= k) ? 0xFFFFFFFFu : (lo < k ? ((1u << (k - lo)) - 1u) : 0u);
                tw[i] = 0u;
            }
            resolve_selection_regs(gt, tw, 0, ss);
            done = true;
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
                for (int j = 0; j < S_SLOTS; ++j) mine += (__float_as_int(omax[j]) >= gq) ? 1 : 0;
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
            MAB_CTICK(8);
            const int T_lo = have_lo ? lo : 0;
            if (T_lo > 0) {
                const float T_lo_f = __int_as_float(T_lo);
                const uint32_t T16 = ((uint32_t)T_lo + 0xFFFFu) >> 16;          // the bound as a bf16 magnitude
                // 1. each warp lists its octets whose maximum reaches the bound and turns their values that
                //    reach it into candidates (any order)
                uint16_t* wlist = ss.oct_list + warp * S_WLIST;
                int n_w = 0;
#pragma unroll
                for (int j = 0; j < S_SLOTS; ++j) {
                    const bool q = omax[j] >= T_lo_f;
                    const unsigned bal = __ballot_sync(0xffffffffu, q);
                    const int at = n_w + __popc(bal & ((1u << lane) - 1u));
                    if (q && at < S_WLIST) wlist[at] = (uint16_t)(t + j * S_NT);
                    n_w += __popc(bal);
                }
                if (lane == 0 && n_w > S_WLIST) ss.ctrl[4] = 1;
                n_w = min(n_w, S_WLIST);
                __syncwarp();
                for (int e0 = 0; e0 < n_w; e0 += 64) {                // two listed octets per lane and round
                    uint32_t o2[2] = {0u, 0u}, mask2[2] = {0u, 0u};
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int e = e0 + h * 32 + lane;
                        if (e < n_w) {
                            o2[h] = wlist[e];
                            const uint4 v = tile4[phys_oct(o2[h], swz)];
                            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                mask2[h] |= ((w[p] & 0x7FFFu) >= T16) ? (1u << (2 * p)) : 0u;
                                mask2[h] |= (((w[p] >> 16) & 0x7FFFu) >= T16) ? (2u << (2 * p)) : 0u;
                            }
                        }
                    }
                    int slot = warp_alloc(__popc(mask2[0]) + __popc(mask2[1]), &ss.n_cand);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint32_t mask = mask2[h];
                        while (mask) {
                            const uint32_t pos = (o2[h] << 3) + (__ffs(mask) - 1);
                            mask &= mask - 1;
                            if (slot < S_CAND_CAP) ss.cand[slot] = ((uint32_t)(tile[phys_pos(pos, swz)] & 0x7FFFu) << 16) | (0xFFFFu - pos);
                            ++slot;
                        }
                    }
                }
                __syncthreads();
                MAB_CTICK(10);
                const int n_cand = ss.n_cand;
                if (n_cand <= S_CAND_CAP && ss.ctrl[4] == 0) {
                    C = n_cand;
                    // 2. the k-th largest candidate.  The composite values are distinct, so no ties are left to
                    //    break.  256-bin radix levels over the live range, filled by all threads; every warp
                    //    reads the histogram for itself (no barrier for the result); the last <= 32 members
                    //    are gathered and ranked directly, again by every warp for itself.
                    {
                        uint32_t lo_c = T16 << 16, hi_c = ((uint32_t)kmax & 0xFFFF0000u) | 0xFFFFu;
                        int k_rem = k;
                        for (int level = 0; level < 6; ++level) {
                            const uint32_t W1 = hi_c - lo_c;
                            const int sh = W1 < 256u ? 0 : (32 - __clz(W1)) - 8;
                            if (level > 0) {
                                __syncthreads();
                                ss.hist[t] = 0;
                                __syncthreads();
                            }
                            for (int i = t; i < C; i += S_NT) {
                                const uint32_t c = ss.cand[i];
                                if (c >= lo_c && c <= hi_c) atomicAdd(&ss.hist[(c - lo_c) >> sh], 1);
                            }
                            __syncthreads();
                            int h[8], sum = 0;
                            {
                                const int4 ha = reinterpret_cast<const int4*>(ss.hist)[lane * 2], hb4 = reinterpret_cast<const int4*>(ss.hist)[lane * 2 + 1];
                                h[0] = ha.x; h[1] = ha.y; h[2] = ha.z; h[3] = ha.w; h[4] = hb4.x; h[5] = hb4.y; h[6] = hb4.z; h[7] = hb4.w;
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) sum += h[j];
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
                            if (sh == 0) { Tc_sel = lo_c; break; }
                            if (hb <= 32) {
                                for (int i = t; i < C; i += S_NT) {
                                    const uint32_t c = ss.cand[i];
                                    if (c >= lo_c && c <= hi_c) ss.member[atomicAdd(&ss.n_member, 1)] = c;
                                }
                                __syncthreads();
                                const uint32_t me = lane < hb ? ss.member[lane] : 0u;
                                int greater = 0;
                                for (int j = 0; j < hb; ++j) greater += (ss.member[j] > me) ? 1 : 0;
                                const unsigned hit = __ballot_sync(0xffffffffu, lane < hb && greater == k_rem - 1);
                                Tc_sel = __shfl_sync(0xffffffffu, me, __ffs(hit) - 1);
                                break;
                            }
                        }
                    }
                    MAB_CTICK(11);
                    // 3. selected positions -> bitmap -> ranks
                    for (int i = t; i < C; i += S_NT) {
                        const uint32_t c = ss.cand[i];
                        if (c >= Tc_sel) { const uint32_t pos = 0xFFFFu - (c & 0xFFFFu); atomicOr(&ss.sel_bm[pos >> 5], 1u << (pos & 31)); }
                    }
                    __syncthreads();
                    {
                        const uint4 wq = reinterpret_cast<const uint4*>(ss.sel_bm)[t];
                        const int c0 = __popc(wq.x), c1 = __popc(wq.y), c2 = __popc(wq.z), c3 = __popc(wq.w);
                        int total;
                        const int before = block_exclusive_scan(c0 + c1 + c2 + c3, ss.scan, total);
                        ushort4 sb;
                        sb.x = (uint16_t)before; sb.y = (uint16_t)(before + c0); sb.z = (uint16_t)(before + c0 + c1); sb.w = (uint16_t)(before + c0 + c1 + c2);
                        reinterpret_cast<ushort4*>(ss.sel_before)[t] = sb;
                    }
                    __syncthreads();
                    done = true;
                }
            }
        }
        MAB_CTICK(2);
        if (!done) {
            // general path: bisection on the key bits over the tile in shared memory (data-independent cost)
            C = -1;
            done = true;
            if (t < 40) ss.counters[t] = 0;
            __syncthreads();
            int Tk = 0;
            for (int bit = 30; bit >= 16; --bit) {          // bf16 keys have 16 zero bits below
                const int cand = Tk | (1 << bit);
                if (tile_count_ge(tile, n_oct, cand, &ss.counters[bit]) >= k) Tk = cand;
            }
            const int n_gt = tile_count_ge(tile, n_oct, Tk + 0x10000, &ss.counters[32]);
            const int need = k - n_gt;
            const float Tf = __int_as_float(Tk);
            uint32_t gt[S_WPT], tw[S_WPT];                  // the thread's 128 positions = 16 octets
#pragma unroll
            for (int i = 0; i < S_WPT; ++i) {
                gt[i] = 0u; tw[i] = 0u;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int o = (t * S_WPT + i) * 4 + b;
                    if (o < n_oct) {
                        float v[8];
                        unpack8(tile4[phys_oct(o, swz)], v);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const bool valid = o * 8 + e < n;     // padding never competes, whatever the threshold
                            gt[i] |= (valid && fabsf(v[e]) > Tf) ? (1u << (8 * b + e)) : 0u;
                            tw[i] |= (valid && fabsf(v[e]) == Tf) ? (1u << (8 * b + e)) : 0u;
                        }
                    }
                }
            }
            resolve_selection_regs(gt, tw, need, ss);
        }

        MAB_CTICK(3);
        // ---- I[row], V[row]; selected positions become 0 in the tile ------------------------------------
        if (C >= 0) {
            for (int i = t; i < C; i += S_NT) {
                const uint32_t c = ss.cand[i];
                if (c >= Tc_sel) {
                    const uint32_t q = 0xFFFFu - (c & 0xFFFFu), w = q >> 5;
                    const int rank = ss.sel_before[w] + __popc(ss.sel_bm[w] & ((1u << (q & 31)) - 1u));
                    const int at = phys_pos(q, swz);
                    i_out[rank] = (int16_t)q;
                    v_out[rank] = tile[at];
                    tile[at] = 0;
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
                    const int at = phys_pos(q, swz);
                    i_out[p] = (int16_t)q;
                    v_out[p++] = tile[at];
                    tile[at] = 0;
                }
            }
        }
        __syncthreads();

        if (T.quant_err != nullptr) {
            // alpha == -2: the residual a also goes to the caller's buffer (same element type as the gradient; linear tile)
            uint16_t* qe = reinterpret_cast<uint16_t*>(T.quant_err) + base;
            const bool vec = aligned16(qe);
            for (int o = t; o < n_oct; o += S_NT) {
                if (vec && o * 8 + 8 <= n) reinterpret_cast<uint4*>(qe)[o] = tile4[o];
                else for (int e = o * 8; e < min(o * 8 + 8, n); ++e) qe[e] = tile[e];
            }
        }
        MAB_CTICK(4);
        // ---- statistics and codes of the residual ----------------------------------------------------------
        uint16_t* mn_out = T.min_vals + qb0;
        uint16_t* mx_out = T.max_vals + qb0;
        if (LOOSE) {
            // the residual goes back to the gradient buffer, the extremes of every quantisation block the tile
            // touches to the scratch arrays
            uint16_t* g_w = const_cast<uint16_t*>(g);
            uint32_t* s_qlo = ss.cand;                       // the candidate list is free again
            uint32_t* s_qhi = ss.cand + LOOSE_MAX_QB;
            static_assert(2 * LOOSE_MAX_QB <= S_CAND_CAP, "block extremes reuse the candidate list");
            for (int i = t; i < LOOSE_MAX_QB; i += S_NT) { s_qlo[i] = 0xFFFFFFFFu; s_qhi[i] = 0u; }
            __syncthreads();
            if (!staged)
                for (int i = t; i < n; i += S_NT) g_w[i] = tile[i];
            MAB_CTICK(6);
            const bool big = la.qbs >= SEL_MAX_TILE;
            const int n_whole = n >> 3;                      // octets without padding
            // a thread's octets are S_NT apart: it keeps the extremes of the block it is in and hands them over
            // when the block changes (for blocks longer than a tile: at most once)
            int cur = -1;
            uint32_t alo = 0x7F807F80u, ahi = 0xFF80FF80u;   // packed bf16 pairs: running minimum from +inf, maximum from -inf
#pragma unroll
            for (int j = 0; j < S_SLOTS; ++j) {
                const int o = t + j * S_NT;
                if (o < n_whole) {
                    const uint4 v = tile4[o];
                    if (staged) reinterpret_cast<uint4*>(g_w)[o] = v;   // whole octets, 16-byte aligned: the residual goes home
                    const int qi = loose_block(lrem0 + o * 8, la.qbs, big);
                    if (qi != cur) {
                        if (cur >= 0) {
                            alo = min_bf16x2(alo, alo >> 16 | alo << 16); ahi = max_bf16x2(ahi, ahi >> 16 | ahi << 16);
                            atomicMin(&s_qlo[cur], ord_key(__uint_as_float(alo << 16)));
                            atomicMax(&s_qhi[cur], ord_key(__uint_as_float(ahi << 16)));
                        }
                        cur = qi; alo = 0x7F807F80u; ahi = 0xFF80FF80u;
                    }
                    ahi = max_bf16x2(max_bf16x2(ahi, v.x), max_bf16x2(max_bf16x2(v.y, v.z), v.w));
                    alo = min_bf16x2(min_bf16x2(alo, v.x), min_bf16x2(min_bf16x2(v.y, v.z), v.w));
                }
            }
            if (t == S_NT - 1 && n_whole < n_oct) {           // the tensor's last, short octet: element by element
                const int qi = loose_block(lrem0 + n_whole * 8, la.qbs, big);
                for (int e = n_whole * 8; e < n; ++e) {
                    const uint32_t key = ord_key(__uint_as_float((uint32_t)tile[e] << 16));
                    atomicMin(&s_qlo[qi], key); atomicMax(&s_qhi[qi], key);
                }
            }
            {
                alo = min_bf16x2(alo, alo >> 16 | alo << 16); ahi = max_bf16x2(ahi, ahi >> 16 | ahi << 16);
                uint32_t klo = ord_key(__uint_as_float(alo << 16)), khi = ord_key(__uint_as_float(ahi << 16));
                const int c_first = __shfl_sync(0xffffffffu, cur, 0);
                if (__all_sync(0xffffffffu, cur == c_first)) {  // the whole warp ended in one block (or holds nothing)
                    klo = __reduce_min_sync(0xffffffffu, klo);
                    khi = __reduce_max_sync(0xffffffffu, khi);
                    if (lane == 0 && cur >= 0) { atomicMin(&s_qlo[cur], klo); atomicMax(&s_qhi[cur], khi); }
                } else if (cur >= 0) {
                    atomicMin(&s_qlo[cur], klo); atomicMax(&s_qhi[cur], khi);
                }
            }
            MAB_CTICK(7);
            __syncthreads();
            {
                const int64_t at = la.qb_first[ti] + qb0;
                for (int i = t; i < n_qb; i += S_NT) {
                    atomicMin(la.st_min + at + i, s_qlo[i]);
                    atomicMax(la.st_max + at + i, s_qhi[i]);
                }
            }
            MAB_CTICK(9);
            __syncthreads();                                 // the tile is overwritten by the next load
        } else if (swz) {
            stats_encode_regular(tile4, n_qb, mn_out, mx_out, ef_out, (reinterpret_cast<uintptr_t>(ef_out) & 15) == 0);
            __syncthreads();                                 // the tile is overwritten by the next load
        } else if (tables && (n & 63) == 0) {
            // whole blocks of 64: statistics block by block (a thread's 8 octets, rotated so that a warp's
            // 16-byte reads spread over the banks), constants to the tables, then codes octet by octet
            for (int b = t; b < n_qb; b += S_NT) {
                uint32_t hi2 = 0xFF80FF80u, lo2 = 0x7F807F80u;  // running packed max (from -inf) and min (from +inf)
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = tile4[(b << 3) + ((c + lane) & 7)];
                    hi2 = max_bf16x2(max_bf16x2(hi2, v.x), max_bf16x2(max_bf16x2(v.y, v.z), v.w));
                    lo2 = min_bf16x2(min_bf16x2(lo2, v.x), min_bf16x2(min_bf16x2(v.y, v.z), v.w));
                }
                hi2 = max_bf16x2(hi2, hi2 >> 16);
                lo2 = min_bf16x2(lo2, lo2 >> 16);
                const uint16_t mn_b = (uint16_t)(lo2 & 0xFFFFu), mx_b = (uint16_t)(hi2 & 0xFFFFu);
                mn_out[b] = mn_b; mx_out[b] = mx_b;
                const QParams q2 = qparams(mn_b, mx_b);
                const EncodeConsts ec = encode_consts(q2);
                ss.qt.mu[b] = make_float2(q2.mn, q2.u);
                ss.qt.r0[b] = ec.fast ? ec.r02.x : 0.0f;
            }
            __syncthreads();
            uint32_t redo = 0u;                              // octets too close to a code boundary, or of a degenerate block
            encode_phase<0>(tile4, ss, ef_out, ef_al4, n, n_oct, redo);
            while (redo) {
                const int j = __ffs(redo) - 1;
                redo &= redo - 1;
                const int o = t + j * S_NT;
                const float2 mu = ss.qt.mu[o >> 3];
                const QParams q2 = {mu.x, mu.y};
                float r[8];
                unpack8(tile4[o], r);
                store_code_word(ef_out, ef_al4, o, n, encode_octet<false>(r, q2));
            }
            __syncthreads();                                 // the tile is overwritten by the next load
        } else {
            // any block size, ragged ends: one thread per quantisation block
            for (int b = t; b < n_qb; b += S_NT) {
                uint32_t hi2 = 0xFF80FF80u, lo2 = 0x7F807F80u;
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
                        store_code_word(ef_out, ef_al4, o, n, cnt >= 8 ? encode_octet<false>(r, q2) : encode_octet_exact(r, q2, cnt));
                    }
                }
            }
            __syncthreads();                                 // the tile is overwritten by the next load
        }
        MAB_CTICK(5);
#ifdef MAB_STATS
        if (threadIdx.x == 0) atomicAdd(&g_stats_c[15], 1ull);
#endif
    }
}

int launch_ef_topk_quant_bf16(const mab_tensor* dev_tensors, int n_tensors, int total_units, int qbs, int max_dbs, cudaStream_t s,
                              const LooseArgs* loose) {
    int qshift = 0;
    if (loose == nullptr) while ((1 << qshift) < qbs) ++qshift;
    const int smem = ((max_dbs * 2 + 127) & ~127) + (int)sizeof(SmemSel);
    const int per_sm = std::min(S_CTAS, (device_max_optin_smem() + 1024) / (smem + 3 * 1024 + 128));
    if (per_sm < 2) return 1;                                // not even two CTAs per SM: the caller uses the other kernel
    const int grid = (int)std::min<int64_t>(total_units, (int64_t)device_sm_count() * per_sm);
    LooseArgs la = {0, nullptr, nullptr, nullptr};
    if (loose) la = *loose;
    auto run = [&](auto kern) -> int {
        MAB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kern<<<grid, S_NT, smem, s>>>(dev_tensors, n_tensors, total_units, qshift, max_dbs, la);
        return MAB_OK;
    };
    const int rc = loose ? run(ef_topk_quant_bf16_kernel<false, true>)
                 : qshift == 6 ? run(ef_topk_quant_bf16_kernel<true, false>) : run(ef_topk_quant_bf16_kernel<false, false>);
    if (rc) return rc;
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

int copy_timeout_bf16(int* out, bool clear) {
    cudaError_t e = cudaMemcpyFromSymbol(out, g_copy_timeout_bf16, sizeof(int));
    if (e == cudaSuccess && clear) { const int z = 0; e = cudaMemcpyToSymbol(g_copy_timeout_bf16, &z, sizeof(int)); }
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "mab_device_error");
}

}  // namespace mab
