// The two consumers of the (I, V) ring buffer outside MicroAdam: Sparse M-FAC's scalar products of a
// dense vector with every sparse row and its linear combination of the rows
// (sparse_mfac/sparse_core_mfac_w_ef.py:188-221, native calls SP and LCG of ista_daslab_cuda_sparse_mfac).
// Row r of the buffer holds, for top-k block b, the in-block positions I[r, b * kbs + j] and the
// values V[r, b * kbs + j]; entry j of a row addresses element (j / kbs) * dbs + I[r, j].
//
// Both results are reproducible bit for bit: fixed assignment of entries to threads, fixed
// reduction trees, rows accumulated in row order.
#include "common.cuh"
#include "window.cuh"

namespace mab {

constexpr int SPR_SR = 7296;          // elements of a block one CTA accumulates at a time (57 * 128)
constexpr int SPR_THREADS = 512;

constexpr int SP_THREADS = 1024;

template <typename T> __device__ __forceinline__ float load_value(const void* p, int64_t i);
template <> __device__ __forceinline__ float load_value<float>(const void* p, int64_t i) { return reinterpret_cast<const float*>(p)[i]; }
template <> __device__ __forceinline__ float load_value<uint16_t>(const void* p, int64_t i) { return bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p)[i]); }

// out[r] = sum_j V[r, j] * g[(j / kbs) * dbs + I[r, j]]: one CTA per row, fp32 products summed per thread in
// entry order, then over the CTA by a fixed tree.
template <typename TG, typename TV>
__global__ void __launch_bounds__(SP_THREADS)
sparse_rows_dot_kernel(int64_t k, int64_t dbs, int64_t kbs, const TG* __restrict__ g, const int16_t* __restrict__ I,
                       const void* __restrict__ V, float* __restrict__ out) {
    __shared__ float s_part[SP_THREADS / 32];
    const int r = blockIdx.x;
    const int16_t* idx = I + (int64_t)r * k;
    float acc = 0.0f;
    for (int64_t j = threadIdx.x; j < k; j += SP_THREADS) {
        const int64_t e = (j / kbs) * dbs + (int64_t)idx[j];
        acc = __fadd_rn(acc, __fmul_rn(load_value<TV>(V, (int64_t)r * k + j), Elem<TG>::load(g, e)));
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
    if (lane_id() == 0) s_part[warp_id()] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < SP_THREADS / 32; ++w) total = __fadd_rn(total, s_part[w]);
        out[r] = total;
    }
}

// out[e] += sum_r M[r] * V[r, j] over the entries (r, j) that address e: one CTA per sub-range of a top-k block
// with a dense fp32 accumulator in shared memory; rows are added in row order (positions are unique inside a
// row, so a row needs no atomics).
template <typename TO, typename TV>
__global__ void __launch_bounds__(SPR_THREADS)
sparse_rows_combine_kernel(int64_t d, int rows, int64_t k, int dbs, int kbs, int nfull, int k_few, const float* __restrict__ M,
                           const int16_t* __restrict__ I, const void* __restrict__ V, TO* __restrict__ out, int total_units) {
    __shared__ float acc[SPR_SR];
    const int subs_per_block = (dbs + SPR_SR - 1) / SPR_SR;
    for (int unit = blockIdx.x; unit < total_units; unit += gridDim.x) {
        int blk = unit / subs_per_block, sub = unit - blk * subs_per_block;
        if (blk > nfull) { sub += (blk - nfull) * subs_per_block; blk = nfull; }
        const int64_t blk_base = (int64_t)blk * dbs;
        const int n_blk = (int)min((int64_t)dbs, d - blk_base);
        const int kcnt = (blk < nfull) ? kbs : k_few;
        const int s0 = sub * SPR_SR;
        const int len = min(SPR_SR, n_blk - s0);
        for (int i = threadIdx.x; i < len; i += SPR_THREADS) acc[i] = 0.0f;
        __syncthreads();
        for (int r = 0; r < rows; ++r) {
            const int64_t row0 = (int64_t)r * k + (int64_t)blk * kbs;
            const float coef = M[r];
            for (int j = threadIdx.x; j < kcnt; j += SPR_THREADS) {
                const int pos = (int)I[row0 + j] - s0;
                if (pos >= 0 && pos < len) acc[pos] = __fadd_rn(acc[pos], __fmul_rn(coef, load_value<TV>(V, row0 + j)));
            }
            __syncthreads();
        }
        for (int i = threadIdx.x; i < len; i += SPR_THREADS) {
            const int64_t e = blk_base + s0 + i;
            Elem<TO>::store(out, e, __fadd_rn(Elem<TO>::load(out, e), acc[i]));
        }
        __syncthreads();
    }
}

}  // namespace mab

using namespace mab;

static int check_geometry(const char* what, int64_t d, int64_t rows, int64_t k, int64_t dbs, int64_t kbs, int* nfull, int* k_few) {
    MAB_REQUIRE(d >= 0 && k >= 0 && rows >= 0 && dbs > 0 && kbs > 0, MAB_ERR_BAD_ARG, "%s: bad sizes", what);
    MAB_REQUIRE(rows <= MAB_MAX_WINDOW, MAB_ERR_LIMIT, "%s: %lld rows, at most %d", what, (long long)rows, MAB_MAX_WINDOW);
    MAB_REQUIRE(dbs <= 32768, MAB_ERR_LIMIT, "%s: d_block_size %lld exceeds 32768", what, (long long)dbs);
    const int64_t nf = d / dbs;
    const int64_t few = k - nf * kbs;
    MAB_REQUIRE(nf < ((int64_t)1 << 28) && few >= 0 && few <= d - nf * dbs, MAB_ERR_BAD_ARG,
                "%s: k=%lld inconsistent with d=%lld, d_block_size=%lld, k_block_size=%lld", what, (long long)k, (long long)d,
                (long long)dbs, (long long)kbs);
    *nfull = (int)nf; *k_few = (int)few;
    return MAB_OK;
}

extern "C" int mab_sparse_rows_dot(int64_t d, int64_t rows, int64_t k, int64_t d_block_size, int64_t k_block_size,
                                   const void* g, int g_dtype, const int16_t* I, const void* V, int v_dtype, float* out,
                                   void* stream) {
    int nfull, k_few;
    if (int rc = check_geometry("sparse_rows_dot", d, rows, k, d_block_size, k_block_size, &nfull, &k_few)) return rc;
    if (rows == 0) return MAB_OK;
    MAB_REQUIRE(g && I && V && out, MAB_ERR_BAD_ARG, "sparse_rows_dot: null pointer");
    MAB_REQUIRE((g_dtype == MAB_F32 || g_dtype == MAB_BF16) && (v_dtype == MAB_F32 || v_dtype == MAB_BF16), MAB_ERR_UNSUPPORTED,
                "sparse_rows_dot: dtypes %d, %d", g_dtype, v_dtype);
    cudaStream_t s = (cudaStream_t)stream;
    const int grid = (int)rows;
    if (g_dtype == MAB_F32 && v_dtype == MAB_BF16)
        sparse_rows_dot_kernel<float, uint16_t><<<grid, SP_THREADS, 0, s>>>(k, d_block_size, k_block_size, (const float*)g, I, V, out);
    else if (g_dtype == MAB_F32)
        sparse_rows_dot_kernel<float, float><<<grid, SP_THREADS, 0, s>>>(k, d_block_size, k_block_size, (const float*)g, I, V, out);
    else if (v_dtype == MAB_BF16)
        sparse_rows_dot_kernel<uint16_t, uint16_t><<<grid, SP_THREADS, 0, s>>>(k, d_block_size, k_block_size, (const uint16_t*)g, I, V, out);
    else
        sparse_rows_dot_kernel<uint16_t, float><<<grid, SP_THREADS, 0, s>>>(k, d_block_size, k_block_size, (const uint16_t*)g, I, V, out);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "sparse_rows_dot_kernel launch");
}

extern "C" int mab_sparse_rows_combine(int64_t d, int64_t rows, int64_t k, int64_t d_block_size, int64_t k_block_size,
                                       const float* M, const int16_t* I, const void* V, int v_dtype, void* out, int out_dtype,
                                       void* stream) {
    int nfull, k_few;
    if (int rc = check_geometry("sparse_rows_combine", d, rows, k, d_block_size, k_block_size, &nfull, &k_few)) return rc;
    if (rows == 0 || d == 0) return MAB_OK;
    MAB_REQUIRE(M && I && V && out, MAB_ERR_BAD_ARG, "sparse_rows_combine: null pointer");
    MAB_REQUIRE((out_dtype == MAB_F32 || out_dtype == MAB_BF16) && (v_dtype == MAB_F32 || v_dtype == MAB_BF16), MAB_ERR_UNSUPPORTED,
                "sparse_rows_combine: dtypes %d, %d", out_dtype, v_dtype);
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    const int dbs = (int)d_block_size;
    const int subs = (dbs + SPR_SR - 1) / SPR_SR;
    const int64_t tail = d - (int64_t)nfull * dbs;
    const int64_t units = (int64_t)nfull * subs + (tail > 0 ? (tail + SPR_SR - 1) / SPR_SR : 0);
    if (units == 0) return MAB_OK;
    const int grid = (int)std::min<int64_t>(units, (int64_t)device_sm_count() * 4);
    cudaStream_t s = (cudaStream_t)stream;
#define MAB_LAUNCH_COMBINE(TO, TV) sparse_rows_combine_kernel<TO, TV><<<grid, SPR_THREADS, 0, s>>>( \
        d, (int)rows, k, dbs, (int)k_block_size, nfull, k_few, M, I, V, (TO*)out, (int)units)
    if (out_dtype == MAB_F32 && v_dtype == MAB_BF16) MAB_LAUNCH_COMBINE(float, uint16_t);
    else if (out_dtype == MAB_F32) MAB_LAUNCH_COMBINE(float, float);
    else if (v_dtype == MAB_BF16) MAB_LAUNCH_COMBINE(uint16_t, uint16_t);
    else MAB_LAUNCH_COMBINE(uint16_t, float);
#undef MAB_LAUNCH_COMBINE
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? MAB_OK : cuda_fail(e, "sparse_rows_combine_kernel launch");
}
