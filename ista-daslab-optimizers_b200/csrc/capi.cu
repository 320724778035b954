// Host side of the C ABI: error reporting, device queries and the driver of the fused step.
#include <math.h>
#include <string.h>
#include <atomic>
#include <vector>
#include <algorithm>
#include "common.cuh"
#include "fused.cuh"
#include "select.cuh"

namespace mab {

static thread_local char g_error[512] = "";
static std::atomic<int64_t> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
    set_error("%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
    return MAB_ERR_CUDA;
}

static int device_attr(cudaDeviceAttr attr, const char* what) {
    int dev = 0, v = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&v, attr, dev);
    if (e != cudaSuccess) { cuda_fail(e, what); return -1; }
    return v;
}

int device_sm_count() {
    static thread_local int cached_dev = -1, cached = -1;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev != cached_dev || cached < 0) {
        cached = device_attr(cudaDevAttrMultiProcessorCount, "query SM count");
        cached_dev = (cached < 0) ? -1 : dev;
    }
    return cached;
}

int device_max_optin_smem() { return device_attr(cudaDevAttrMaxSharedMemoryPerBlockOptin, "query shared memory per block"); }

}  // namespace mab

using namespace mab;

extern "C" const char* mab_last_error(void) { return g_error; }

extern "C" int64_t mab_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int mab_device_error(void) {
    int a = 0, b = 0, c = 0;
    if (int rc = copy_timeout_f32(&a, false)) return rc;
    if (int rc = copy_timeout_bf16(&b, false)) return rc;
    if (int rc = copy_timeout_window(&c, false)) return rc;
    return (a | b | c) ? 1 : 0;
}

extern "C" int mab_device_error_clear(void) {
    int v = 0;
    if (int rc = copy_timeout_f32(&v, true)) return rc;
    if (int rc = copy_timeout_bf16(&v, true)) return rc;
    return copy_timeout_window(&v, true);
}

extern "C" int mab_wait_selftest(int probe_limit, void* stream) {
    MAB_REQUIRE(probe_limit >= 1 && probe_limit <= 4096, MAB_ERR_BAD_ARG, "mab_wait_selftest: probe_limit=%d outside [1, 4096]", probe_limit);
    return launch_wait_selftest(probe_limit, (cudaStream_t)stream);
}

extern "C" int mab_get_sm_count(void) { return device_sm_count(); }

extern "C" int mab_get_max_floats_for_shared_memory_per_thread_block(void) {
    const int bytes = device_max_optin_smem();
    return bytes < 0 ? bytes : bytes / 4;
}

extern "C" int64_t mab_fused_step_workspace_bytes(int n_tensors) {
    return (int64_t)std::max(n_tensors, 1) * (int64_t)sizeof(mab_tensor);
}

static bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }

// Quantisation blocks that the one-kernel form of kernel A covers: they tile every top-k block exactly.
static bool aligned_qbs(int64_t qbs) { return is_pow2(qbs) && qbs >= 8 && qbs <= 128; }

static int64_t round256(int64_t v) { return (v + 255) & ~(int64_t)255; }

// Workspace of a call whose quantisation blocks have any other size ("loose"): the descriptor table, the first
// scratch entry of every tensor, and two uint32 per quantisation block for the merged extremes.
struct LooseLayout { int64_t off_first, off_min, off_max, total_qb, bytes; };
static LooseLayout loose_layout(const mab_tensor* tensors, int n, int64_t qbs) {
    LooseLayout L;
    L.total_qb = 0;
    for (int i = 0; i < n; ++i) L.total_qb += tensors[i].d > 0 ? ceil_div64(tensors[i].d, qbs) : 0;
    L.off_first = round256(mab_fused_step_workspace_bytes(n));
    L.off_min = L.off_first + round256((int64_t)std::max(n, 1) * 8);
    L.off_max = L.off_min + round256(L.total_qb * 4);
    L.bytes = L.off_max + round256(L.total_qb * 4);
    return L;
}

extern "C" int64_t mab_fused_step_workspace_bytes_for(const mab_tensor* tensors, int n_tensors, const mab_step_args* args) {
    if (!tensors || !args || n_tensors <= 0 || args->quant_block_size <= 0 || aligned_qbs(args->quant_block_size))
        return mab_fused_step_workspace_bytes(n_tensors);
    return loose_layout(tensors, n_tensors, args->quant_block_size).bytes;
}

// Why a tensor cannot take the fused path, or nullptr if it can.
// `window_only`: kernel B alone with alpha == 0 reads neither the error feedback nor the gradient, so the
// quantisation geometry does not matter (any quant_block_size) and those buffers may be absent.
static const char* fused_obstacle(const mab_tensor* t, const mab_step_args* a, bool window_only = false) {
    if (!t || !a) return "null argument";
    if (t->d <= 0) return "empty tensor";
    window_only = window_only && a->alpha == 0.0f;
    if (!t->param || !t->I || !t->V) return "null buffer";
    if (!window_only && (!t->grad || !t->error || !t->min_vals || !t->max_vals)) return "null buffer";
    if (t->param_dtype != MAB_F32 && t->param_dtype != MAB_BF16) return "param dtype is neither f32 nor bf16";
    if (t->grad_dtype != MAB_F32 && t->grad_dtype != MAB_BF16) return "grad dtype is neither f32 nor bf16";
    const int qbs = window_only ? 8 : a->quant_block_size;
    const bool loose = !aligned_qbs(qbs);                  // quantisation blocks that ignore the borders of the top-k blocks
    if (loose) {
        if (qbs < 64 || qbs % 8 != 0 || qbs > (1 << 30)) return "quant_block_size is neither a power of two in [8, 128] nor a multiple of 8 in [64, 2^30]";
        if (a->alpha != 0.0f) return "quantisation blocks that straddle top-k blocks need alpha == 0 on the fused path";
    }
    if (a->alpha == -2.0f) {
        if (!t->quant_err) return "alpha == -2 needs quant_err";
        if (t->param_dtype != t->grad_dtype) return "alpha == -2 needs gradient and parameter of one element type";
    } else if (!(a->alpha >= 0.0f && a->alpha < 1.0f)) return "alpha outside [0, 1) and not -2";
    if (a->m < 1 || a->m > MAB_MAX_WINDOW) return "window rows outside [1, MAB_MAX_WINDOW]";
    if (t->d_block_size <= 0 || t->d_block_size > SEL_MAX_TILE) return "d_block_size outside (0, 32768]";
    const int64_t nfull = t->topk_full_blocks_count;
    const int64_t covered = nfull * t->d_block_size;
    if (nfull < 0 || covered > t->d || t->d - covered >= t->d_block_size) return "block counts inconsistent with d";
    const bool multi = covered < t->d ? nfull >= 1 : nfull > 1;
    if (multi && !loose && t->d_block_size % qbs != 0) return "d_block_size is not a multiple of quant_block_size";
    if (multi && loose && t->d_block_size % 8 != 0) return "d_block_size is not a multiple of 8";
    if (t->k_block_size_many < 1 || t->k_block_size_many > t->d_block_size) return "k_block_size_many out of range";
    if ((covered < t->d) != (t->k_block_size_few > 0) || t->k_block_size_few > t->d - covered) return "k_block_size_few out of range";
    if (t->k != nfull * t->k_block_size_many + t->k_block_size_few) return "k inconsistent with the block geometry";
    if (t->row_pitch != 0 && t->row_pitch < t->k) return "row_pitch smaller than k";
    if (nfull + 1 >= (int64_t)1 << 28) return "too many blocks";
    if (t->ring_index < 0 || t->ring_index >= a->m) return "ring_index outside [0, m)";
    const size_t pe = t->param_dtype == MAB_F32 ? 4 : 2, ge = t->grad_dtype == MAB_F32 ? 4 : 2;
    if (!aligned_to(t->param, pe) || !aligned_to(t->I, 2) || !aligned_to(t->V, 2) ||
        (t->quant_err && !aligned_to(t->quant_err, pe))) return "buffer not aligned to its element size";
    if (!window_only && (!aligned_to(t->grad, ge) || !aligned_to(t->min_vals, 2) || !aligned_to(t->max_vals, 2)))
        return "buffer not aligned to its element size";
    return nullptr;
}

extern "C" int mab_fused_supported(const mab_tensor* t, const mab_step_args* args) {
    if (fused_obstacle(t, args) != nullptr) return 0;
    return aligned_qbs(args->quant_block_size) ? 1 : 2;
}

extern "C" int mab_fused_window_supported(const mab_tensor* t, const mab_step_args* args) {
    return fused_obstacle(t, args, true) == nullptr ? 1 : 0;
}

enum { RUN_A = 1, RUN_B = 2 };

static int fused_run(mab_tensor* tensors, int n, const mab_step_args* args, void* workspace, int64_t workspace_bytes,
                     void* stream, int what) {
    MAB_REQUIRE(n >= 0, MAB_ERR_BAD_ARG, "fused step: n_tensors=%d", n);
    if (n == 0) return MAB_OK;
    MAB_REQUIRE(tensors && args && workspace, MAB_ERR_BAD_ARG, "fused step: null argument");
    const bool loose = (what & RUN_A) && !aligned_qbs(args->quant_block_size);
    MAB_REQUIRE(args->quant_block_size > 0, MAB_ERR_BAD_ARG, "fused step: quant_block_size=%d", args->quant_block_size);
    const int64_t need = loose ? mab_fused_step_workspace_bytes_for(tensors, n, args) : mab_fused_step_workspace_bytes(n);
    MAB_REQUIRE(workspace_bytes >= need, MAB_ERR_BAD_ARG,
                "fused step: workspace of %lld bytes, %lld needed%s", (long long)workspace_bytes, (long long)need,
                loose ? " (mab_fused_step_workspace_bytes_for gives the size for this quant_block_size)" : "");
    MAB_REQUIRE(aligned_to(workspace, 16), MAB_ERR_BAD_ARG, "fused step: workspace must be 16-byte aligned");
    MAB_REQUIRE(args->steps >= 1, MAB_ERR_BAD_ARG, "fused step: steps=%lld", (long long)args->steps);
    for (int i = 0; i < n; ++i) {
        const char* why = fused_obstacle(&tensors[i], args, what == RUN_B);
        MAB_REQUIRE(why == nullptr, MAB_ERR_UNSUPPORTED, "fused step: tensor %d: %s", i, why);
    }
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    cudaStream_t s = (cudaStream_t)stream;

    // Group tensors by (grad dtype, param dtype): each group is launched with its own kernel
    // instantiation, in chunks whose unit prefix fits the kernels' shared-memory table.
    std::vector<int> order(n);
    for (int i = 0; i < n; ++i) order[i] = i;
    auto key = [&](int i) { return tensors[i].grad_dtype * 2 + tensors[i].param_dtype; };
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return key(x) < key(y); });

    struct Chunk { int first, count, units_a, units_b, grad_dtype, param_dtype, max_k, max_dbs; };
    std::vector<Chunk> chunks;
    static thread_local std::vector<mab_tensor> staged;
    staged.resize(n);
    const int max_tensors = WIN_MAX_TENSORS;              // kernels A and B size their unit-prefix tables by it
    const int64_t unit_cap = (int64_t)1 << 30;
    for (int pos = 0; pos < n;) {
        Chunk c = {pos, 0, 0, 0, tensors[order[pos]].grad_dtype, tensors[order[pos]].param_dtype, 0, 0};
        int64_t ua = 0, ub = 0;
        while (pos < n && c.count < max_tensors && key(order[pos]) == c.grad_dtype * 2 + c.param_dtype) {
            mab_tensor& t = tensors[order[pos]];
            const int64_t na = units_a_of(t), nb = units_b_of(t);
            if (c.count > 0 && (ua + na > unit_cap || ub + nb > unit_cap)) break;
            MAB_REQUIRE(na <= unit_cap && nb <= unit_cap, MAB_ERR_LIMIT, "fused step: tensor %d has too many blocks", order[pos]);
            t.decay_f32 = (float)(1.0 - t.lr * t.weight_decay);
            t.neg_lr_f32 = (float)(-t.lr);
            t.first_unit_a = (int32_t)ua;
            t.first_unit_b = (int32_t)ub;
            staged[pos] = t;
            ua += na; ub += nb;
            c.max_k = std::max(c.max_k, std::max(t.k_block_size_many, t.k_block_size_few));
            c.max_dbs = std::max(c.max_dbs, t.d_block_size);
            ++c.count; ++pos;
        }
        c.units_a = (int)ua; c.units_b = (int)ub;
        chunks.push_back(c);
    }
    MAB_CUDA_TRY(cudaMemcpyAsync(workspace, staged.data(), (size_t)n * sizeof(mab_tensor), cudaMemcpyHostToDevice, s));
    const mab_tensor* dev = reinterpret_cast<const mab_tensor*>(workspace);

    if (loose) {
        // kernel A in two parts: residual + merged block extremes, then statistics + codes.  The gradient
        // buffers end up holding the residual, so their probe runs first.
        const int qbs = args->quant_block_size;
        const LooseLayout L = loose_layout(tensors, n, qbs);
        unsigned char* ws = static_cast<unsigned char*>(workspace);
        static thread_local std::vector<int64_t> qb_first;
        qb_first.resize(n);
        int64_t at = 0;
        for (int i = 0; i < n; ++i) { qb_first[i] = at; at += ceil_div64(staged[i].d, qbs); }
        MAB_CUDA_TRY(cudaMemcpyAsync(ws + L.off_first, qb_first.data(), (size_t)n * 8, cudaMemcpyHostToDevice, s));
        MAB_CUDA_TRY(cudaMemsetAsync(ws + L.off_min, 0xFF, (size_t)L.total_qb * 4, s));
        MAB_CUDA_TRY(cudaMemsetAsync(ws + L.off_max, 0x00, (size_t)L.total_qb * 4, s));
        if (args->probe_out)
            for (const Chunk& c : chunks)
                if (int rc = launch_probe(dev + c.first, c.count, c.units_a, qbs, args->probe_out, s, PROBE_G)) return rc;
        for (const Chunk& c : chunks) {
            const LooseArgs la = {qbs, reinterpret_cast<uint32_t*>(ws + L.off_min), reinterpret_cast<uint32_t*>(ws + L.off_max),
                                  reinterpret_cast<const int64_t*>(ws + L.off_first) + c.first};
            if (int rc = launch_ef_topk_quant(dev + c.first, c.count, c.units_a, c.grad_dtype, qbs, c.max_dbs, s, &la)) return rc;
        }
        for (const Chunk& c : chunks) {
            const LooseArgs la = {qbs, reinterpret_cast<uint32_t*>(ws + L.off_min), reinterpret_cast<uint32_t*>(ws + L.off_max),
                                  reinterpret_cast<const int64_t*>(ws + L.off_first) + c.first};
            if (int rc = launch_requant_loose(dev + c.first, c.count, c.units_a, c.grad_dtype, la, s)) return rc;
        }
    } else if (what & RUN_A) {
        for (const Chunk& c : chunks)
            if (int rc = launch_ef_topk_quant(dev + c.first, c.count, c.units_a, c.grad_dtype, args->quant_block_size, c.max_dbs, s)) return rc;
    }
    if (what & RUN_B) {
        WindowArgs wa;
        if (int rc = fill_window_args(wa, args->steps, args->m, args->beta1, args->beta2, args->eps, args->alpha,
                                      args->quant_block_size)) return rc;
        wa.probe = args->probe_out;
        for (const Chunk& c : chunks) {
            if (int rc = launch_window_step(dev + c.first, c.count, c.units_a, c.units_b, c.max_k, c.max_dbs, c.param_dtype, wa, s)) return rc;
        }
    }
    if (args->probe_out && (what & RUN_A))                     // gradient and final error feedback: after the call's last kernel
        for (const Chunk& c : chunks)
            if (int rc = launch_probe(dev + c.first, c.count, c.units_a, args->quant_block_size, args->probe_out, s,
                                      loose ? PROBE_E : PROBE_G | PROBE_E)) return rc;
    return MAB_OK;
}

extern "C" int mab_fused_step(mab_tensor* tensors, int n_tensors, const mab_step_args* args, void* workspace,
                              int64_t workspace_bytes, void* stream) {
    return fused_run(tensors, n_tensors, args, workspace, workspace_bytes, stream, RUN_A | RUN_B);
}

extern "C" int mab_fused_ef_topk_quant(mab_tensor* tensors, int n_tensors, const mab_step_args* args, void* workspace,
                                       int64_t workspace_bytes, void* stream) {
    return fused_run(tensors, n_tensors, args, workspace, workspace_bytes, stream, RUN_A);
}

extern "C" int mab_fused_window_adam_update(mab_tensor* tensors, int n_tensors, const mab_step_args* args, void* workspace,
                                            int64_t workspace_bytes, void* stream) {
    return fused_run(tensors, n_tensors, args, workspace, workspace_bytes, stream, RUN_B);
}

// ---- fused step whose descriptor table lives inside the library --------------------------------
//
// For callers that cannot hand over a device workspace (see the header).  The table is a file-scope
// device array; in host code its name is only a handle, so its device address is looked up once
// per device with cudaGetSymbolAddress and that pointer is what the copy and the kernels receive.

static __device__ __align__(256) unsigned char g_static_table[MAB_STATIC_MAX_TENSORS * sizeof(mab_tensor)];

static int static_table_address(void** out) {
    constexpr int kMaxDevices = 64;
    static std::atomic<void*> cached[kMaxDevices];   // one device address per GPU; racing first calls store the same value
    int dev = -1;
    MAB_CUDA_TRY(cudaGetDevice(&dev));
    MAB_REQUIRE(dev >= 0 && dev < kMaxDevices, MAB_ERR_LIMIT, "mab_fused_step_static: device ordinal %d beyond %d", dev, kMaxDevices);
    void* p = cached[dev].load(std::memory_order_relaxed);
    if (p == nullptr) {
        MAB_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_table));
        MAB_REQUIRE(p != nullptr, MAB_ERR_CUDA, "mab_fused_step_static: no device address for the descriptor table");
        cached[dev].store(p, std::memory_order_relaxed);
    }
    *out = p;
    return MAB_OK;
}

// End (exclusive) of the run of tensors starting at `first` that one launch can take: same element
// types, at most 512 tensors, unit counts within the kernels' 32-bit prefix.  Fills the library-owned
// fields of those tensors and reports the run's totals.
static int static_run_end(mab_tensor* tensors, int n, int first, int* units_a, int* units_b, int* max_k, int* max_dbs) {
    const int gd = tensors[first].grad_dtype, pd = tensors[first].param_dtype;
    const int64_t unit_cap = (int64_t)1 << 30;
    int64_t ua = 0, ub = 0;
    int i = first, mk = 0, md = 0;
    while (i < n && i - first < WIN_MAX_TENSORS && tensors[i].grad_dtype == gd && tensors[i].param_dtype == pd) {
        mab_tensor& t = tensors[i];
        const int64_t na = units_a_of(t), nb = units_b_of(t);
        if (i > first && (ua + na > unit_cap || ub + nb > unit_cap)) break;
        t.decay_f32 = (float)(1.0 - t.lr * t.weight_decay);
        t.neg_lr_f32 = (float)(-t.lr);
        t.first_unit_a = (int32_t)ua;
        t.first_unit_b = (int32_t)ub;
        ua += na; ub += nb;
        mk = std::max(mk, std::max(t.k_block_size_many, t.k_block_size_few));
        md = std::max(md, t.d_block_size);
        ++i;
    }
    *units_a = (int)ua; *units_b = (int)ub; *max_k = mk; *max_dbs = md;
    return i;
}

extern "C" int mab_fused_step_static(mab_tensor* tensors, int n, const mab_step_args* args, void* stream) {
    MAB_REQUIRE(n >= 0, MAB_ERR_BAD_ARG, "mab_fused_step_static: n_tensors=%d", n);
    MAB_REQUIRE(n <= MAB_STATIC_MAX_TENSORS, MAB_ERR_LIMIT,
                "mab_fused_step_static: %d tensors in one call, the built-in table holds %d; split the step into several calls",
                n, MAB_STATIC_MAX_TENSORS);
    if (n == 0) return MAB_OK;
    MAB_REQUIRE(tensors && args, MAB_ERR_BAD_ARG, "mab_fused_step_static: null argument");
    MAB_REQUIRE(args->steps >= 1, MAB_ERR_BAD_ARG, "mab_fused_step_static: steps=%lld", (long long)args->steps);
    MAB_REQUIRE(aligned_qbs(args->quant_block_size), MAB_ERR_UNSUPPORTED,
                "mab_fused_step_static: quant_block_size=%d needs scratch memory (a power of two in [8, 128] does not); use mab_fused_step",
                args->quant_block_size);
    for (int i = 0; i < n; ++i) {
        const char* why = fused_obstacle(&tensors[i], args);
        MAB_REQUIRE(why == nullptr, MAB_ERR_UNSUPPORTED, "mab_fused_step_static: tensor %d: %s", i, why);
        MAB_REQUIRE(units_a_of(tensors[i]) <= ((int64_t)1 << 30) && units_b_of(tensors[i]) <= ((int64_t)1 << 30), MAB_ERR_LIMIT,
                    "mab_fused_step_static: tensor %d has too many blocks", i);
    }
    if (device_sm_count() < 0) return MAB_ERR_CUDA;
    void* table = nullptr;
    if (int rc = static_table_address(&table)) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    WindowArgs wa;
    if (int rc = fill_window_args(wa, args->steps, args->m, args->beta1, args->beta2, args->eps, args->alpha,
                                  args->quant_block_size)) return rc;

    // first pass: fill the library-owned fields of every run, then ship the table
    int ua, ub, mk, md;
    for (int first = 0; first < n;) first = static_run_end(tensors, n, first, &ua, &ub, &mk, &md);
    MAB_CUDA_TRY(cudaMemcpyAsync(table, tensors, (size_t)n * sizeof(mab_tensor), cudaMemcpyHostToDevice, s));
    const mab_tensor* dev = reinterpret_cast<const mab_tensor*>(table);
    // kernel A over every run, then kernel B over every run (the runs are recomputed, not stored)
    for (int first = 0; first < n;) {
        const int end = static_run_end(tensors, n, first, &ua, &ub, &mk, &md);
        if (int rc = launch_ef_topk_quant(dev + first, end - first, ua, tensors[first].grad_dtype, args->quant_block_size, md, s)) return rc;
        first = end;
    }
    wa.probe = args->probe_out;
    for (int first = 0; first < n;) {
        const int end = static_run_end(tensors, n, first, &ua, &ub, &mk, &md);
        if (int rc = launch_window_step(dev + first, end - first, ua, ub, mk, md, tensors[first].param_dtype, wa, s)) return rc;
        first = end;
    }
    if (args->probe_out)
        for (int first = 0; first < n;) {
            const int end = static_run_end(tensors, n, first, &ua, &ub, &mk, &md);
            if (int rc = launch_probe(dev + first, end - first, ua, args->quant_block_size, args->probe_out, s)) return rc;
            first = end;
        }
    return MAB_OK;
}
