/*
 * microadam_b200.h - C ABI of the B200 (sm_100a) MicroAdam step library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*,
 * it is a cudaStream_t; NULL = the legacy default stream), enqueues its work on that stream
 * without synchronising, and returns MAB_OK or a negative status; mab_last_error() then
 * holds a message for the calling thread.  Nothing here allocates device memory, and there
 * is no CPU implementation behind any of these calls: without a CUDA device they fail.
 *
 * bf16 data is passed as uint16_t bit patterns.  Element types of x / param / grad buffers
 * are given by a dtype code (MAB_F32, MAB_BF16).
 *
 * Citations are to files of IST-DASLab/ISTA-DASLab-Optimizers; the functions that
 * micro_adam.py imports from `ista_daslab_cuda_tools` and `ista_daslab_cuda_micro_adam` come
 * from the separate package `ista-daslab-optimizers-cuda`, so each replacement cites the call
 * site that fixes its meaning.
 */
#ifndef MICROADAM_B200_H
#define MICROADAM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MAB_OK               0
#define MAB_ERR_BAD_ARG     (-1)  /* null pointer, negative size, misaligned buffer, bad enum     */
#define MAB_ERR_UNSUPPORTED (-2)  /* dtype / geometry outside what the kernels were written for   */
#define MAB_ERR_CUDA        (-3)  /* a CUDA runtime call or a kernel launch failed                */
#define MAB_ERR_LIMIT       (-4)  /* size beyond a documented maximum                             */

#define MAB_F32   0
#define MAB_BF16  1

#define MAB_K2D 0                 /* tools.py:12-14 CopyDirection.k2d */
#define MAB_D2K 1                 /* tools.py:12-14 CopyDirection.d2k */

#define MAB_MAX_WINDOW 128        /* largest m (window rows) the update kernels accept */

/* Message of the last failure on the calling thread ("" if none). */
const char* mab_last_error(void);

/* Number of kernels this library has launched in this process (all threads, all devices).
 * No counterpart in the reference; it lets a benchmark state how many launches it timed. */
int64_t mab_kernel_launch_count(void);

/* 1 if a kernel of this library on the current device ever gave up a (bounded) wait for the copy
 * engine and returned early, 0 if not, < 0 on failure.  Synchronises with the device.  A non-zero
 * value means the step it happened in is incomplete.  No counterpart in the reference. */
int mab_device_error(void);

/* Clears that flag on the current device.  Synchronises with the device.  No counterpart in the reference. */
int mab_device_error_clear(void);

/* Runs a one-block kernel whose bounded wait cannot be satisfied (its barrier expects bytes that no copy
 * delivers): after probe_limit (1..4096) probes it gives up exactly as the step kernels would, so
 * mab_device_error() reads 1 afterwards.  Nothing faults and the context stays usable; it exists so that
 * the give-up path can be tested.  No counterpart in the reference. */
int mab_wait_selftest(int probe_limit, void* stream);

/* ---- device queries ------------------------------------------------------------------- */

/* Replaces ista_daslab_cuda_tools.get_sm_count() (micro_adam.py:40).  < 0 on failure. */
int mab_get_sm_count(void);

/* Replaces ista_daslab_cuda_tools.get_max_floats_for_shared_memory_per_thread_block()
 * (micro_adam.py:43): opt-in dynamic shared memory per block / 4.  58112 on a B200, which makes
 * d_block_size = 29056.  < 0 on failure. */
int mab_get_max_floats_for_shared_memory_per_thread_block(void);

/* ---- operator-for-operator replacements of the reference's native calls ------------------ */

/* x += alpha * Qinv(error).  Replaces ista_daslab_cuda_micro_adam.asymm_block_quant_inv
 * (micro_adam.py:190,267,298,313,322). */
int mab_asymm_block_quant_inv(int64_t d, int64_t quant_block_size, const uint8_t* error,
                              const uint16_t* min_vals, const uint16_t* max_vals,
                              void* x, int x_dtype, float alpha, void* stream);

/* error = Q(x; min_vals, max_vals), 4-bit codes, two per byte, even element in the high nibble.
 * Replaces ista_daslab_cuda_micro_adam.asymm_block_quant (micro_adam.py:231,316). */
int mab_asymm_block_quant(int64_t d, int64_t quant_block_size, uint8_t* error,
                          const uint16_t* min_vals, const uint16_t* max_vals,
                          const void* x, int x_dtype, void* stream);

/* d2k: out[j] = inp[(j / k_block_size) * d_block_size + indices[j]]  (out has k elements);
 * k2d: out[(j / k_block_size) * d_block_size + indices[j]] = inp[j]   (out has d elements).
 * Replaces ista_daslab_cuda_tools.copy_values (micro_adam.py:202-209;
 * sparse_mfac/sparse_core_mfac_w_ef.py:105-124). */
int mab_copy_values(int64_t d, int64_t k, int64_t d_block_size, int64_t k_block_size,
                    const int16_t* indices, const void* inp, int inp_dtype,
                    void* out, int out_dtype, int direction, void* stream);

/* x[(j / k_block_size) * d_block_size + indices[j]] = 0 for j < k.
 * Replaces ista_daslab_cuda_tools.zerorize_block_components (micro_adam.py:214). */
int mab_zerorize_block_components(void* x, int x_dtype, const int16_t* indices, int64_t d, int64_t k,
                                  int64_t d_block_size, int64_t k_block_size, void* stream);

/* out = Adam-style update from the sparse window (I, V), dense over d, 0 where no row touches.
 * Replaces ista_daslab_cuda_micro_adam.compute_microadam_update (micro_adam.py:277-291).
 * blocks / threads / carveout are accepted for signature compatibility and ignored. */
int mab_compute_microadam_update(int blocks, int threads, int carveout, int64_t steps,
                                 double beta1, double beta2, double eps,
                                 int64_t d_block_size, int64_t k_block_size, int64_t d, int64_t m, int64_t k,
                                 const int16_t* I, const uint16_t* V, void* out, int out_dtype, void* stream);

/* indices_row[k] = per block of d_block_size elements of x, the in-block positions of the
 * k_block_size_many (last short block: k_block_size_few) largest |x|, ties to the lower
 * position, ascending.  Replaces the two torch.topk calls at micro_adam.py:193-200. */
int mab_block_topk(int64_t d, int64_t d_block_size, int64_t k_block_size_many, int64_t k_block_size_few,
                   const void* x, int x_dtype, int16_t* indices_row, void* stream);

/* min_vals[b], max_vals[b] = bf16(min / max of x over quantisation block b), b = i / quant_block_size.
 * Replaces the torch min/max calls of _update_quantization_statistics (micro_adam.py:217-226). */
int mab_quant_stats(int64_t d, int64_t quant_block_size, uint16_t* min_vals, uint16_t* max_vals,
                    const void* x, int x_dtype, void* stream);

/* ---- other consumers of the (I, V) ring buffer ---------------------------------------------------- */

/* out[r] = sum_j V[r, j] * g[(j / k_block_size) * d_block_size + I[r, j]] for r < rows: the scalar products of a
 * dense vector with every sparse row.  I is int16 [rows, k], V is [rows, k] of v_dtype, out is float [rows].
 * Replaces ista_daslab_cuda_sparse_mfac.SP (sparse_mfac/sparse_core_mfac_w_ef.py:188-203); fp32 accumulation in
 * a fixed order. */
int mab_sparse_rows_dot(int64_t d, int64_t rows, int64_t k, int64_t d_block_size, int64_t k_block_size,
                        const void* g, int g_dtype, const int16_t* I, const void* V, int v_dtype, float* out,
                        void* stream);

/* out[(j / k_block_size) * d_block_size + I[r, j]] += M[r] * V[r, j] over r < rows, j < k: the linear combination of
 * the sparse rows with float coefficients M [rows], added to out [d] (the caller zeroes it first).
 * Replaces ista_daslab_cuda_sparse_mfac.LCG (sparse_mfac/sparse_core_mfac_w_ef.py:205-221); rows are accumulated in
 * fp32 in row order. */
int mab_sparse_rows_combine(int64_t d, int64_t rows, int64_t k, int64_t d_block_size, int64_t k_block_size,
                            const float* M, const int16_t* I, const void* V, int v_dtype, void* out, int out_dtype,
                            void* stream);

/* ---- fused step over a list of tensors ------------------------------------------------------ */

/* One parameter tensor of the step.  State buffers have the shapes micro_adam.py:86-94 gives them. */
typedef struct mab_tensor {
    void*     param;             /* [d], param_dtype; updated in place                         */
    const void* grad;            /* [d], grad_dtype; read only (the fused step leaves it as is) */
    uint8_t*  error;             /* [ceil(d/2)] 4-bit error feedback                            */
    uint16_t* min_vals;          /* [d / qbs + 1] bf16                                         */
    uint16_t* max_vals;          /* [d / qbs + 1] bf16                                         */
    int16_t*  I;                 /* [m, k] window indices                                      */
    uint16_t* V;                 /* [m, k] window values, bf16                                 */
    int64_t   d;
    int64_t   k;                 /* row length of I and V                                       */
    int32_t   d_block_size;      /* st['d_block_size']                                          */
    int32_t   topk_full_blocks_count;
    int32_t   k_block_size_many;
    int32_t   k_block_size_few;
    int32_t   param_dtype;
    int32_t   grad_dtype;
    int32_t   ring_index;        /* st['index']: row of I, V written this step                  */
    int32_t   row_pitch;         /* elements between consecutive rows of I and of V; 0 = k (rows of
                                    several tensors side by side in one buffer have a larger pitch) */
    double    lr;                /* group['lr'] of this step                                    */
    double    weight_decay;      /* group['weight_decay'] of this step                          */
    /* filled in by the library */
    float     decay_f32;         /* f32(1 - lr * weight_decay)                                  */
    float     neg_lr_f32;        /* f32(-lr)                                                    */
    int32_t   first_unit_a;      /* first work unit (top-k block) of this tensor in kernel A    */
    int32_t   first_unit_b;      /* first work unit (block sub-range) of this tensor in kernel B */
    /* alpha == -2 only (else NULL) */
    void*     quant_err;         /* [d], param_dtype: st['quant_err'] (micro_adam.py:67-68); kernel A leaves the
                                    residual a in it, kernel B turns it into a - Qinv(e)            */
} mab_tensor;

/* Slots of the probe buffer (doubles) a step adds to when mab_step_args.probe_out is given: the quantities the
 * reference logs every log_interval steps (micro_adam.py:155-156, 272-273, 306-308, 320-324). */
#define MAB_PROBE_NORM_G    0    /* sum of g^2 over the gradients of the call's tensors                */
#define MAB_PROBE_NORM_U    1    /* sum of u^2 over the updates                                          */
#define MAB_PROBE_NORM_E    2    /* sum of Qinv(e)^2 over the error feedback the step leaves            */
#define MAB_PROBE_ZEROS_U   3    /* number of exact zeros in u                                           */
#define MAB_PROBE_NORM_QE   4    /* alpha == -2: sum of quant_err^2                                      */
#define MAB_PROBE_ZEROS_QE  5    /* alpha == -2: number of exact zeros in quant_err                      */
#define MAB_PROBE_SLOTS     8

/* Scalars of one step, the same for every tensor. */
typedef struct mab_step_args {
    int64_t steps;               /* 1-based step counter (self.steps after the increment)        */
    int32_t m;                   /* window rows                                                   */
    int32_t quant_block_size;
    float   alpha;               /* 0 <= alpha < 1, or -2 (micro_adam.py:238-273)                 */
    int32_t reserved0;
    double  beta1, beta2, eps;
    double* probe_out;           /* NULL, or MAB_PROBE_SLOTS doubles in device memory that the call ADDS its
                                    probes to (the caller zeroes them): kernel B adds the update's, and one
                                    more small kernel at the end of the call the gradient's and the error
                                    feedback's.  mab_fused_ef_topk_quant alone adds the latter two (they
                                    describe the final state only when alpha is 0 or -2),
                                    mab_fused_window_adam_update alone the update's.               */
} mab_step_args;

/* Bytes of device workspace mab_fused_step needs for n_tensors tensors when quant_block_size is a power of two
 * in [8, 128]. */
int64_t mab_fused_step_workspace_bytes(int n_tensors);

/* Bytes of device workspace for these tensors and this quant_block_size, whatever it is: for a power of two in
 * [8, 128] the figure above, otherwise also 8 bytes per quantisation block of every tensor (scratch in which
 * the tiles of a block merge their minima and maxima) and 8 bytes per tensor. */
int64_t mab_fused_step_workspace_bytes_for(const mab_tensor* tensors, int n_tensors, const mab_step_args* args);

/* Whether the fused kernels cover this geometry (d_block_size <= 32768, supported dtypes, aligned pointers):
 *   1  quant_block_size is a power of two in [8, 128] that divides d_block_size; alpha in [0, 1), or alpha == -2
 *      with quant_err and equal gradient / parameter element types.  The gradient buffer is only read.
 *   2  any other quant_block_size that is a multiple of 8 in [64, 2^30] (the reference's README uses 100000),
 *      alpha == 0.  Quantisation blocks then ignore the borders of the top-k blocks (micro_adam.py:217-231), so
 *      kernel A runs in two parts: the first leaves the residual IN THE GRADIENT BUFFER (the reference overwrites
 *      it in the same step too) and each block's extremes in the workspace, the second writes statistics and
 *      codes.  The workspace size comes from mab_fused_step_workspace_bytes_for; mab_fused_step_static does
 *      not take this form.
 *   0  neither. */
int mab_fused_supported(const mab_tensor* t, const mab_step_args* args);

/* 1 if mab_fused_window_adam_update alone covers this tensor.  With alpha == 0 kernel B reads neither the error
 * feedback nor the gradient, so any quant_block_size qualifies and error / min_vals / max_vals / grad may be NULL:
 * a step whose first half ran on the operator-level calls (quantisation blocks that straddle top-k blocks) can
 * still take its second half fused.  Otherwise the same conditions as mab_fused_supported. */
int mab_fused_window_supported(const mab_tensor* t, const mab_step_args* args);

/* The whole step of micro_adam.py:146-328 for n_tensors tensors in two kernels:
 *   A  dequantise EF + add gradient, block top-k into row ring_index of I / V, zero the selected
 *      entries, block min / max, requantise EF                      (micro_adam.py:190-231)
 *   B  window -> Adam update, weight decay, alpha EF integration, parameter update, EF shrink
 *                                                                   (micro_adam.py:234-235, 276-316)
 * alpha == -2 (micro_adam.py:238-273; gradient and parameter of one element type, quant_err given): A also
 * writes the residual a to quant_err, and B applies p <- decay(p) - a + Qinv(e) before the update and leaves
 * a - Qinv(e) in quant_err.
 * `tensors` is host memory; it is copied to `workspace` (device, >= workspace_bytes) on `stream`
 * and its first_unit_* fields are overwritten.  Every tensor must satisfy mab_fused_supported. */
int mab_fused_step(mab_tensor* tensors, int n_tensors, const mab_step_args* args,
                   void* workspace, int64_t workspace_bytes, void* stream);

/* The two halves of mab_fused_step on their own (same arguments). */
int mab_fused_ef_topk_quant(mab_tensor* tensors, int n_tensors, const mab_step_args* args,
                            void* workspace, int64_t workspace_bytes, void* stream);
int mab_fused_window_adam_update(mab_tensor* tensors, int n_tensors, const mab_step_args* args,
                                 void* workspace, int64_t workspace_bytes, void* stream);

/* Most tensors one call of mab_fused_step_static accepts. */
#define MAB_STATIC_MAX_TENSORS 1024

/* mab_fused_step for callers that have no device buffer to offer as workspace.  (It has no
 * counterpart in the reference, whose native calls take one tensor at a time and need no table.)
 *
 * Who needs it: a trainer that gives all of HBM to one arena at start-up (a fixed memory plan, a
 * pooling allocator that has already claimed the device) has nothing left that cudaMalloc could
 * return, and a host that reaches this library through a foreign-function interface may be able to
 * pass only the buffers its own runtime tracks (parameters, gradients, optimizer state) and not
 * create a new one.  For them the table of tensor descriptors that the two kernels read lives in
 * a fixed array inside the library instead: MAB_STATIC_MAX_TENSORS * sizeof(mab_tensor) bytes
 * (144 KiB) of device memory per GPU, held by every GPU that loads the library until the process
 * exits.  The call allocates nothing, on the device or on the host.
 *
 * Same arguments, results and errors as mab_fused_step, minus the workspace, with these differences:
 *  - n_tensors > MAB_STATIC_MAX_TENSORS fails with MAB_ERR_LIMIT (split the step into several calls);
 *  - tensors are processed in the order given; consecutive tensors with the same (grad, param) element
 *    types share a kernel launch, so keep equal types together;
 *  - the first call on a device looks up the array's device address (once per device, with that device
 *    current); make that first call outside any stream capture;
 *  - `tensors` is copied to the device asynchronously on `stream`; if it lives in page-locked host memory,
 *    leave it unchanged until the stream has passed this call (pageable memory is staged before the
 *    call returns);
 *  - all calls on a device share the one array.  Calls on the same stream are ordered and safe; two
 *    calls whose kernels can overlap on the GPU (different streams without an event between them)
 *    race on it.  Nothing in the array has to start at zero: each call overwrites what it uses. */
int mab_fused_step_static(mab_tensor* tensors, int n_tensors, const mab_step_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MICROADAM_B200_H */
