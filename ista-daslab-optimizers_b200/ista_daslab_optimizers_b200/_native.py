"""ctypes binding of libmicroadam_b200.so (declared in include/microadam_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
Torch is used only to obtain device pointers and the current CUDA stream.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_void_p

import torch

LIB_NAME = 'libmicroadam_b200.so'
LIB_PATH = os.environ.get('MICROADAM_B200_LIB') or os.path.join(os.path.dirname(os.path.abspath(__file__)), 'lib', LIB_NAME)

MAB_OK = 0
MAB_F32, MAB_BF16 = 0, 1
MAB_K2D, MAB_D2K = 0, 1
MAB_MAX_WINDOW = 128
MAB_STATIC_MAX_TENSORS = 1024
MAB_PROBE_NORM_G, MAB_PROBE_NORM_U, MAB_PROBE_NORM_E, MAB_PROBE_ZEROS_U, MAB_PROBE_NORM_QE, MAB_PROBE_ZEROS_QE = range(6)
MAB_PROBE_SLOTS = 8

_DTYPE_CODE = {torch.float32: MAB_F32, torch.bfloat16: MAB_BF16}


class NativeError(RuntimeError):
    """A call into libmicroadam_b200.so returned a failure status."""


class MabTensor(Structure):
    """struct mab_tensor."""
    _fields_ = [
        ('param', c_void_p), ('grad', c_void_p), ('error', c_void_p), ('min_vals', c_void_p),
        ('max_vals', c_void_p), ('I', c_void_p), ('V', c_void_p),
        ('d', c_int64), ('k', c_int64),
        ('d_block_size', c_int32), ('topk_full_blocks_count', c_int32),
        ('k_block_size_many', c_int32), ('k_block_size_few', c_int32),
        ('param_dtype', c_int32), ('grad_dtype', c_int32),
        ('ring_index', c_int32), ('row_pitch', c_int32),
        ('lr', c_double), ('weight_decay', c_double),
        ('decay_f32', c_float), ('neg_lr_f32', c_float),
        ('first_unit_a', c_int32), ('first_unit_b', c_int32),
        ('quant_err', c_void_p),
    ]


class MabStepArgs(Structure):
    """struct mab_step_args."""
    _fields_ = [
        ('steps', c_int64), ('m', c_int32), ('quant_block_size', c_int32),
        ('alpha', c_float), ('reserved0', c_int32),
        ('beta1', c_double), ('beta2', c_double), ('eps', c_double),
        ('probe_out', c_void_p),
    ]


# name -> (restype, argtypes); every symbol include/microadam_b200.h declares
SIGNATURES = {
    'mab_last_error': (c_char_p, []),
    'mab_kernel_launch_count': (c_int64, []),
    'mab_device_error': (c_int, []),
    'mab_device_error_clear': (c_int, []),
    'mab_wait_selftest': (c_int, [c_int, c_void_p]),
    'mab_get_sm_count': (c_int, []),
    'mab_get_max_floats_for_shared_memory_per_thread_block': (c_int, []),
    'mab_asymm_block_quant_inv': (c_int, [c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p]),
    'mab_asymm_block_quant': (c_int, [c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    'mab_copy_values': (c_int, [c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]),
    'mab_zerorize_block_components': (c_int, [c_void_p, c_int, c_void_p, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    'mab_compute_microadam_update': (c_int, [c_int, c_int, c_int, c_int64, c_double, c_double, c_double, c_int64, c_int64,
                                             c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    'mab_block_topk': (c_int, [c_int64, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p]),
    'mab_quant_stats': (c_int, [c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    'mab_sparse_rows_dot': (c_int, [c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    'mab_sparse_rows_combine': (c_int, [c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    'mab_fused_step_workspace_bytes': (c_int64, [c_int]),
    'mab_fused_step_workspace_bytes_for': (c_int64, [POINTER(MabTensor), c_int, POINTER(MabStepArgs)]),
    'mab_fused_supported': (c_int, [POINTER(MabTensor), POINTER(MabStepArgs)]),
    'mab_fused_window_supported': (c_int, [POINTER(MabTensor), POINTER(MabStepArgs)]),
    'mab_fused_step': (c_int, [POINTER(MabTensor), c_int, POINTER(MabStepArgs), c_void_p, c_int64, c_void_p]),
    'mab_fused_ef_topk_quant': (c_int, [POINTER(MabTensor), c_int, POINTER(MabStepArgs), c_void_p, c_int64, c_void_p]),
    'mab_fused_window_adam_update': (c_int, [POINTER(MabTensor), c_int, POINTER(MabStepArgs), c_void_p, c_int64, c_void_p]),
    'mab_fused_step_static': (c_int, [POINTER(MabTensor), c_int, POINTER(MabStepArgs), c_void_p]),
}

_lib = None


def load(path: str = LIB_PATH) -> ctypes.CDLL:
    """Loads the library once and attaches the prototypes.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(path):
            raise NativeError(
                f'{path} is missing: build it with `python ista-daslab-optimizers_b200/build.py` '
                '(needs nvcc); this package has no CPU or PyTorch fallback')
        lib = ctypes.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != MAB_OK:
        msg = load().mab_last_error().decode('utf-8', 'replace')
        raise NativeError(f'{what} failed with status {status}: {msg}')


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise NativeError(f'unsupported element type {t.dtype}: the kernels take float32 and bfloat16') from None


def dev_ptr(t: torch.Tensor, what: str) -> int:
    if not t.is_cuda:
        raise NativeError(f'{what} must be a CUDA tensor (got {t.device}); there is no CPU implementation')
    if not t.is_contiguous():
        raise NativeError(f'{what} must be contiguous')
    return t.data_ptr()


def current_stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# ------------------------------------------------------------------------------------------------
# Operator-level calls with the argument order of the reference's native modules
# (micro_adam.py:40,43,190,202-209,214,231,277-291), on torch CUDA tensors.

def kernel_launch_count() -> int:
    return load().mab_kernel_launch_count()


def device_error() -> int:
    """1 if a kernel ever gave up waiting for the copy engine on the current device (synchronises)."""
    v = load().mab_device_error()
    if v < 0:
        check(v, 'device_error')
    return v


def device_error_clear() -> None:
    check(load().mab_device_error_clear(), 'device_error_clear')


def get_sm_count() -> int:
    v = load().mab_get_sm_count()
    if v < 0:
        check(v, 'get_sm_count')
    return v


def get_max_floats_for_shared_memory_per_thread_block() -> int:
    v = load().mab_get_max_floats_for_shared_memory_per_thread_block()
    if v < 0:
        check(v, 'get_max_floats_for_shared_memory_per_thread_block')
    return v


def _run(anchor: torch.Tensor, what: str, fn, *args):
    """Calls fn(*args, stream) with anchor's device current.  Pointer arguments are resolved (and
    checked) by the caller before this point, so a CPU tensor is rejected before any CUDA call."""
    with torch.cuda.device(anchor.device):
        check(fn(*args, current_stream(anchor.device)), what)


def asymm_block_quant_inv(d, quant_block_size, error, min_vals, max_vals, x, alpha):
    _run(x, 'asymm_block_quant_inv', load().mab_asymm_block_quant_inv, d, quant_block_size, dev_ptr(error, 'error'),
         dev_ptr(min_vals, 'min_vals'), dev_ptr(max_vals, 'max_vals'), dev_ptr(x, 'x'), dtype_code(x), float(alpha))


def asymm_block_quant(d, quant_block_size, error, min_vals, max_vals, x):
    _run(x, 'asymm_block_quant', load().mab_asymm_block_quant, d, quant_block_size, dev_ptr(error, 'error'),
         dev_ptr(min_vals, 'min_vals'), dev_ptr(max_vals, 'max_vals'), dev_ptr(x, 'x'), dtype_code(x))


def copy_values(d, k, d_block_size, k_block_size, indices, inp, out, direction):
    _run(inp, 'copy_values', load().mab_copy_values, d, k, d_block_size, k_block_size, dev_ptr(indices, 'indices'),
         dev_ptr(inp, 'inp'), dtype_code(inp), dev_ptr(out, 'out'), dtype_code(out), int(direction))


def zerorize_block_components(x, indices, d, k, d_block_size, k_block_size):
    _run(x, 'zerorize_block_components', load().mab_zerorize_block_components, dev_ptr(x, 'x'), dtype_code(x),
         dev_ptr(indices, 'indices'), d, k, d_block_size, k_block_size)


def compute_microadam_update(blocks, threads, carveout, steps, beta1, beta2, eps, d_block_size, k_block_size, d, m, k,
                             I, V, out):
    _run(out, 'compute_microadam_update', load().mab_compute_microadam_update, int(blocks), int(threads), int(carveout),
         steps, beta1, beta2, eps, d_block_size, k_block_size, d, m, k, dev_ptr(I, 'I'), dev_ptr(V, 'V'),
         dev_ptr(out, 'out'), dtype_code(out))


def block_topk(d, d_block_size, k_block_size_many, k_block_size_few, x, indices_row):
    _run(x, 'block_topk', load().mab_block_topk, d, d_block_size, k_block_size_many, k_block_size_few, dev_ptr(x, 'x'),
         dtype_code(x), dev_ptr(indices_row, 'indices_row'))


def quant_stats(d, quant_block_size, min_vals, max_vals, x):
    _run(x, 'quant_stats', load().mab_quant_stats, d, quant_block_size, dev_ptr(min_vals, 'min_vals'),
         dev_ptr(max_vals, 'max_vals'), dev_ptr(x, 'x'), dtype_code(x))


def sparse_rows_dot(d, rows, k, d_block_size, k_block_size, g, I, V, out):
    """out[r] = <row r of the sparse buffer, g> (ista_daslab_cuda_sparse_mfac.SP, sparse_core_mfac_w_ef.py:188-203)."""
    if out.dtype != torch.float32:
        raise NativeError('sparse_rows_dot writes float32 scalar products')
    _run(g, 'sparse_rows_dot', load().mab_sparse_rows_dot, d, rows, k, d_block_size, k_block_size, dev_ptr(g, 'g'), dtype_code(g),
         dev_ptr(I, 'I'), dev_ptr(V, 'V'), dtype_code(V), dev_ptr(out, 'out'))


def sparse_rows_combine(d, rows, k, d_block_size, k_block_size, M, I, V, out):
    """out += sum_r M[r] * row r of the sparse buffer (ista_daslab_cuda_sparse_mfac.LCG, sparse_core_mfac_w_ef.py:205-221)."""
    if M.dtype != torch.float32:
        raise NativeError('sparse_rows_combine takes float32 coefficients')
    _run(out, 'sparse_rows_combine', load().mab_sparse_rows_combine, d, rows, k, d_block_size, k_block_size, dev_ptr(M, 'M'),
         dev_ptr(I, 'I'), dev_ptr(V, 'V'), dtype_code(V), dev_ptr(out, 'out'), dtype_code(out))
