"""The C ABI without a GPU: the header is valid C, the library loads and exports every declared
symbol, the ctypes mirror has the C layout, and calls fail loudly instead of falling back."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'microadam_b200.h')


@pytest.fixture(scope='module')
def native():
    sys.path.insert(0, os.path.join(ROOT, 'ista-daslab-optimizers_b200'))
    import build
    build.build()
    from ista_daslab_optimizers_b200 import _native
    return _native


def declared_symbols():
    text = re.sub(r'/\*.*?\*/', '', open(HEADER).read(), flags=re.S)
    return sorted(set(re.findall(r'\b(mab_[a-z0-9_]+)\s*\(', text)))


def test_every_declared_symbol_is_exported_and_bound(native):
    lib = native.load()
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(native.SIGNATURES) == names


def test_header_is_plain_c_and_layout_matches_ctypes(native, tmp_path):
    src = tmp_path / 'sizes.c'
    src.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "microadam_b200.h"\n'
                   'int main(void){printf("%zu %zu %zu %zu %zu\\n", sizeof(mab_tensor), sizeof(mab_step_args),'
                   ' offsetof(mab_tensor, lr), offsetof(mab_tensor, first_unit_b), offsetof(mab_step_args, beta1));return 0;}\n')
    exe = tmp_path / 'sizes'
    subprocess.run(['gcc', '-std=c99', '-Wall', '-Werror', '-I', os.path.dirname(HEADER), str(src), '-o', str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    assert got == [ctypes.sizeof(native.MabTensor), ctypes.sizeof(native.MabStepArgs), native.MabTensor.lr.offset,
                   native.MabTensor.first_unit_b.offset, native.MabStepArgs.beta1.offset]


@pytest.mark.skipif(torch.cuda.is_available(), reason='checks the behaviour without a device')
def test_no_cpu_fallback(native):
    with pytest.raises(native.NativeError):
        native.get_sm_count()
    x = torch.zeros(64)
    with pytest.raises(native.NativeError, match='no CPU implementation'):
        native.quant_stats(64, 64, torch.zeros(2, dtype=torch.bfloat16), torch.zeros(2, dtype=torch.bfloat16), x)
    from ista_daslab_optimizers_b200 import MicroAdam
    with pytest.raises(native.NativeError):
        MicroAdam([torch.nn.Parameter(torch.zeros(8))], m=10, lr=1e-3, quant_block_size=64)


def test_bad_arguments_are_rejected_before_any_launch(native):
    lib = native.load()
    assert lib.mab_asymm_block_quant_inv(10, 0, None, None, None, None, 0, 1.0, None) == -1
    assert b'qbs' in lib.mab_last_error()
    assert lib.mab_block_topk(100, 40000, 400, 0, 1, 0, 1, None) == -4      # d_block_size beyond 32768
    assert lib.mab_copy_values(10, 5, 10, 5, 1, 1, 0, 1, 0, 7, None) == -1   # bad direction
    assert lib.mab_fused_step(None, 3, None, None, 0, None) == -1
    assert lib.mab_fused_step_workspace_bytes(10) == 10 * ctypes.sizeof(native.MabTensor)
    t, a = native.MabTensor(), native.MabStepArgs()
    assert lib.mab_fused_supported(ctypes.byref(t), ctypes.byref(a)) == 0


def _geometry(t, d, dbs=29056, k_init=0.01):
    import math
    t.d, t.d_block_size = d, min(d, dbs)
    nfull, rest = divmod(d, t.d_block_size)
    t.topk_full_blocks_count = nfull
    t.k_block_size_many = math.ceil(t.d_block_size * k_init)
    t.k_block_size_few = math.ceil(rest * k_init) if rest else 0
    t.k = nfull * t.k_block_size_many + t.k_block_size_few


def test_which_quantisation_block_sizes_take_which_fused_form(native):
    """Host-side answers only (no launch): 1 = blocks that tile the top-k blocks, 2 = any other multiple of 8 from 64 up
    with alpha == 0 (kernel A in two parts, more workspace), 0 = operator-level calls; and whether the update kernel
    alone can follow an operator-level first half."""
    lib = native.load()
    t, a = native.MabTensor(), native.MabStepArgs()
    _geometry(t, 3 * 29056 + 100)
    for name in ('param', 'grad', 'error', 'min_vals', 'max_vals', 'I', 'V'):
        setattr(t, name, 4096)                       # any aligned non-null address: nothing is dereferenced here
    t.param_dtype = t.grad_dtype = native.MAB_F32
    a.steps, a.m, a.alpha = 1, 10, 0.0
    answers = {}
    for qbs in (64, 128, 32, 100000, 1000, 72, 100, 48, 256):
        a.quant_block_size = qbs
        answers[qbs] = (lib.mab_fused_supported(ctypes.byref(t), ctypes.byref(a)),
                        lib.mab_fused_window_supported(ctypes.byref(t), ctypes.byref(a)))
    assert answers == {64: (1, 1), 128: (1, 1), 32: (1, 1), 100000: (2, 1), 1000: (2, 1), 72: (2, 1), 256: (2, 1),
                       100: (0, 1), 48: (0, 1)}
    a.quant_block_size, a.alpha = 100000, 0.5        # the alpha term needs the operator-level path with loose blocks
    assert lib.mab_fused_supported(ctypes.byref(t), ctypes.byref(a)) == 0
    assert lib.mab_fused_window_supported(ctypes.byref(t), ctypes.byref(a)) == 0
    # workspace: the descriptor table alone for aligned blocks; plus 8 bytes per tensor and per quantisation block otherwise
    ts = (native.MabTensor * 2)()
    _geometry(ts[0], 250001)
    _geometry(ts[1], 4096)
    a.alpha = 0.0
    a.quant_block_size = 64
    table = lib.mab_fused_step_workspace_bytes(2)
    assert lib.mab_fused_step_workspace_bytes_for(ts, 2, ctypes.byref(a)) == table
    a.quant_block_size = 100000
    need = lib.mab_fused_step_workspace_bytes_for(ts, 2, ctypes.byref(a))
    blocks = 3 + 1                                   # ceil(250001 / 100000) + ceil(4096 / 100000)
    assert table + 2 * 8 + blocks * 8 <= need <= table + 4 * 256 + 2 * 8 + blocks * 8
    assert lib.mab_fused_step_static(ts, 2, ctypes.byref(a), None) < 0       # that entry point has no scratch memory
    assert b'quant_block_size' in lib.mab_last_error()
