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
